// peer_select_noalloc: product-key selection for callers that must not allocate.
//
// Some embedders of this library cannot call cudaMalloc once they are up: an inference server
// that hands the whole GPU to its own memory pool at start-up has nothing left for the driver
// to give, and a latency-critical decode loop cannot afford the device-wide synchronisation
// (or the failure path) that an allocation brings.  peer_create allocates its scratch, so
// those callers get this one entry point instead: it needs no handle, and the scratch the
// selection kernels use (the normalised sub-keys, the normalised queries and the candidate
// pair table) lives in a fixed array that is part of the library image.
//
// Consequences the caller has to know:
//  * every GPU that loads the library carries the array (PEER_NOALLOC_SCRATCH_BYTES) until the
//    process exits, used or not;
//  * the problem has to fit: a call whose scratch would exceed the array is refused with
//    PEER_ERR_UNSUPPORTED and a message that states both sizes;
//  * all calls on a device share the array.  Nothing in it has to start at zero (each call
//    overwrites what it reads), but two calls whose kernels overlap on the GPU (different
//    streams, no dependency) race on it and produce garbage: serialise them;
//  * the first call on each device looks up the array's device address and raises the
//    shared-memory limit of the selection kernel (under a lock, so two host threads may make
//    it at once); make that first call during start-up, outside any stream capture.  Every
//    later call only enqueues kernels on the caller's stream: nothing is copied from host
//    memory (the candidate-pair table is written by a kernel), and nothing synchronises.
#include <cmath>
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

#define PEER_NOALLOC_SCRATCH_BYTES (8u << 20)

// The array itself.  On the host this name is only a handle for cudaGetSymbolAddress; it is
// never passed to a kernel as if it were a pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PEER_NOALLOC_SCRATCH_BYTES];

namespace peer { void set_global_error(const char* msg); int candidates_per_dim_2d(int top_k, int dim_size); }

namespace {
constexpr int MAX_DEVICES = 64;
unsigned char* g_scratch_ptr[MAX_DEVICES] = {};   // device address of the array, per device (guarded by g_setup_lock)
std::mutex g_setup_lock;

// Candidate pairs (a, b) with (a+1)(b+1) <= k, a-major: the only ones that can reach the final top k
// because both per-half lists are sorted.  Written on the device so that a call never reads host memory.
__global__ void noalloc_pairs_kernel(uint16_t* pairs, int kp0, int kp1, int k, int cap) {
    if (threadIdx.x || blockIdx.x) return;
    int n = 0;
    for (int a = 0; a < kp0; ++a)
        for (int b = 0; b < kp1; ++b)
            if ((a + 1) * (b + 1) <= k && n < cap) pairs[n++] = static_cast<uint16_t>((a << 8) | b);
}

int refuse(int code, const char* fmt, long long a = 0, long long b = 0, long long c = 0) {
    char buf[384];
    snprintf(buf, sizeof buf, fmt, a, b, c);
    peer::set_global_error(buf);
    return code;
}
size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }
}  // namespace

extern "C" int peer_select_noalloc(const peer_config_t* c, const float* queries, const void* keys0,
                                   const void* keys1, int64_t n_tokens, int64_t* ids_out, float* scores_out,
                                   void* stream) {
    using namespace peer;
    if (!c || !queries || !keys0 || !keys1 || !ids_out || !scores_out)
        return refuse(PEER_ERR_INVALID_ARG, "peer_select_noalloc: null argument");
    if (c->abi_version != PEER_B200_ABI_VERSION) return refuse(PEER_ERR_INVALID_ARG, "peer_select_noalloc: abi_version mismatch");
    if (n_tokens < 0) return refuse(PEER_ERR_INVALID_ARG, "peer_select_noalloc: negative token count");
    if (n_tokens == 0) return PEER_OK;
    if (c->act_dtype != PEER_DTYPE_F32 && c->act_dtype != PEER_DTYPE_BF16)
        return refuse(PEER_ERR_UNSUPPORTED, "peer_select_noalloc: sub-keys must be fp32 or bf16");
    if (c->index_mode != PEER_INDEX_REFERENCE && c->index_mode != PEER_INDEX_PRODUCT)
        return refuse(PEER_ERR_INVALID_ARG, "peer_select_noalloc: index_mode %lld", c->index_mode);
    if (c->query_dim <= 0 || c->query_dim % 2 || c->query_dim > 256 || c->num_heads <= 0 || c->n_keys0 <= 0 ||
        c->n_keys1 <= 0 || c->top_k <= 0 || c->top_k > 32)
        return refuse(PEER_ERR_UNSUPPORTED, "peer_select_noalloc: query_dim even and <= 256, top_k <= 32, positive sizes");
    const int kp0 = candidates_per_dim_2d(c->top_k, c->n_keys0), kp1 = candidates_per_dim_2d(c->top_k, c->n_keys1);
    if (kp0 > 32 || kp1 > 32 || static_cast<int64_t>(kp0) * kp1 < c->top_k)
        return refuse(PEER_ERR_UNSUPPORTED, "peer_select_noalloc: top_k=%lld does not fit a %lld x %lld key grid", c->top_k,
                      c->n_keys0, c->n_keys1);

    // ---- carve the fixed array; refuse what does not fit
    const int hw = c->query_dim / 2;
    const size_t k0_bytes = align256(sizeof(float) * hw * c->n_keys0);
    const size_t k1_bytes = align256(sizeof(float) * hw * c->n_keys1);
    const size_t q_bytes = align256(sizeof(float) * static_cast<size_t>(n_tokens) * c->num_heads * c->query_dim);
    const size_t pair_bytes = align256(sizeof(uint16_t) * MAX_PAIRS);
    const size_t need = k0_bytes + k1_bytes + q_bytes + pair_bytes;
    if (need > PEER_NOALLOC_SCRATCH_BYTES)
        return refuse(PEER_ERR_UNSUPPORTED,
                      "peer_select_noalloc: %lld tokens need %lld bytes of scratch, the built-in array holds %lld; "
                      "use fewer tokens per call or the handle-based peer_select",
                      n_tokens, static_cast<long long>(need), static_cast<long long>(PEER_NOALLOC_SCRATCH_BYTES));

    // ---- once per device, with that device current: the array's device address
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
        return refuse(PEER_ERR_CUDA, "peer_select_noalloc: cudaGetDevice failed or device index out of range");
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> guard(g_setup_lock);
        if (!g_scratch_ptr[dev]) {
            unsigned char* ptr = nullptr;
            e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
            if (e != cudaSuccess || !ptr) {
                peer::set_global_error(cudaGetErrorString(e));
                return PEER_ERR_CUDA;
            }
            e = select_simt_setup();
            if (e != cudaSuccess) { peer::set_global_error(cudaGetErrorString(e)); return PEER_ERR_CUDA; }
            g_scratch_ptr[dev] = ptr;
        }
        base = g_scratch_ptr[dev];
    }
    float* khat0 = reinterpret_cast<float*>(base);
    float* khat1 = reinterpret_cast<float*>(base + k0_bytes);
    float* q_hat = reinterpret_cast<float*>(base + k0_bytes + k1_bytes);
    uint16_t* pairs_dev = reinterpret_cast<uint16_t*>(base + k0_bytes + k1_bytes + q_bytes);

    // how many candidate pairs the device-side enumeration will write
    int n_pairs = 0;
    for (int a = 0; a < kp0; ++a)
        for (int b = 0; b < kp1; ++b)
            if ((a + 1) * (b + 1) <= c->top_k) ++n_pairs;
    if (n_pairs > MAX_PAIRS) return refuse(PEER_ERR_UNSUPPORTED, "peer_select_noalloc: too many candidate pairs");

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    noalloc_pairs_kernel<<<1, 32, 0, s>>>(pairs_dev, kp0, kp1, c->top_k, MAX_PAIRS);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = launch_normalize_rows(keys0, c->act_dtype, c->n_keys0, hw, c->norm_keys, 1, khat0, s);
    if (e == cudaSuccess) e = launch_normalize_rows(keys1, c->act_dtype, c->n_keys1, hw, c->norm_keys, 1, khat1, s);
    if (e == cudaSuccess) e = launch_normalize_halves(queries, n_tokens * c->num_heads, c->query_dim, c->norm_query, q_hat, s);
    if (e == cudaSuccess) {
        SelectArgs a{};
        a.q_hat = q_hat; a.khat0 = khat0; a.khat1 = khat1; a.rows = n_tokens * c->num_heads; a.Q = c->query_dim;
        a.n0 = c->n_keys0; a.n1 = c->n_keys1; a.kp0 = kp0; a.kp1 = kp1; a.k = c->top_k;
        a.mult0 = c->index_mode == PEER_INDEX_PRODUCT ? c->n_keys1 : 1; a.mult1 = 1;
        a.pairs = pairs_dev; a.n_pairs = n_pairs; a.ids64 = ids_out; a.raw_scores = scores_out;
        e = launch_select_simt(a, s);
    }
    if (e != cudaSuccess) { peer::set_global_error(cudaGetErrorString(e)); return PEER_ERR_CUDA; }
    return PEER_OK;
}
