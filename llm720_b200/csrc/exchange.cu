// Direct exchange for the expert-parallel layer (tables split by rows over the GPUs of one node): the three
// exchange steps of a decode-shaped batch - every rank needs every token's activations, every tuple
// (token, expert, weight) has to reach the rank that owns the expert's rows, every partial sum has to come back
// to the token's rank - done by plain stores into the peers' memory over NVLink instead of three collectives.
//
// The reference has no sharded PEER (expert sharding is announced in docs/paper/paper.tex:446 and listed as
// future work in docs/CUTLASS_KERNEL.md:181); what has to be exchanged follows from its forward
// (llm/models/experts.py:332-382).  The wire format is the one of route.cu.
//
// Every rank owns one region (cudaMalloc, exported with CUDA IPC and mapped by its peers):
//     x_all   [2][world * T, d_in]         activations of all tokens, written by their owners
//     recv    [2][world][2 * T * E + T]    tuple blocks, block r written by rank r
//     part_in [2][world][T, d_out] fp32    partial sums of my tokens, slot r written by rank r
//     flags   [3][world] int32             step numbers: "rank r's x / tuples / partial sums of step s are here"
// (T tokens per rank, E = heads * top_k).  The data buffers exist twice and a step uses the copy of its parity:
// a rank can be at most one step ahead of a peer (it cannot finish step s without that peer's step-s partial
// sums, which the peer sends after it has read what it received for step s - 1), so what a peer writes for step
// s + 1 never lands in a buffer that step s still reads.
//
// Ordering.  A writer stores its data, fences at system scope, and only then stores the step number; a reader
// polls the step numbers with acquire loads at system scope before the kernels that read the data start.
// Only plain loads and stores touch a peer's memory: no bulk or tensor copies, no multicast.
// Every wait is bounded in time (WAIT_NS): when it runs out the kernel records STATUS_TIMEOUT and returns, so a
// peer that died or fell behind shows as an error code, not as a hang.
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace peer {
void set_global_error(const char* msg);
}

namespace {

using namespace peer;

constexpr unsigned long long WAIT_NS = 2000000000ULL;      // two seconds
constexpr int MAX_WORLD = 16;

struct Region {            // byte offsets inside a rank's region (the same on every rank)
    size_t x_all[2], recv[2], part_in[2], flags, total;
};

struct PeerPtrs {          // the region of every rank, as mapped here (own rank: the allocation itself)
    char* base[MAX_WORLD];
};

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Blocks (d, 0 .. gridDim.y) copy `bytes` (a multiple of 16) from src + d * src_stride to rank d's region at
// dst_off; the last of them to finish announces `step` in rank d's flag.  Several blocks per destination: one
// SM alone keeps too few stores in flight over NVLink (a single block moved 256 KB in 20 us).
constexpr int PUSH_BLOCKS = 16;
__global__ void __launch_bounds__(512)
push_kernel(const char* __restrict__ src, int64_t src_stride, PeerPtrs peers, size_t dst_off, int64_t bytes,
            size_t flag_off, int step, unsigned* blocks_done) {
    const int d = blockIdx.x;
    const uint4* s = reinterpret_cast<const uint4*>(src + d * src_stride);
    uint4* t = reinterpret_cast<uint4*>(peers.base[d] + dst_off);
    const int64_t n = bytes / 16;
    for (int64_t i = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.y) * blockDim.x)
        t[i] = s[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned done = atomicAdd(blocks_done + d, 1u);
        if (done == gridDim.y - 1) {                          // every block's stores for rank d are fenced by now
            blocks_done[d] = 0;
            __threadfence_system();
            st_release_sys(reinterpret_cast<int*>(peers.base[d] + flag_off), step);
        }
    }
}

// Waits until flags[row][0..world) >= step for the one or two flag rows given (row_b < 0: one); one thread per flag.
__global__ void wait_kernel(const int* __restrict__ flags, int row_a, int row_b, int world, int step, int* status) {
    const int i = threadIdx.x;
    const int n = (row_b >= 0 ? 2 : 1) * world;
    if (i >= n) return;
    const int* f = flags + (i < world ? row_a : row_b) * MAX_WORLD + (i % world);
    const unsigned long long t0 = now_ns();
    while (ld_acquire_sys(f) < step) {
        if (now_ns() - t0 > WAIT_NS) { atomicMax(status, STATUS_TIMEOUT); return; }
        __nanosleep(200);
    }
}

// out[i][c] = sum over ranks r (in rank order) of part_in[r][i][c]; waits for the ranks' step numbers first.
template <typename T>
__global__ void __launch_bounds__(256)
sum_cast_kernel(const float* part_in, const int* flags, int world, int64_t n, int step,
                T* __restrict__ out, int* status) {
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if (threadIdx.x < world) {
        const unsigned long long t0 = now_ns();
        while (ld_acquire_sys(flags + threadIdx.x) < step) {
            if (now_ns() - t0 > WAIT_NS) { atomicMax(status, STATUS_TIMEOUT); ok = 0; break; }
            __nanosleep(200);
        }
    }
    __syncthreads();
    if (!ok) return;
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(part_in + r * n + i));   // written by a peer while this
                                                                                         // kernel waited: read past L1
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    out[i] = from_f32<T>(s.x); out[i + 1] = from_f32<T>(s.y); out[i + 2] = from_f32<T>(s.z); out[i + 3] = from_f32<T>(s.w);
}

size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

}  // namespace

struct peer_xchg {
    int world = 0, rank = 0, device = 0, act_dtype = 0, entries = 0, d_in = 0, d_out = 0;
    int64_t t_local = 0;
    int step = 0;                       // number of the step in progress (1, 2, ...); parity picks the buffers
    Region lay{};
    PeerPtrs map{};
    bool attached = false;
    unsigned* blocks_done = nullptr;    // device counters of the push kernel, one per destination ([1]: for the activations)
    int32_t* send = nullptr;            // [world] tuple blocks as routed here, before they go to their owners
    int* status = nullptr;              // device status word
    cudaStream_t side = nullptr;        // peer_xchg_forward sends the activations beside the selection
    cudaEvent_t fork = nullptr;
    std::string error;
};

namespace {

int xfail(peer_xchg* h, int code, const std::string& msg) {
    if (h) h->error = msg;
    peer::set_global_error(msg.c_str());
    return code;
}
#define XCU(h, call)                                                                   \
    do {                                                                               \
        const cudaError_t e_ = (call);                                                 \
        if (e_ != cudaSuccess) return xfail(h, PEER_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); \
    } while (0)

int act_size(int dt) { return dt == PEER_DTYPE_F32 ? 4 : 2; }

}  // namespace

extern "C" int peer_xchg_create(int32_t world, int32_t rank, int64_t tokens_per_rank, int32_t entries_per_token,
                                int32_t input_dim, int32_t output_dim, int32_t act_dtype, peer_xchg_t* out) {
    if (!out) return xfail(nullptr, PEER_ERR_INVALID_ARG, "peer_xchg_create: out is null");
    *out = nullptr;
    if (world < 1 || world > MAX_WORLD || rank < 0 || rank >= world || tokens_per_rank < 1 || entries_per_token < 1 ||
        input_dim < 1 || output_dim < 1)
        return xfail(nullptr, PEER_ERR_INVALID_ARG, "peer_xchg_create: world in [1, 16], rank in [0, world), positive sizes");
    if (act_dtype != PEER_DTYPE_BF16 && act_dtype != PEER_DTYPE_F16 && act_dtype != PEER_DTYPE_F32)
        return xfail(nullptr, PEER_ERR_INVALID_ARG, "peer_xchg_create: unknown activation dtype");
    if ((static_cast<int64_t>(input_dim) * act_size(act_dtype)) % 16 || output_dim % 4)
        return xfail(nullptr, PEER_ERR_UNSUPPORTED, "peer_xchg_create: rows must be whole 16-byte chunks");
    if ((tokens_per_rank * (2 * static_cast<int64_t>(entries_per_token) + 1)) % 4)
        return xfail(nullptr, PEER_ERR_UNSUPPORTED, "peer_xchg_create: a tuple block (tokens_per_rank * (2 * entries + 1) words) must be whole 16-byte chunks");
    peer_xchg* h = new peer_xchg();
    h->world = world; h->rank = rank; h->t_local = tokens_per_rank; h->entries = entries_per_token;
    h->d_in = input_dim; h->d_out = output_dim; h->act_dtype = act_dtype;
    cudaGetDevice(&h->device);
    const size_t x_bytes = static_cast<size_t>(world) * tokens_per_rank * input_dim * act_size(act_dtype);
    const size_t blk_bytes = (2 * static_cast<size_t>(tokens_per_rank) * entries_per_token + tokens_per_rank) * 4;
    const size_t part_bytes = static_cast<size_t>(world) * tokens_per_rank * output_dim * 4;
    size_t off = 0;
    for (int p = 0; p < 2; ++p) { h->lay.x_all[p] = off; off = up256(off + x_bytes); }
    for (int p = 0; p < 2; ++p) { h->lay.recv[p] = off; off = up256(off + world * blk_bytes); }
    for (int p = 0; p < 2; ++p) { h->lay.part_in[p] = off; off = up256(off + part_bytes); }
    h->lay.flags = off; off = up256(off + 3 * MAX_WORLD * 4);
    h->lay.total = off;
    void* base = nullptr;
    cudaError_t e = cudaMalloc(&base, h->lay.total);
    if (e == cudaSuccess) e = cudaMemset(base, 0, h->lay.total);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&h->blocks_done), 2 * MAX_WORLD * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(h->blocks_done, 0, 2 * MAX_WORLD * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&h->send), world * blk_bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&h->status), sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(h->status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->side, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        const int rc = xfail(nullptr, PEER_ERR_CUDA, std::string("peer_xchg_create: ") + cudaGetErrorString(e));
        cudaFree(base); cudaFree(h->blocks_done); cudaFree(h->status); cudaFree(h->send);
        if (h->side) cudaStreamDestroy(h->side);
        if (h->fork) cudaEventDestroy(h->fork);
        delete h;
        return rc;
    }
    for (int r = 0; r < MAX_WORLD; ++r) h->map.base[r] = nullptr;
    h->map.base[rank] = static_cast<char*>(base);
    h->attached = world == 1;
    *out = h;
    return PEER_OK;
}

extern "C" int peer_xchg_export(peer_xchg_t h, unsigned char* handle64) {
    if (!h || !handle64) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t ipc;
    XCU(h, cudaIpcGetMemHandle(&ipc, h->map.base[h->rank]));
    std::memcpy(handle64, &ipc, 64);
    return PEER_OK;
}

extern "C" int peer_xchg_attach(peer_xchg_t h, const unsigned char* handles) {
    if (!h || !handles) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_attach: null argument");
    if (h->attached) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_attach: already attached");
    XCU(h, cudaSetDevice(h->device));
    for (int r = 0; r < h->world; ++r) {
        if (r == h->rank) continue;
        cudaIpcMemHandle_t ipc;
        std::memcpy(&ipc, handles + 64 * r, 64);
        void* p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, ipc, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess)
            return xfail(h, PEER_ERR_CUDA, "peer_xchg_attach: cannot map the region of rank " + std::to_string(r) + ": " +
                                               cudaGetErrorString(e));
        h->map.base[r] = static_cast<char*>(p);
    }
    h->attached = true;
    return PEER_OK;
}

extern "C" int peer_xchg_destroy(peer_xchg_t h) {
    if (!h) return PEER_OK;
    cudaSetDevice(h->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < h->world; ++r)
        if (r != h->rank && h->map.base[r]) cudaIpcCloseMemHandle(h->map.base[r]);
    cudaFree(h->map.base[h->rank]);
    cudaFree(h->blocks_done);
    cudaFree(h->status);
    cudaFree(h->send);
    cudaStreamDestroy(h->side);
    cudaEventDestroy(h->fork);
    delete h;
    return PEER_OK;
}

// Step part 1: my tokens' activations to every rank (and the step number with them).  Starts a new step.
extern "C" int peer_xchg_push_x(peer_xchg_t h, const void* x_local, void* stream) {
    if (!h || !x_local) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_push_x: null argument");
    if (!h->attached) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_push_x: peer_xchg_attach has not been called");
    h->step += 1;
    const int p = h->step & 1;
    const int64_t bytes = h->t_local * h->d_in * act_size(h->act_dtype);
    push_kernel<<<dim3(h->world, PUSH_BLOCKS), 512, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const char*>(x_local), 0, h->map, h->lay.x_all[p] + static_cast<size_t>(h->rank) * bytes, bytes,
        h->lay.flags + (0 * MAX_WORLD + h->rank) * 4, h->step, h->blocks_done + MAX_WORLD);
    XCU(h, cudaGetLastError());
    return PEER_OK;
}

// Step part 2: my tokens' tuples (flat expert ids, softmax weights: [T, E]) into the owners' blocks.
extern "C" int peer_xchg_route(peer_xchg_t h, const int32_t* ids, const float* weights, int64_t rows_per_rank, void* stream) {
    if (!h || !ids || !weights || rows_per_rank < 1) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_route: bad argument");
    if (h->step < 1) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_route: no step in progress (peer_xchg_push_x starts one)");
    const int p = h->step & 1;
    const size_t blk_bytes = (2 * static_cast<size_t>(h->t_local) * h->entries + h->t_local) * 4;
    // the blocks are formed here (route.cu) and then go out in whole 16-byte stores, like the activations
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    XCU(h, launch_route_tuples(ids, weights, h->t_local, h->entries, rows_per_rank, h->world, h->send, s));
    push_kernel<<<dim3(h->world, PUSH_BLOCKS), 512, 0, s>>>(reinterpret_cast<const char*>(h->send), static_cast<int64_t>(blk_bytes),
                                                          h->map, h->lay.recv[p] + h->rank * blk_bytes, static_cast<int64_t>(blk_bytes),
                                                          h->lay.flags + (1 * MAX_WORLD + h->rank) * 4, h->step, h->blocks_done);
    XCU(h, cudaGetLastError());
    return PEER_OK;
}

// Step part 3: wait (bounded) until every rank's activations and tuples of this step are here; returns where.
extern "C" int peer_xchg_wait_inputs(peer_xchg_t h, const void** x_all, const int32_t** recv, void* stream) {
    if (!h || !x_all || !recv) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_wait_inputs: null argument");
    if (h->step < 1) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_wait_inputs: no step in progress");
    const int p = h->step & 1;
    char* mine = h->map.base[h->rank];
    wait_kernel<<<1, 2 * MAX_WORLD, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const int*>(mine + h->lay.flags), 0, 1, h->world, h->step, h->status);
    XCU(h, cudaGetLastError());
    *x_all = mine + h->lay.x_all[p];
    *recv = reinterpret_cast<const int32_t*>(mine + h->lay.recv[p]);
    return PEER_OK;
}

// Step part 4: my partial sums of all tokens (fp32 [world * T, d_out]) to the tokens' ranks; then the sum over
// the ranks' contributions to my tokens, in rank order, cast to the activation dtype: out [T, d_out].
extern "C" int peer_xchg_combine(peer_xchg_t h, const float* partial, void* out, void* stream) {
    if (!h || !partial || !out) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_combine: null argument");
    if (h->step < 1) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_combine: no step in progress");
    const int p = h->step & 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t slot_bytes = h->t_local * h->d_out * 4;
    push_kernel<<<dim3(h->world, PUSH_BLOCKS), 512, 0, s>>>(reinterpret_cast<const char*>(partial), slot_bytes, h->map,
                                                          h->lay.part_in[p] + static_cast<size_t>(h->rank) * slot_bytes, slot_bytes,
                                                          h->lay.flags + (2 * MAX_WORLD + h->rank) * 4, h->step, h->blocks_done);
    XCU(h, cudaGetLastError());
    char* mine = h->map.base[h->rank];
    const int64_t n = h->t_local * h->d_out;
    const unsigned blocks = static_cast<unsigned>((n / 4 + 255) / 256);
    const float* pin = reinterpret_cast<const float*>(mine + h->lay.part_in[p]);
    const int* fl = reinterpret_cast<const int*>(mine + h->lay.flags) + 2 * MAX_WORLD;
    if (h->act_dtype == PEER_DTYPE_F32)
        sum_cast_kernel<float><<<blocks, 256, 0, s>>>(pin, fl, h->world, n, h->step, static_cast<float*>(out), h->status);
    else if (h->act_dtype == PEER_DTYPE_F16)
        sum_cast_kernel<__half><<<blocks, 256, 0, s>>>(pin, fl, h->world, n, h->step, static_cast<__half*>(out), h->status);
    else
        sum_cast_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(pin, fl, h->world, n, h->step, static_cast<__nv_bfloat16*>(out), h->status);
    XCU(h, cudaGetLastError());
    return PEER_OK;
}

// One whole step of the expert-parallel layer in one call (the host's time to enqueue a step is what bounds a
// decode-shaped batch): push x, select for my tokens, route, wait, evaluate against my rows, combine.
// t->x = my T tokens; ids_scratch / weights_scratch [T, E] and partial_scratch fp32 [world * T, d_out] are the
// caller's device buffers; expert_down / expert_up (+ scales) are this rank's rows; out [T, d_out].
extern "C" int peer_xchg_forward(peer_xchg_t x, peer_handle_t h, const peer_tensors_t* t, int32_t* ids_scratch,
                                 float* weights_scratch, int64_t rows_per_rank, float* partial_scratch, void* out,
                                 void* stream) {
    if (!x || !h || !t || !ids_scratch || !weights_scratch || !partial_scratch || !out)
        return xfail(x, PEER_ERR_INVALID_ARG, "peer_xchg_forward: null argument");
    // The activations travel on a stream of their own while the selection runs: nothing on `stream` has to wait
    // for them before peer_xchg_wait_inputs, which sees this rank's own step number like everybody else's.
    // (Their push uses its own completion counters: the routing's push may run at the same time.)
    cudaStream_t main_s = static_cast<cudaStream_t>(stream);
    XCU(x, cudaEventRecord(x->fork, main_s));
    XCU(x, cudaStreamWaitEvent(x->side, x->fork, 0));
    int rc = peer_xchg_push_x(x, t->x, x->side);
    if (rc) return rc;
    rc = peer_select_tokens(h, t, x->t_local, ids_scratch, weights_scratch, stream);
    if (rc) return xfail(x, rc, std::string("peer_xchg_forward: selection: ") + peer_last_error(h));
    rc = peer_xchg_route(x, ids_scratch, weights_scratch, rows_per_rank, stream);
    if (rc) return rc;
    const void* x_all = nullptr; const int32_t* recv = nullptr;
    rc = peer_xchg_wait_inputs(x, &x_all, &recv, stream);
    if (rc) return rc;
    rc = peer_gather_eval_routed(h, x_all, recv, x->world, x->t_local, t->expert_down, t->expert_up, t->down_scale,
                                 t->up_scale, rows_per_rank, partial_scratch, stream);
    if (rc) return xfail(x, rc, std::string("peer_xchg_forward: expert stage: ") + peer_last_error(h));
    return peer_xchg_combine(x, partial_scratch, out, stream);
}

// How many tuples each of the world * T tokens brought to this rank in the current step (the counts of the
// received blocks, after peer_xchg_wait_inputs): int32 [world * T] on the device.
extern "C" int peer_xchg_counts(peer_xchg_t h, int32_t* counts_out, void* stream) {
    if (!h || !counts_out) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_counts: null argument");
    if (h->step < 1) return xfail(h, PEER_ERR_INVALID_ARG, "peer_xchg_counts: no step in progress");
    const int p = h->step & 1;
    const size_t blk_words = 2 * static_cast<size_t>(h->t_local) * h->entries + h->t_local;
    const int32_t* recv = reinterpret_cast<const int32_t*>(h->map.base[h->rank] + h->lay.recv[p]);
    for (int r = 0; r < h->world; ++r)
        XCU(h, cudaMemcpyAsync(counts_out + r * h->t_local, recv + r * blk_words + 2 * h->t_local * h->entries,
                               h->t_local * sizeof(int32_t), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
    return PEER_OK;
}

// Synchronises the stream and reports a wait that ran out (a peer that did not deliver within two seconds).
extern "C" int peer_xchg_status(peer_xchg_t h, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    int st = 0;
    XCU(h, cudaMemcpyAsync(&st, h->status, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    XCU(h, cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    if (st == STATUS_TIMEOUT) {
        cudaMemset(h->status, 0, sizeof(int));
        return xfail(h, PEER_ERR_DEVICE_TIMEOUT, "peer_xchg: a rank's data did not arrive within two seconds");
    }
    return PEER_OK;
}
