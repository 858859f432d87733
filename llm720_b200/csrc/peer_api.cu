// C ABI of the PEER forward library: handle management, argument checking
// and the stage pipeline.  See include/peer_b200.h for the contract.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"

using namespace peer;

struct peer_op {
    peer_config_t cfg;
    int device = 0;
    int sm_count = 0;
    int kp0 = 0, kp1 = 0, k_final = 0;
    int mult0 = 1, mult1 = 1;
    int n_pairs = 0;
    // general form: any number of key dimensions, any number of neurons per expert
    int nd = 2;
    int n[4] = {0, 0, 0, 0};
    int kp[4] = {0, 0, 0, 0};
    long long mult[4] = {1, 1, 1, 1};
    bool general_select = false;  // key grid that is not two-dimensional: select_nd.cu
    int hidden = 1;
    // device scratch
    float* khat0 = nullptr;       // [Q/2, n0] normalised sub-keys, transposed
    float* khat1 = nullptr;       // [Q/2, n1]
    float* q_hat = nullptr;       // [max_tokens, H, Q]
    __nv_bfloat16* q_split = nullptr;   // [3][max_tokens, H, Q]: hi/mid/lo bf16 terms of q_hat (tensor-core path)
    bool use_tc = false;          // bf16 layer whose shapes the tcgen05 query kernel covers
    bool use_tc_select = false;   // ... and the tcgen05 select kernel
    float* invn0 = nullptr;       // [n0] 1/||key|| (tensor-core select)
    float* invn1 = nullptr;       // [n1]
    int32_t* ovf_rows = nullptr;  // [max_tokens*H] rows the tensor-core select leaves to the exact kernel
    int* ovf_count = nullptr;
    unsigned long long* sel_stats = nullptr;   // [2] accumulated: pooled row-halves, rows redone by the exact kernel
    float* sel_eps = nullptr;                  // [2] error bound of the select kernel's two-term first pass, per table
    // tiered residency (peer_set_row_tier; caller-owned): which rows sit in the HBM cache, and the cache
    const int32_t* tier_map = nullptr;
    const void* tier_cache_down = nullptr;
    const void* tier_cache_up = nullptr;
    void* x_ln = nullptr;         // [max_tokens, D] act dtype: LayerNorm of the block input (peer_block_forward)
    int32_t* sel_ids = nullptr;   // [max_tokens, H*k]
    float* sel_w = nullptr;       // [max_tokens, H*k]
    uint16_t* pairs = nullptr;
    int* status = nullptr;
    // host-buffer pipeline (created on first peer_forward_host)
    int64_t host_chunk = 0;
    cudaStream_t st_in = nullptr, st_run = nullptr, st_out = nullptr;
    cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_run[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
    void* d_x[2] = {nullptr, nullptr};
    void* d_out[2] = {nullptr, nullptr};
    int64_t* d_ids[2] = {nullptr, nullptr};
    float* d_sc[2] = {nullptr, nullptr};
    int64_t host_slices = 0;      // slices submitted so far by the host-buffer path (staging buffers alternate)
    int64_t host_calls = 0;       // calls submitted so far: the ticket of the next call
    cudaEvent_t ev_call[8] = {};  // completion of the last 8 calls (recorded after their last copy-out)
    int64_t launches = 0;
    // optional per-stage timing (peer_stage_timing): events recorded around each stage launch
    bool timing = false;
    // peer_freeze_keys: what the selection derives from the sub-keys is reused while the same tables come on the same stream
    bool keys_frozen = false;
    const void* frozen_k0 = nullptr; const void* frozen_k1 = nullptr; cudaStream_t frozen_stream = nullptr; bool frozen_valid = false;
    std::vector<cudaEvent_t> tev;   // 4 per slice: before query, before select, before expert stage, after
    size_t tev_used = 0;
    std::string err;
};

// errors that have no handle to live on (failed peer_create, handle-free entry points): one text per host thread
static thread_local std::string g_create_error;

static int fail(peer_op* h, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (h) h->err = buf; else g_create_error = buf;
    return code;
}

#define CU_TRY(h, expr)                                                                   \
    do {                                                                                  \
        cudaError_t e_ = (expr);                                                          \
        if (e_ != cudaSuccess)                                                            \
            return fail(h, PEER_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

namespace peer {
// used by entry points that have no handle to hang an error text on
void set_global_error(const char* msg) { g_create_error = msg ? msg : ""; }
}  // namespace peer

static int act_bytes(int dt) { return dt == PEER_DTYPE_F32 ? 4 : ((dt == PEER_DTYPE_BF16 || dt == PEER_DTYPE_F16) ? 2 : 1); }
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// k' of the reference (llm/models/experts.py:168-187).
static int candidates_per_dim(int top_k, int dim_size, int num_dims = 2) {
    const int base = static_cast<int>(std::ceil(std::pow(static_cast<double>(top_k), 1.0 / num_dims))) + 2;
    int kp = base < dim_size ? base : dim_size;
    const int want = dim_size >= top_k ? top_k : dim_size;
    if (kp < want) kp = want;
    if (kp > dim_size) kp = dim_size;
    return kp < 1 ? 1 : kp;
}

namespace peer { int candidates_per_dim_2d(int top_k, int dim_size) { return candidates_per_dim(top_k, dim_size); } }

static void free_all(peer_op* h) {
    cudaFree(h->khat0); cudaFree(h->khat1); cudaFree(h->q_hat); cudaFree(h->q_split); cudaFree(h->invn0); cudaFree(h->invn1); cudaFree(h->ovf_rows); cudaFree(h->ovf_count); cudaFree(h->sel_stats); cudaFree(h->sel_eps); cudaFree(h->sel_ids);
    cudaFree(h->sel_w); cudaFree(h->pairs); cudaFree(h->status); cudaFree(h->x_ln);
    for (int b = 0; b < 2; ++b) {
        cudaFree(h->d_x[b]); cudaFree(h->d_out[b]); cudaFree(h->d_ids[b]); cudaFree(h->d_sc[b]);
        if (h->ev_in[b]) cudaEventDestroy(h->ev_in[b]);
        if (h->ev_run[b]) cudaEventDestroy(h->ev_run[b]);
        if (h->ev_out[b]) cudaEventDestroy(h->ev_out[b]);
    }
    for (int i = 0; i < 8; ++i) if (h->ev_call[i]) cudaEventDestroy(h->ev_call[i]);
    for (cudaEvent_t e : h->tev) cudaEventDestroy(e);
    h->tev.clear();
    if (h->st_in) cudaStreamDestroy(h->st_in);
    if (h->st_run) cudaStreamDestroy(h->st_run);
    if (h->st_out) cudaStreamDestroy(h->st_out);
}

extern "C" int peer_abi_version(void) { return PEER_B200_ABI_VERSION; }

extern "C" const char* peer_last_error(peer_handle_t h) {
    return h ? h->err.c_str() : g_create_error.c_str();
}

extern "C" int64_t peer_launch_count(peer_handle_t h) { return h ? h->launches : 0; }

extern "C" int peer_create(const peer_config_t* c, peer_handle_t* out) {
    if (!c || !out) return fail(nullptr, PEER_ERR_INVALID_ARG, "peer_create: null argument");
    *out = nullptr;
    if (c->abi_version != PEER_B200_ABI_VERSION)
        return fail(nullptr, PEER_ERR_INVALID_ARG, "peer_create: abi_version %d, library has %d",
                    c->abi_version, PEER_B200_ABI_VERSION);
    if (c->expert_hidden_size < 1 || c->expert_hidden_size > 16)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "expert_hidden_size=%d: 1 to 16 neurons per expert are implemented",
                    c->expert_hidden_size);
    if (c->expert_hidden_size > 1 && c->table_dtype != c->act_dtype)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "experts with several neurons need tables in the layer's dtype");
    const int nd = c->num_key_dims == 0 ? 2 : c->num_key_dims;
    if (nd < 1 || nd > 4)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "num_key_dims=%d: 1 to 4 key dimensions are implemented", nd);
    const int nkeys[4] = {c->n_keys0, nd > 1 ? c->n_keys1 : 1, nd > 2 ? c->n_keys2 : 1, nd > 3 ? c->n_keys3 : 1};
    if (c->activation != PEER_ACT_GELU && c->activation != PEER_ACT_RELU)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "activation %d is not implemented", c->activation);
    if (c->act_dtype != PEER_DTYPE_F32 && c->act_dtype != PEER_DTYPE_BF16 && c->act_dtype != PEER_DTYPE_F16)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "act_dtype must be fp32, bf16 or fp16");
    const bool combo = (c->act_dtype == PEER_DTYPE_F32 && c->table_dtype == PEER_DTYPE_F32) ||
                       (c->act_dtype == PEER_DTYPE_F16 && c->table_dtype == PEER_DTYPE_F16) ||
                       (c->act_dtype == PEER_DTYPE_BF16 && (c->table_dtype == PEER_DTYPE_BF16 || c->table_dtype == PEER_DTYPE_E4M3));
    if (!combo)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "unsupported dtype pair: act %d, table %d (fp32/fp32, bf16/bf16, bf16/e4m3, fp16/fp16)",
                    c->act_dtype, c->table_dtype);
    if (c->input_dim <= 0 || c->output_dim <= 0 || c->num_heads <= 0 || c->top_k <= 0 || nkeys[0] <= 0 ||
        nkeys[1] <= 0 || nkeys[2] <= 0 || nkeys[3] <= 0 || c->query_dim <= 0 || c->max_tokens <= 0)
        return fail(nullptr, PEER_ERR_INVALID_ARG, "peer_create: non-positive dimension");
    if (static_cast<int64_t>(nkeys[0]) * nkeys[1] * nkeys[2] * nkeys[3] != c->num_experts)
        return fail(nullptr, PEER_ERR_INVALID_ARG, "product of key dimensions %d x %d x %d x %d must equal num_experts %lld",
                    nkeys[0], nkeys[1], nkeys[2], nkeys[3], static_cast<long long>(c->num_experts));
    if (c->num_experts > 0x7fffffffLL)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "num_experts above 2^31-1");
    if (c->query_dim % nd || c->query_dim > 256)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "query_dim=%d: must be a multiple of the %d key dimensions and <= 256",
                    c->query_dim, nd);
    if (c->input_dim % 8)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "input_dim=%d: must be a multiple of 8", c->input_dim);
    const int tb = act_bytes(c->table_dtype);
    if ((c->input_dim * tb) % 16 || (c->output_dim * tb) % 16 || (c->output_dim * act_bytes(c->act_dtype)) % 16)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "table rows and output rows must be multiples of 16 bytes");
    if (c->top_k > 32)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "top_k=%d: at most 32", c->top_k);
    if (c->index_mode != PEER_INDEX_REFERENCE && c->index_mode != PEER_INDEX_PRODUCT)
        return fail(nullptr, PEER_ERR_INVALID_ARG, "index_mode %d", c->index_mode);

    int dev = 0;
    cudaDeviceProp prop;
    CU_TRY(nullptr, cudaGetDevice(&dev));
    CU_TRY(nullptr, cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only",
                    dev, prop.major, prop.minor);

    peer_op* h = new (std::nothrow) peer_op();
    if (!h) return fail(nullptr, PEER_ERR_CUDA, "out of host memory");
    h->cfg = *c;
    h->device = dev;
    h->sm_count = prop.multiProcessorCount;
    h->nd = nd;
    h->hidden = c->expert_hidden_size;
    h->general_select = nd != 2;
    {   // per-dimension candidate counts, id strides, and how many entries the folds leave
        long long len = 0;
        for (int d = 0; d < nd; ++d) {
            h->n[d] = nkeys[d];
            h->kp[d] = candidates_per_dim(c->top_k, nkeys[d], nd);
            if (h->kp[d] > 32) { delete h; return fail(nullptr, PEER_ERR_UNSUPPORTED, "more than 32 candidates per key dimension"); }
            if (d == 0) len = nd == 1 ? (c->top_k < h->kp[0] ? c->top_k : h->kp[0]) : h->kp[0];
            else {
                const long long count = len * h->kp[d];
                const long long keep = d < nd - 1 ? 4LL * c->top_k : c->top_k;
                len = keep < count ? keep : count;
            }
        }
        h->mult[nd - 1] = 1;
        for (int d = nd - 2; d >= 0; --d) h->mult[d] = h->mult[d + 1] * nkeys[d + 1];
        if (c->index_mode == PEER_INDEX_REFERENCE) h->mult[0] = nd == 1 ? 0 : 1;   // llm/models/experts.py:203-204; 1-D: :197-200
        if (len < c->top_k) {
            delete h;
            return fail(nullptr, PEER_ERR_UNSUPPORTED, "top_k=%d exceeds the %lld candidates this key grid yields",
                        c->top_k, len);
        }
    }
    if (h->general_select) {
        h->k_final = c->top_k;
        const int64_t HKg = static_cast<int64_t>(c->num_heads) * c->top_k;
        cudaError_t eg = cudaMalloc(reinterpret_cast<void**>(&h->q_hat), sizeof(float) * c->max_tokens * c->num_heads * c->query_dim);
        if (eg == cudaSuccess) eg = cudaMalloc(reinterpret_cast<void**>(&h->sel_ids), sizeof(int32_t) * c->max_tokens * HKg);
        if (eg == cudaSuccess) eg = cudaMalloc(reinterpret_cast<void**>(&h->sel_w), sizeof(float) * c->max_tokens * HKg);
        if (eg == cudaSuccess) eg = cudaMalloc(reinterpret_cast<void**>(&h->status), sizeof(int));
        if (eg == cudaSuccess) eg = cudaMemset(h->status, 0, sizeof(int));
        if (eg != cudaSuccess) {
            fail(nullptr, PEER_ERR_CUDA, "peer_create: %s", cudaGetErrorString(eg));
            free_all(h);
            delete h;
            return PEER_ERR_CUDA;
        }
        *out = h;
        return PEER_OK;
    }
    h->kp0 = candidates_per_dim(c->top_k, c->n_keys0);
    h->kp1 = candidates_per_dim(c->top_k, c->n_keys1);
    if (h->kp0 > 32 || h->kp1 > 32) { delete h; return fail(nullptr, PEER_ERR_UNSUPPORTED, "more than 32 candidates per half"); }
    const int64_t cand = static_cast<int64_t>(h->kp0) * h->kp1;
    h->k_final = c->top_k < cand ? c->top_k : static_cast<int>(cand);
    if (h->k_final != c->top_k) {
        delete h;
        return fail(nullptr, PEER_ERR_UNSUPPORTED, "top_k=%d exceeds the %lld candidates of a %dx%d key grid",
                    c->top_k, static_cast<long long>(cand), c->n_keys0, c->n_keys1);
    }
    h->mult0 = c->index_mode == PEER_INDEX_PRODUCT ? c->n_keys1 : 1;
    h->mult1 = 1;

    std::vector<uint16_t> pairs;
    for (int a = 0; a < h->kp0; ++a)
        for (int b = 0; b < h->kp1; ++b)
            if ((a + 1) * (b + 1) <= h->k_final) pairs.push_back(static_cast<uint16_t>((a << 8) | b));
    h->n_pairs = static_cast<int>(pairs.size());
    if (h->n_pairs > MAX_PAIRS) { delete h; return fail(nullptr, PEER_ERR_UNSUPPORTED, "too many candidate pairs"); }

    const int hw = c->query_dim / 2;
    const int64_t HK = static_cast<int64_t>(c->num_heads) * c->top_k;
    cudaError_t e = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(p, bytes); };
    alloc(reinterpret_cast<void**>(&h->khat0), sizeof(float) * hw * c->n_keys0);
    alloc(reinterpret_cast<void**>(&h->khat1), sizeof(float) * hw * c->n_keys1);
    alloc(reinterpret_cast<void**>(&h->q_hat), sizeof(float) * c->max_tokens * c->num_heads * c->query_dim);
    {
        QueryArgs probe{};
        probe.act_dtype = c->act_dtype; probe.Q = c->query_dim; probe.D = c->input_dim;
        h->use_tc = query_tc_supported(probe);
    }
    h->use_tc_select = h->use_tc && select_tc_supported(c->act_dtype, c->query_dim, c->n_keys0, c->n_keys1,
                                                        h->k_final, h->kp0, h->kp1);
    if (h->use_tc_select) {
        alloc(reinterpret_cast<void**>(&h->invn0), sizeof(float) * c->n_keys0);
        alloc(reinterpret_cast<void**>(&h->invn1), sizeof(float) * c->n_keys1);
        alloc(reinterpret_cast<void**>(&h->ovf_rows), sizeof(int32_t) * c->max_tokens * c->num_heads);
        alloc(reinterpret_cast<void**>(&h->ovf_count), sizeof(int));
        alloc(reinterpret_cast<void**>(&h->sel_stats), 2 * sizeof(unsigned long long));
        if (c->norm_query)          // the two-term first pass needs unit queries for its error bound
            alloc(reinterpret_cast<void**>(&h->sel_eps), 2 * sizeof(float));
        if (e == cudaSuccess) e = cudaMemset(h->sel_stats, 0, 2 * sizeof(unsigned long long));
    }
    if (h->use_tc)
        alloc(reinterpret_cast<void**>(&h->q_split), sizeof(__nv_bfloat16) * 3 * c->max_tokens * c->num_heads * c->query_dim);
    alloc(reinterpret_cast<void**>(&h->sel_ids), sizeof(int32_t) * c->max_tokens * HK);
    alloc(reinterpret_cast<void**>(&h->sel_w), sizeof(float) * c->max_tokens * HK);
    alloc(reinterpret_cast<void**>(&h->pairs), sizeof(uint16_t) * MAX_PAIRS);
    alloc(reinterpret_cast<void**>(&h->status), sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpy(h->pairs, pairs.data(), sizeof(uint16_t) * pairs.size(), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(h->status, 0, sizeof(int));
    if (e == cudaSuccess) e = select_simt_setup();
    if (e == cudaSuccess && h->use_tc) e = query_tc_setup();
    if (e == cudaSuccess && h->use_tc_select) e = select_tc_setup();
    if (e != cudaSuccess) {
        fail(nullptr, PEER_ERR_CUDA, "peer_create: %s", cudaGetErrorString(e));
        free_all(h);
        delete h;
        return PEER_ERR_CUDA;
    }
    *out = h;
    return PEER_OK;
}

extern "C" int peer_destroy(peer_handle_t h) {
    if (!h) return PEER_OK;
    cudaDeviceSynchronize();
    free_all(h);
    delete h;
    return PEER_OK;
}

static int check_tensors(peer_op* h, const peer_tensors_t* t, bool need_tables) {
    const peer_config_t& c = h->cfg;
    if (!t) return fail(h, PEER_ERR_INVALID_ARG, "null tensor struct");
    if (!t->x || !t->query_w || !t->keys0 || (h->nd > 1 && !t->keys1) || (h->nd > 2 && !t->keys2) || (h->nd > 3 && !t->keys3))
        return fail(h, PEER_ERR_INVALID_ARG, "x, query_w and one sub-key table per key dimension are required");
    if (need_tables) {
        if (!t->expert_down || !t->expert_up || !t->out)
            return fail(h, PEER_ERR_INVALID_ARG, "expert_down, expert_up and out are required");
        if (c.table_dtype == PEER_DTYPE_E4M3 && (!t->down_scale || !t->up_scale))
            return fail(h, PEER_ERR_INVALID_ARG, "FP8 tables need down_scale and up_scale");
        if (!aligned16(t->expert_down) || !aligned16(t->expert_up) || !aligned16(t->out))
            return fail(h, PEER_ERR_INVALID_ARG, "expert tables and out must be 16-byte aligned");
    }
    if (!aligned16(t->x) || !aligned16(t->query_w))
        return fail(h, PEER_ERR_INVALID_ARG, "x and query_w must be 16-byte aligned");
    return PEER_OK;
}

static bool keys_still_prepared(peer_op* h, const void* keys0, const void* keys1, cudaStream_t s) {
    return h->keys_frozen && h->frozen_valid && h->frozen_k0 == keys0 && h->frozen_k1 == keys1 && h->frozen_stream == s;
}
static void keys_prepared(peer_op* h, const void* keys0, const void* keys1, cudaStream_t s) {
    h->frozen_k0 = keys0; h->frozen_k1 = keys1; h->frozen_stream = s; h->frozen_valid = true;
}

static int normalise_keys(peer_op* h, const void* keys0, const void* keys1, cudaStream_t s) {
    if (keys_still_prepared(h, keys0, keys1, s)) return PEER_OK;
    const peer_config_t& c = h->cfg;
    const int hw = c.query_dim / 2;
    CU_TRY(h, launch_normalize_rows(keys0, c.act_dtype, c.n_keys0, hw, c.norm_keys, 1, h->khat0, s));
    CU_TRY(h, launch_normalize_rows(keys1, c.act_dtype, c.n_keys1, hw, c.norm_keys, 1, h->khat1, s));
    h->launches += 2;
    keys_prepared(h, keys0, keys1, s);
    return PEER_OK;
}

// Tensor-core selection: 1/||key|| per sub-key for the kernel itself (it contracts with the keys as stored), the
// normalised keys for the exact kernel behind it, and the first pass's error bounds, in one launch
static int key_prep(peer_op* h, const void* keys0, const void* keys1, cudaStream_t s) {
    if (keys_still_prepared(h, keys0, keys1, s)) return PEER_OK;
    const peer_config_t& c = h->cfg;
    CU_TRY(h, launch_key_prep(keys0, keys1, c.n_keys0, c.n_keys1, c.query_dim / 2, c.norm_keys, h->khat0, h->khat1,
                              h->invn0, h->invn1, h->sel_eps, s));
    h->launches += 1;
    keys_prepared(h, keys0, keys1, s);
    return PEER_OK;
}

static SelectArgs select_args(peer_op* h, int64_t n_tokens) {
    const peer_config_t& c = h->cfg;
    SelectArgs a{};
    a.q_hat = h->q_hat; a.khat0 = h->khat0; a.khat1 = h->khat1;
    a.rows = n_tokens * c.num_heads; a.Q = c.query_dim; a.n0 = c.n_keys0; a.n1 = c.n_keys1;
    a.kp0 = h->kp0; a.kp1 = h->kp1; a.k = h->k_final; a.mult0 = h->mult0; a.mult1 = h->mult1;
    a.pairs = h->pairs; a.n_pairs = h->n_pairs;
    return a;
}

// Tensor-core selection of one slice from h->q_split (hi/mid/lo terms of the normalised queries), followed by
// the exact CUDA-core kernel on the rows the tensor-core kernel handed over (none for ordinary data).
static int select_tc_slice(peer_op* h, const void* keys0, const void* keys1, int64_t n, int32_t* ids32, float* weights,
                           int64_t* ids_out, float* scores_out, int32_t* prod_out, cudaStream_t s) {
    const peer_config_t& c = h->cfg;
    SelectTcArgs ta{};
    ta.q_split = h->q_split; ta.term_rows = c.max_tokens * c.num_heads; ta.keys0 = keys0; ta.keys1 = keys1;
    ta.invn0 = h->invn0; ta.invn1 = h->invn1; ta.rows = n * c.num_heads; ta.Q = c.query_dim;
    ta.n0 = c.n_keys0; ta.n1 = c.n_keys1; ta.kp0 = h->kp0; ta.kp1 = h->kp1; ta.k = h->k_final;
    ta.mult0 = h->mult0; ta.mult1 = h->mult1; ta.ids32 = ids32; ta.weights = weights;
    ta.ids64 = ids_out; ta.raw_scores = scores_out; ta.status = h->status; ta.sm_count = h->sm_count;
    ta.prod_ids = prod_out;
    ta.overflow_rows = h->ovf_rows; ta.overflow_count = h->ovf_count; ta.stats = h->sel_stats;
    if (h->sel_eps) { ta.eps0 = h->sel_eps; ta.eps1 = h->sel_eps + 1; }
    CU_TRY(h, cudaMemsetAsync(h->ovf_count, 0, sizeof(int), s));
    CU_TRY(h, launch_select_tc(ta, s));
    SelectArgs fx = select_args(h, n);
    fx.q_hat = nullptr; fx.q_split = h->q_split; fx.split_stride = c.max_tokens * c.num_heads * c.query_dim;
    fx.row_list = h->ovf_rows; fx.row_count = h->ovf_count;
    fx.ids32 = ids32; fx.weights = weights; fx.ids64 = ids_out; fx.raw_scores = scores_out;
    fx.prod_ids = prod_out;
    CU_TRY(h, launch_select_simt(fx, s));
    return PEER_OK;
}

// One slice (n <= max_tokens) of the layer, all pointers on the device.
static int forward_slice(peer_op* h, const peer_tensors_t* t, const void* x, void* out, int64_t* ids_out,
                         float* scores_out, int64_t n, cudaStream_t s, const void* residual = nullptr,
                         int32_t* prod_out = nullptr, int32_t* sel_ids_to = nullptr, float* sel_w_to = nullptr) {
    // where the selection goes: the handle's scratch, or (peer_select_tokens) the caller's buffers
    int32_t* const sel_ids = sel_ids_to ? sel_ids_to : h->sel_ids;
    float* const sel_w = sel_w_to ? sel_w_to : h->sel_w;
    const peer_config_t& c = h->cfg;
    QueryArgs q{};
    q.x = x; q.w = t->query_w; q.b = t->query_b; q.ln_w = t->ln_w; q.ln_b = t->ln_b;
    q.q_ln_out = nullptr; q.q_hat_out = h->use_tc_select ? nullptr : h->q_hat; q.T = n; q.D = c.input_dim; q.H = c.num_heads;
    q.Q = c.query_dim; q.layer_norm = c.layer_norm; q.norm_query = c.norm_query; q.act_dtype = c.act_dtype;
    if (h->general_select) { q.q_ln_out = h->q_hat; q.q_hat_out = nullptr; }
    cudaEvent_t* ev = nullptr;
    if (h->timing) {
        if (h->tev_used + 4 > h->tev.size()) {
            for (int i = 0; i < 4; ++i) {
                cudaEvent_t e;
                CU_TRY(h, cudaEventCreate(&e));
                h->tev.push_back(e);
            }
        }
        ev = &h->tev[h->tev_used];
        h->tev_used += 4;
        CU_TRY(h, cudaEventRecord(ev[0], s));
    }
    if (h->use_tc)
        CU_TRY(h, launch_query_tc(q, h->q_split, c.max_tokens * c.num_heads * c.query_dim, h->status, h->sm_count, s));
    else
        CU_TRY(h, launch_query_simt(q, s));
    if (ev) CU_TRY(h, cudaEventRecord(ev[1], s));

    if (h->general_select) {
        SelectNdArgs na{};
        na.q_ln = h->q_hat;
        const void* kk[4] = {t->keys0, t->keys1, t->keys2, t->keys3};
        for (int d = 0; d < h->nd; ++d) { na.keys[d] = kk[d]; na.n[d] = h->n[d]; na.kp[d] = h->kp[d]; na.mult[d] = h->mult[d]; }
        na.nd = h->nd; na.Q = c.query_dim; na.k = c.top_k; na.norm_keys = c.norm_keys; na.norm_query = c.norm_query;
        na.act_dtype = c.act_dtype; na.rows = n * c.num_heads;
        na.ids32 = sel_ids; na.weights = sel_w; na.ids64 = ids_out; na.raw_scores = scores_out;
        na.prod_ids = prod_out;
        na.stride[h->nd - 1] = 1;
        for (int d = h->nd - 2; d >= 0; --d) na.stride[d] = na.stride[d + 1] * h->n[d + 1];
        cudaError_t se = launch_select_nd(na, s);
        if (se == cudaErrorInvalidValue) return fail(h, PEER_ERR_UNSUPPORTED, "selection over this key grid is not implemented");
        CU_TRY(h, se);
    } else if (h->use_tc_select) {
        const int rc_sel = select_tc_slice(h, t->keys0, t->keys1, n, sel_ids, sel_w, ids_out, scores_out, prod_out, s);
        if (rc_sel) return rc_sel;
        h->launches += 1;
    } else {
        SelectArgs sa = select_args(h, n);
        sa.ids32 = sel_ids; sa.weights = sel_w; sa.ids64 = ids_out; sa.raw_scores = scores_out;
        sa.prod_ids = prod_out;
        CU_TRY(h, launch_select_simt(sa, s));
    }
    if (ev) CU_TRY(h, cudaEventRecord(ev[2], s));
    if (!out) {                 // query and selection stages only (peer_select_tokens)
        if (ev) CU_TRY(h, cudaEventRecord(ev[3], s));
        h->launches += 2;
        return PEER_OK;
    }

    GatherArgs g{};
    g.x = x; g.ids = sel_ids; g.weights = sel_w; g.down = t->expert_down; g.up = t->expert_up;
    g.down_scale = t->down_scale; g.up_scale = t->up_scale; g.out = out; g.T = n;
    g.HK = c.num_heads * c.top_k; g.N = c.num_experts; g.D = c.input_dim; g.Dout = c.output_dim;
    g.act_dtype = c.act_dtype; g.table_dtype = c.table_dtype; g.activation = c.activation;
    g.status = h->status; g.sm_count = h->sm_count; g.hidden = h->hidden; g.residual = residual;
    // ids of the reference's arithmetic stay below n0 + n1: a few thousand rows, which live in L2
    g.rows_l2_resident = c.index_mode == PEER_INDEX_REFERENCE && h->nd == 2 &&
                         static_cast<int64_t>(c.n_keys0 + c.n_keys1) * (c.input_dim + c.output_dim) * act_bytes(c.table_dtype) <= (64LL << 20);
    const bool general_rows = h->hidden > 1 || c.act_dtype == PEER_DTYPE_F16;     // fp16 layers: the general kernel
    if (general_rows && g.hidden < 1) g.hidden = 1;
    if (h->tier_map) {
        if (general_rows || c.table_dtype == PEER_DTYPE_F32)
            return fail(h, PEER_ERR_UNSUPPORTED, "tiered table residency: bf16 and FP8 tables of single-neuron experts only");
        g.row_map = h->tier_map; g.cache_down = h->tier_cache_down; g.cache_up = h->tier_cache_up;
        g.rows_l2_resident = 0;
    }
    cudaError_t e = general_rows ? launch_gather_hidden(g, s) : launch_gather_eval(g, s);
    if (e == cudaErrorInvalidValue)
        return fail(h, PEER_ERR_UNSUPPORTED, "expert stage: row width %d/%d with this table dtype, or num_heads*top_k=%d, is not implemented",
                    c.input_dim, c.output_dim, g.HK);
    CU_TRY(h, e);
    if (ev) CU_TRY(h, cudaEventRecord(ev[3], s));
    h->launches += 3;
    return PEER_OK;
}

extern "C" int peer_set_row_tier(peer_handle_t h, const int32_t* row_map, const void* cache_down, const void* cache_up) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (!row_map) {             // back to tables that are wholly device-resident
        h->tier_map = nullptr; h->tier_cache_down = nullptr; h->tier_cache_up = nullptr;
        return PEER_OK;
    }
    if (!cache_down || !cache_up || !aligned16(cache_down) || !aligned16(cache_up))
        return fail(h, PEER_ERR_INVALID_ARG, "peer_set_row_tier: both cache tables are required, 16-byte aligned");
    if (h->hidden > 1 || h->cfg.act_dtype == PEER_DTYPE_F16 || h->cfg.table_dtype == PEER_DTYPE_F32)
        return fail(h, PEER_ERR_UNSUPPORTED, "tiered table residency: bf16 and FP8 tables of single-neuron experts only");
    h->tier_map = row_map; h->tier_cache_down = cache_down; h->tier_cache_up = cache_up;
    return PEER_OK;
}

extern "C" int peer_freeze_keys(peer_handle_t h, int frozen) {
    if (!h) return PEER_ERR_INVALID_ARG;
    h->keys_frozen = frozen != 0;
    h->frozen_valid = false;              // the next call prepares them (again)
    return PEER_OK;
}

extern "C" int peer_stage_timing(peer_handle_t h, int enable) {
    if (!h) return PEER_ERR_INVALID_ARG;
    h->timing = enable != 0;
    h->tev_used = 0;
    return PEER_OK;
}

extern "C" int peer_stage_times(peer_handle_t h, double* ms3, int64_t* n_slices) {
    if (!h || !ms3 || !n_slices) return PEER_ERR_INVALID_ARG;
    ms3[0] = ms3[1] = ms3[2] = 0.0;
    *n_slices = static_cast<int64_t>(h->tev_used / 4);
    for (size_t i = 0; i + 4 <= h->tev_used; i += 4) {
        CU_TRY(h, cudaEventSynchronize(h->tev[i + 3]));
        for (int j = 0; j < 3; ++j) {
            float ms = 0.f;
            CU_TRY(h, cudaEventElapsedTime(&ms, h->tev[i + j], h->tev[i + j + 1]));
            ms3[j] += ms;
        }
    }
    h->tev_used = 0;
    return PEER_OK;
}

extern "C" int peer_forward(peer_handle_t h, const peer_tensors_t* t, int64_t n_tokens, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens < 0) return fail(h, PEER_ERR_INVALID_ARG, "negative token count");
    if (n_tokens == 0) return PEER_OK;
    int rc = check_tensors(h, t, true);
    if (rc) return rc;
    const peer_config_t& c = h->cfg;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rc = h->general_select ? PEER_OK : (h->use_tc_select ? key_prep(h, t->keys0, t->keys1, s) : normalise_keys(h, t->keys0, t->keys1, s));
    if (rc) return rc;
    const int ab = act_bytes(c.act_dtype);
    const int64_t HK = static_cast<int64_t>(c.num_heads) * c.top_k;
    for (int64_t t0 = 0; t0 < n_tokens; t0 += c.max_tokens) {
        const int64_t n = n_tokens - t0 < c.max_tokens ? n_tokens - t0 : c.max_tokens;
        rc = forward_slice(h, t, static_cast<const char*>(t->x) + t0 * c.input_dim * ab,
                           static_cast<char*>(t->out) + t0 * c.output_dim * ab,
                           t->ids_out ? t->ids_out + t0 * HK : nullptr,
                           t->scores_out ? t->scores_out + t0 * HK : nullptr, n, s, nullptr,
                           t->product_ids_out ? t->product_ids_out + t0 * HK : nullptr);
        if (rc) return rc;
    }
    return PEER_OK;
}

static int host_pipeline_setup(peer_op* h, bool want_ids) {
    const peer_config_t& c = h->cfg;
    if (!h->st_in) {
        // Four rounds of one-token-per-warp of the expert stage (4,736 tokens on 148 SMs), capped by the
        // scratch: measured best on B200 (1,184: 2.50 M tokens/s end to end; 2,368: 3.27 M; 4,736: 3.56 M;
        // 8,192: 3.15 M) - every slice costs about 0.2 ms of launch gaps and partial waves, while long
        // slices delay the first kernel and the last copy-out.
        // That holds for a call that blocks until its output is complete.  Batches submitted ahead of one another
        // (peer_forward_host_async) hide the first copy-in and the last copy-out behind their neighbours' kernels,
        // so they run as one slice of up to max_tokens; the staging buffers are sized for that.
        int64_t chunk = static_cast<int64_t>(h->sm_count) * 8 * 4;
        if (chunk > c.max_tokens) chunk = c.max_tokens;
        h->host_chunk = chunk;
        chunk = c.max_tokens;
        CU_TRY(h, cudaStreamCreateWithFlags(&h->st_in, cudaStreamNonBlocking));
        CU_TRY(h, cudaStreamCreateWithFlags(&h->st_run, cudaStreamNonBlocking));
        CU_TRY(h, cudaStreamCreateWithFlags(&h->st_out, cudaStreamNonBlocking));
        const int ab = act_bytes(c.act_dtype);
        for (int b = 0; b < 2; ++b) {
            CU_TRY(h, cudaEventCreateWithFlags(&h->ev_in[b], cudaEventDisableTiming));
            CU_TRY(h, cudaEventCreateWithFlags(&h->ev_run[b], cudaEventDisableTiming));
            CU_TRY(h, cudaEventCreateWithFlags(&h->ev_out[b], cudaEventDisableTiming));
            CU_TRY(h, cudaMalloc(&h->d_x[b], static_cast<size_t>(chunk) * c.input_dim * ab));
            CU_TRY(h, cudaMalloc(&h->d_out[b], static_cast<size_t>(chunk) * c.output_dim * ab));
        }
    }
    if (want_ids && !h->d_ids[0]) {
        const size_t n = static_cast<size_t>(c.max_tokens) * c.num_heads * c.top_k;
        for (int b = 0; b < 2; ++b) {
            CU_TRY(h, cudaMalloc(reinterpret_cast<void**>(&h->d_ids[b]), n * sizeof(int64_t)));
            CU_TRY(h, cudaMalloc(reinterpret_cast<void**>(&h->d_sc[b]), n * sizeof(float)));
        }
    }
    return PEER_OK;
}

extern "C" int peer_block_forward(peer_handle_t h, const peer_tensors_t* t, const float* ln_w, const float* ln_b,
                                  float ln_eps, int64_t n_tokens, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens < 0) return fail(h, PEER_ERR_INVALID_ARG, "negative token count");
    if (n_tokens == 0) return PEER_OK;
    int rc = check_tensors(h, t, true);
    if (rc) return rc;
    const peer_config_t& c = h->cfg;
    if (c.input_dim != c.output_dim)
        return fail(h, PEER_ERR_INVALID_ARG, "peer_block_forward adds the input back: input_dim %d must equal output_dim %d",
                    c.input_dim, c.output_dim);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t ab = static_cast<size_t>(act_bytes(c.act_dtype));
    if (!h->x_ln) CU_TRY(h, cudaMalloc(&h->x_ln, ab * c.max_tokens * c.input_dim));
    rc = h->general_select ? PEER_OK : (h->use_tc_select ? key_prep(h, t->keys0, t->keys1, s) : normalise_keys(h, t->keys0, t->keys1, s));
    if (rc) return rc;
    const int64_t HK = static_cast<int64_t>(c.num_heads) * c.top_k;
    for (int64_t t0 = 0; t0 < n_tokens; t0 += c.max_tokens) {
        const int64_t n = n_tokens - t0 < c.max_tokens ? n_tokens - t0 : c.max_tokens;
        const char* xs = static_cast<const char*>(t->x) + t0 * c.input_dim * ab;
        CU_TRY(h, launch_block_ln(xs, c.act_dtype, n, c.input_dim, ln_w, ln_b, ln_eps, h->x_ln, s));
        h->launches += 1;
        rc = forward_slice(h, t, h->x_ln, static_cast<char*>(t->out) + t0 * c.output_dim * ab,
                           t->ids_out ? t->ids_out + t0 * HK : nullptr, t->scores_out ? t->scores_out + t0 * HK : nullptr,
                           n, s, xs);
        if (rc) return rc;
    }
    return PEER_OK;
}

static int host_submit(peer_op* h, const peer_tensors_t* t, int64_t n_tokens, int64_t* ticket, bool blocking) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens < 0) return fail(h, PEER_ERR_INVALID_ARG, "negative token count");
    if (!t || !t->x || !t->out) return fail(h, PEER_ERR_INVALID_ARG, "x and out are required");
    const peer_config_t& c = h->cfg;
    const bool want_ids = t->ids_out || t->scores_out;
    int rc = host_pipeline_setup(h, want_ids);
    if (rc) return rc;
    peer_tensors_t dt = *t;
    dt.x = h->d_x[0]; dt.out = h->d_out[0];
    rc = check_tensors(h, &dt, true);
    if (rc) return rc;
    rc = h->general_select ? PEER_OK : (h->use_tc_select ? key_prep(h, t->keys0, t->keys1, h->st_run) : normalise_keys(h, t->keys0, t->keys1, h->st_run));
    if (rc) return rc;

    const int ab = act_bytes(c.act_dtype);
    const int64_t HK = static_cast<int64_t>(c.num_heads) * c.top_k;
    const int64_t chunk = blocking ? h->host_chunk : c.max_tokens;
    for (int64_t t0 = 0; t0 < n_tokens; t0 += chunk, ++h->host_slices) {
        const int64_t i = h->host_slices;          // counts across calls: a call may start while the previous one drains
        const int b = static_cast<int>(i & 1);
        const int64_t n = n_tokens - t0 < chunk ? n_tokens - t0 : chunk;
        // x staging buffer b is free once the kernels of slice i-2 are done
        if (i >= 2) CU_TRY(h, cudaStreamWaitEvent(h->st_in, h->ev_run[b], 0));
        CU_TRY(h, cudaMemcpyAsync(h->d_x[b], static_cast<const char*>(t->x) + t0 * c.input_dim * ab,
                                  static_cast<size_t>(n) * c.input_dim * ab, cudaMemcpyHostToDevice, h->st_in));
        CU_TRY(h, cudaEventRecord(h->ev_in[b], h->st_in));
        CU_TRY(h, cudaStreamWaitEvent(h->st_run, h->ev_in[b], 0));
        // out staging buffer b is free once slice i-2 has been copied out
        if (i >= 2) CU_TRY(h, cudaStreamWaitEvent(h->st_run, h->ev_out[b], 0));
        rc = forward_slice(h, t, h->d_x[b], h->d_out[b], want_ids ? h->d_ids[b] : nullptr,
                           want_ids ? h->d_sc[b] : nullptr, n, h->st_run);
        if (rc) return rc;
        CU_TRY(h, cudaEventRecord(h->ev_run[b], h->st_run));
        CU_TRY(h, cudaStreamWaitEvent(h->st_out, h->ev_run[b], 0));
        CU_TRY(h, cudaMemcpyAsync(static_cast<char*>(t->out) + t0 * c.output_dim * ab, h->d_out[b],
                                  static_cast<size_t>(n) * c.output_dim * ab, cudaMemcpyDeviceToHost, h->st_out));
        if (t->ids_out)
            CU_TRY(h, cudaMemcpyAsync(t->ids_out + t0 * HK, h->d_ids[b], static_cast<size_t>(n) * HK * sizeof(int64_t),
                                      cudaMemcpyDeviceToHost, h->st_out));
        if (t->scores_out)
            CU_TRY(h, cudaMemcpyAsync(t->scores_out + t0 * HK, h->d_sc[b], static_cast<size_t>(n) * HK * sizeof(float),
                                      cudaMemcpyDeviceToHost, h->st_out));
        CU_TRY(h, cudaEventRecord(h->ev_out[b], h->st_out));
    }
    cudaEvent_t& done = h->ev_call[h->host_calls & 7];
    if (!done) CU_TRY(h, cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
    CU_TRY(h, cudaEventRecord(done, h->st_out));
    if (ticket) *ticket = h->host_calls;
    ++h->host_calls;
    return PEER_OK;
}

extern "C" int peer_forward_host_wait(peer_handle_t h, int64_t ticket) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (ticket < 0 || ticket >= h->host_calls) return fail(h, PEER_ERR_INVALID_ARG, "no such call: ticket %lld", static_cast<long long>(ticket));
    if (ticket + 8 <= h->host_calls) {             // its event has been reused: everything up to now covers it
        CU_TRY(h, cudaStreamSynchronize(h->st_out));
        return PEER_OK;
    }
    CU_TRY(h, cudaEventSynchronize(h->ev_call[ticket & 7]));
    return PEER_OK;
}

extern "C" int peer_forward_host_async(peer_handle_t h, const peer_tensors_t* t, int64_t n_tokens, int64_t* ticket) {
    return host_submit(h, t, n_tokens, ticket, false);
}

extern "C" int peer_forward_host(peer_handle_t h, const peer_tensors_t* t, int64_t n_tokens) {
    int64_t ticket = 0;
    const int rc = host_submit(h, t, n_tokens, &ticket, true);
    if (rc) return rc;
    return peer_forward_host_wait(h, ticket);
}

extern "C" int peer_project_queries(peer_handle_t h, const peer_tensors_t* t, int64_t n_tokens,
                                    float* queries_out, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens == 0) return PEER_OK;
    if (!queries_out) return fail(h, PEER_ERR_INVALID_ARG, "queries_out is null");
    int rc = check_tensors(h, t, false);
    if (rc) return rc;
    const peer_config_t& c = h->cfg;
    QueryArgs q{};
    q.x = t->x; q.w = t->query_w; q.b = t->query_b; q.ln_w = t->ln_w; q.ln_b = t->ln_b;
    q.q_ln_out = queries_out; q.q_hat_out = nullptr; q.T = n_tokens; q.D = c.input_dim; q.H = c.num_heads;
    q.Q = c.query_dim; q.layer_norm = c.layer_norm; q.norm_query = c.norm_query; q.act_dtype = c.act_dtype;
    if (h->use_tc)
        CU_TRY(h, launch_query_tc(q, nullptr, 0, h->status, h->sm_count, static_cast<cudaStream_t>(stream)));
    else
        CU_TRY(h, launch_query_simt(q, static_cast<cudaStream_t>(stream)));
    h->launches += 1;
    return PEER_OK;
}

extern "C" int peer_select(peer_handle_t h, const float* queries, const void* keys0, const void* keys1,
                           int64_t n_tokens, int64_t* ids_out, float* scores_out, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens == 0) return PEER_OK;
    if (!queries || !keys0 || !keys1) return fail(h, PEER_ERR_INVALID_ARG, "queries and keys are required");
    if (h->general_select)
        return fail(h, PEER_ERR_UNSUPPORTED, "peer_select takes two sub-key tables; this layer has %d key dimensions: use peer_select_nd", h->nd);
    const peer_config_t& c = h->cfg;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = h->use_tc_select ? key_prep(h, keys0, keys1, s) : normalise_keys(h, keys0, keys1, s);
    if (rc) return rc;
    const int64_t HK = static_cast<int64_t>(c.num_heads) * c.top_k;
    const int64_t HQ = static_cast<int64_t>(c.num_heads) * c.query_dim;
    for (int64_t t0 = 0; t0 < n_tokens; t0 += c.max_tokens) {
        const int64_t n = n_tokens - t0 < c.max_tokens ? n_tokens - t0 : c.max_tokens;
        if (h->use_tc_select) {
            // the same kernels the whole layer runs: the given fp32 queries are normalised and split into the
            // three bf16 terms the tensor-core kernel contracts
            CU_TRY(h, launch_normalize_halves(queries + t0 * HQ, n * c.num_heads, c.query_dim, c.norm_query, nullptr, s,
                                              h->q_split, c.max_tokens * HQ));
            rc = select_tc_slice(h, keys0, keys1, n, nullptr, nullptr, ids_out ? ids_out + t0 * HK : nullptr,
                                 scores_out ? scores_out + t0 * HK : nullptr, nullptr, s);
            if (rc) return rc;
            h->launches += 3;
            continue;
        }
        CU_TRY(h, launch_normalize_halves(queries + t0 * HQ, n * c.num_heads, c.query_dim, c.norm_query, h->q_hat, s));
        SelectArgs sa = select_args(h, n);
        sa.ids64 = ids_out ? ids_out + t0 * HK : nullptr;
        sa.raw_scores = scores_out ? scores_out + t0 * HK : nullptr;
        CU_TRY(h, launch_select_simt(sa, s));
        h->launches += 2;
    }
    return PEER_OK;
}

extern "C" int peer_select_tokens(peer_handle_t h, const peer_tensors_t* t, int64_t n_tokens, int32_t* ids_out,
                                  float* weights_out, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens < 0) return fail(h, PEER_ERR_INVALID_ARG, "negative token count");
    if (n_tokens == 0) return PEER_OK;
    if (!ids_out || !weights_out) return fail(h, PEER_ERR_INVALID_ARG, "peer_select_tokens: ids_out and weights_out are required");
    int rc = check_tensors(h, t, false);
    if (rc) return rc;
    const peer_config_t& c = h->cfg;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rc = h->general_select ? PEER_OK : (h->use_tc_select ? key_prep(h, t->keys0, t->keys1, s) : normalise_keys(h, t->keys0, t->keys1, s));
    if (rc) return rc;
    const int ab = act_bytes(c.act_dtype);
    const int64_t HK = static_cast<int64_t>(c.num_heads) * c.top_k;
    for (int64_t t0 = 0; t0 < n_tokens; t0 += c.max_tokens) {
        const int64_t n = n_tokens - t0 < c.max_tokens ? n_tokens - t0 : c.max_tokens;
        rc = forward_slice(h, t, static_cast<const char*>(t->x) + t0 * c.input_dim * ab, nullptr,
                           t->ids_out ? t->ids_out + t0 * HK : nullptr, t->scores_out ? t->scores_out + t0 * HK : nullptr,
                           n, s, nullptr, nullptr, ids_out + t0 * HK, weights_out + t0 * HK);
        if (rc) return rc;
    }
    return PEER_OK;
}

extern "C" int peer_route_tuples(const int32_t* ids, const float* weights, int64_t n_tokens, int32_t entries_per_token,
                                 int64_t rows_per_rank, int32_t world, int32_t* send, void* stream) {
    if (!ids || !weights || !send || n_tokens < 0) {
        peer::set_global_error("peer_route_tuples: null pointer or negative token count");
        return PEER_ERR_INVALID_ARG;
    }
    const cudaError_t e = launch_route_tuples(ids, weights, n_tokens, entries_per_token, rows_per_rank, world, send,
                                              static_cast<cudaStream_t>(stream));
    if (e == cudaErrorInvalidValue) {
        peer::set_global_error("peer_route_tuples: world, rows_per_rank and entries_per_token must be positive");
        return PEER_ERR_INVALID_ARG;
    }
    if (e != cudaSuccess) { peer::set_global_error(cudaGetErrorString(e)); return PEER_ERR_CUDA; }
    return PEER_OK;
}

extern "C" int peer_gather_eval_routed(peer_handle_t h, const void* x, const int32_t* recv, int32_t world,
                                       int64_t tokens_per_rank, const void* expert_down, const void* expert_up,
                                       const float* down_scale, const float* up_scale, int64_t n_local_rows,
                                       float* out_f32, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    const peer_config_t& c = h->cfg;
    if (!x || !recv || !expert_down || !expert_up || !out_f32)
        return fail(h, PEER_ERR_INVALID_ARG, "peer_gather_eval_routed: null pointer");
    if (world < 1 || tokens_per_rank < 0 || n_local_rows <= 0 || n_local_rows > c.num_experts)
        return fail(h, PEER_ERR_INVALID_ARG, "peer_gather_eval_routed: world >= 1, tokens_per_rank >= 0, 0 < rows <= num_experts");
    if (tokens_per_rank == 0) return PEER_OK;
    if (h->hidden > 1 || c.act_dtype == PEER_DTYPE_F16)
        return fail(h, PEER_ERR_UNSUPPORTED, "peer_gather_eval_routed: experts with several neurons and fp16 layers are not implemented");
    if (c.table_dtype == PEER_DTYPE_E4M3 && (!down_scale || !up_scale))
        return fail(h, PEER_ERR_INVALID_ARG, "FP8 tables need down_scale and up_scale");
    if (!aligned16(x) || !aligned16(expert_down) || !aligned16(expert_up) || !aligned16(out_f32))
        return fail(h, PEER_ERR_INVALID_ARG, "x, tables and out must be 16-byte aligned");
    const int64_t E = static_cast<int64_t>(c.num_heads) * c.top_k;
    GatherArgs g{};
    g.x = x; g.ids = recv; g.weights = reinterpret_cast<const float*>(recv + tokens_per_rank * E);
    g.counts = recv + 2 * tokens_per_rank * E;
    g.block_tokens = tokens_per_rank; g.block_stride = 2 * tokens_per_rank * E + tokens_per_rank;
    g.down = expert_down; g.up = expert_up; g.down_scale = down_scale; g.up_scale = up_scale;
    g.out = out_f32; g.out_f32 = out_f32; g.T = tokens_per_rank * world; g.HK = static_cast<int>(E); g.N = n_local_rows;
    g.D = c.input_dim; g.Dout = c.output_dim; g.act_dtype = c.act_dtype; g.table_dtype = c.table_dtype;
    g.activation = c.activation; g.status = h->status; g.sm_count = h->sm_count;
    cudaError_t e = launch_gather_eval(g, static_cast<cudaStream_t>(stream));
    if (e == cudaErrorInvalidValue)
        return fail(h, PEER_ERR_UNSUPPORTED, "expert stage: row width %d/%d with this table dtype, or %d entries per token, is not implemented",
                    c.input_dim, c.output_dim, static_cast<int>(E));
    CU_TRY(h, e);
    h->launches += 1;
    return PEER_OK;
}

extern "C" int peer_select_stats(peer_handle_t h, int64_t* pooled_lists, int64_t* refined_rows, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    unsigned long long v[2] = {0, 0};
    if (h->sel_stats) {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        CU_TRY(h, cudaMemcpyAsync(v, h->sel_stats, sizeof v, cudaMemcpyDeviceToHost, s));
        CU_TRY(h, cudaMemsetAsync(h->sel_stats, 0, sizeof v, s));
        CU_TRY(h, cudaStreamSynchronize(s));
    }
    if (pooled_lists) *pooled_lists = static_cast<int64_t>(v[0]);
    if (refined_rows) *refined_rows = static_cast<int64_t>(v[1]);
    return PEER_OK;
}

extern "C" int peer_select_nd(peer_handle_t h, const float* queries, const void* const* keys, int64_t n_tokens,
                              int64_t* ids_out, float* scores_out, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens == 0) return PEER_OK;
    if (!queries || !keys) return fail(h, PEER_ERR_INVALID_ARG, "queries and keys are required");
    const peer_config_t& c = h->cfg;
    SelectNdArgs na{};
    na.q_ln = queries;
    for (int d = 0; d < h->nd; ++d) {
        if (!keys[d]) return fail(h, PEER_ERR_INVALID_ARG, "sub-key table %d is null", d);
        na.keys[d] = keys[d]; na.n[d] = h->n[d]; na.kp[d] = h->kp[d]; na.mult[d] = h->mult[d];
    }
    na.nd = h->nd; na.Q = c.query_dim; na.k = c.top_k; na.norm_keys = c.norm_keys; na.norm_query = c.norm_query;
    na.act_dtype = c.act_dtype; na.rows = n_tokens * c.num_heads;
    na.ids64 = ids_out; na.raw_scores = scores_out;
    cudaError_t e = launch_select_nd(na, static_cast<cudaStream_t>(stream));
    if (e == cudaErrorInvalidValue) return fail(h, PEER_ERR_UNSUPPORTED, "selection over this key grid is not implemented");
    CU_TRY(h, e);
    h->launches += 1;
    return PEER_OK;
}

extern "C" int peer_select_backward(peer_handle_t h, const float* queries, const void* const* keys,
                                    const int32_t* product_ids, const float* scores, const float* grad_weights,
                                    int64_t n_tokens, float* grad_queries, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens == 0) return PEER_OK;
    if (!queries || !keys || !product_ids || !scores || !grad_weights || !grad_queries)
        return fail(h, PEER_ERR_INVALID_ARG, "peer_select_backward: null pointer");
    const peer_config_t& c = h->cfg;
    SelectGradArgs ga{};
    ga.q_ln = queries;
    for (int d = 0; d < h->nd; ++d) {
        if (!keys[d]) return fail(h, PEER_ERR_INVALID_ARG, "sub-key table %d is null", d);
        ga.keys[d] = keys[d]; ga.n[d] = h->n[d];
    }
    ga.stride[h->nd - 1] = 1;
    for (int d = h->nd - 2; d >= 0; --d) ga.stride[d] = ga.stride[d + 1] * h->n[d + 1];
    ga.nd = h->nd; ga.Q = c.query_dim; ga.k = c.top_k; ga.norm_keys = c.norm_keys; ga.norm_query = c.norm_query;
    ga.act_dtype = c.act_dtype; ga.rows = n_tokens * c.num_heads;
    ga.prod_ids = product_ids; ga.scores = scores; ga.grad_weights = grad_weights; ga.grad_q = grad_queries;
    ga.status = h->status;
    cudaError_t e = launch_select_grad(ga, static_cast<cudaStream_t>(stream));
    if (e == cudaErrorInvalidValue) return fail(h, PEER_ERR_UNSUPPORTED, "score-path backward: this key grid is not implemented");
    CU_TRY(h, e);
    h->launches += 1;
    return PEER_OK;
}

extern "C" int peer_gather_eval(peer_handle_t h, const void* x, const int32_t* ids, const float* weights,
                                const void* expert_down, const void* expert_up, const float* down_scale,
                                const float* up_scale, void* out, int64_t n_tokens, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens == 0) return PEER_OK;
    const peer_config_t& c = h->cfg;
    if (!x || !ids || !weights || !expert_down || !expert_up || !out)
        return fail(h, PEER_ERR_INVALID_ARG, "peer_gather_eval: null pointer");
    if (c.table_dtype == PEER_DTYPE_E4M3 && (!down_scale || !up_scale))
        return fail(h, PEER_ERR_INVALID_ARG, "FP8 tables need down_scale and up_scale");
    if (!aligned16(x) || !aligned16(expert_down) || !aligned16(expert_up) || !aligned16(out))
        return fail(h, PEER_ERR_INVALID_ARG, "x, tables and out must be 16-byte aligned");
    GatherArgs g{};
    g.x = x; g.ids = ids; g.weights = weights; g.down = expert_down; g.up = expert_up;
    g.down_scale = down_scale; g.up_scale = up_scale; g.out = out; g.T = n_tokens;
    g.HK = c.num_heads * c.top_k; g.N = c.num_experts; g.D = c.input_dim; g.Dout = c.output_dim;
    g.act_dtype = c.act_dtype; g.table_dtype = c.table_dtype; g.activation = c.activation;
    g.status = h->status; g.sm_count = h->sm_count; g.hidden = h->hidden;
    const bool general_rows = h->hidden > 1 || c.act_dtype == PEER_DTYPE_F16;
    if (general_rows && g.hidden < 1) g.hidden = 1;
    cudaError_t e = general_rows ? launch_gather_hidden(g, static_cast<cudaStream_t>(stream))
                                 : launch_gather_eval(g, static_cast<cudaStream_t>(stream));
    if (e == cudaErrorInvalidValue)
        return fail(h, PEER_ERR_UNSUPPORTED, "expert stage: row width %d/%d with this table dtype, or num_heads*top_k=%d, is not implemented",
                    c.input_dim, c.output_dim, g.HK);
    CU_TRY(h, e);
    h->launches += 1;
    return PEER_OK;
}

extern "C" int peer_gather_eval_partial(peer_handle_t h, const void* x, const int32_t* ids, const float* weights,
                                        const int32_t* counts, int32_t entries_per_token, const void* expert_down,
                                        const void* expert_up, const float* down_scale, const float* up_scale,
                                        int64_t n_local_rows, float* out_f32, int64_t n_tokens, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens == 0) return PEER_OK;
    const peer_config_t& c = h->cfg;
    if (!x || !ids || !weights || !counts || !expert_down || !expert_up || !out_f32)
        return fail(h, PEER_ERR_INVALID_ARG, "peer_gather_eval_partial: null pointer");
    if (h->hidden > 1 || c.act_dtype == PEER_DTYPE_F16)
        return fail(h, PEER_ERR_UNSUPPORTED, "peer_gather_eval_partial: experts with several neurons and fp16 layers are not implemented");
    if (entries_per_token <= 0 || n_local_rows <= 0 || n_local_rows > c.num_experts)
        return fail(h, PEER_ERR_INVALID_ARG, "peer_gather_eval_partial: entries_per_token and n_local_rows must be positive, rows <= num_experts");
    if (c.table_dtype == PEER_DTYPE_E4M3 && (!down_scale || !up_scale))
        return fail(h, PEER_ERR_INVALID_ARG, "FP8 tables need down_scale and up_scale");
    if (!aligned16(x) || !aligned16(expert_down) || !aligned16(expert_up) || !aligned16(out_f32))
        return fail(h, PEER_ERR_INVALID_ARG, "x, tables and out must be 16-byte aligned");
    GatherArgs g{};
    g.x = x; g.ids = ids; g.weights = weights; g.down = expert_down; g.up = expert_up;
    g.down_scale = down_scale; g.up_scale = up_scale; g.out = out_f32; g.out_f32 = out_f32; g.counts = counts;
    g.T = n_tokens; g.HK = entries_per_token; g.N = n_local_rows; g.D = c.input_dim; g.Dout = c.output_dim;
    g.act_dtype = c.act_dtype; g.table_dtype = c.table_dtype; g.activation = c.activation;
    g.status = h->status; g.sm_count = h->sm_count;
    cudaError_t e = launch_gather_eval(g, static_cast<cudaStream_t>(stream));
    if (e == cudaErrorInvalidValue)
        return fail(h, PEER_ERR_UNSUPPORTED, "expert stage: row width %d/%d with this table dtype, or %d entries per token, is not implemented",
                    c.input_dim, c.output_dim, entries_per_token);
    CU_TRY(h, e);
    h->launches += 1;
    return PEER_OK;
}

extern "C" int peer_gather_eval_backward_rows(peer_handle_t h, const void* x, const void* grad_out, const int32_t* ids,
                                              const float* weights, const void* expert_down, const void* expert_up,
                                              float* grad_x, float* grad_weights, void* grad_down, void* grad_up,
                                              int32_t grad_table_dtype, int64_t n_grad_rows, int64_t n_tokens, void* stream);

extern "C" int peer_gather_eval_backward(peer_handle_t h, const void* x, const void* grad_out, const int32_t* ids,
                                         const float* weights, const void* expert_down, const void* expert_up,
                                         float* grad_x, float* grad_weights, void* grad_down, void* grad_up,
                                         int32_t grad_table_dtype, int64_t n_tokens, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    return peer_gather_eval_backward_rows(h, x, grad_out, ids, weights, expert_down, expert_up, grad_x, grad_weights,
                                          grad_down, grad_up, grad_table_dtype, h->cfg.num_experts, n_tokens, stream);
}

extern "C" int peer_gather_eval_backward_rows(peer_handle_t h, const void* x, const void* grad_out, const int32_t* ids,
                                              const float* weights, const void* expert_down, const void* expert_up,
                                              float* grad_x, float* grad_weights, void* grad_down, void* grad_up,
                                              int32_t grad_table_dtype, int64_t n_grad_rows, int64_t n_tokens, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    if (n_tokens == 0) return PEER_OK;
    if (n_grad_rows <= 0 || n_grad_rows > h->cfg.num_experts)
        return fail(h, PEER_ERR_INVALID_ARG, "peer_gather_eval_backward_rows: n_grad_rows must lie in [1, num_experts]");
    const peer_config_t& c = h->cfg;
    if (!x || !grad_out || !ids || !weights || !expert_down || !expert_up || !grad_x || !grad_weights || !grad_down || !grad_up)
        return fail(h, PEER_ERR_INVALID_ARG, "peer_gather_eval_backward: null pointer");
    if (c.table_dtype != c.act_dtype)
        return fail(h, PEER_ERR_UNSUPPORTED, "backward needs tables in the layer's dtype (fp32 or bf16); quantised tables are inference-only");
    if (grad_table_dtype != PEER_DTYPE_F32 && (grad_table_dtype != c.table_dtype || h->hidden > 1))
        return fail(h, PEER_ERR_UNSUPPORTED, "table gradients are accumulated in fp32, or (single-neuron experts) in the tables' own dtype");
    if (!aligned16(x) || !aligned16(grad_out) || !aligned16(expert_down) || !aligned16(expert_up) || !aligned16(grad_x) ||
        !aligned16(grad_down) || !aligned16(grad_up))
        return fail(h, PEER_ERR_INVALID_ARG, "x, grad_out, tables and gradient buffers must be 16-byte aligned");
    GatherGradArgs g{};
    g.x = x; g.dy = grad_out; g.ids = ids; g.weights = weights; g.down = expert_down; g.up = expert_up;
    g.d_down = grad_down; g.d_up = grad_up; g.dx = grad_x; g.dweights = grad_weights;
    g.T = n_tokens; g.HK = c.num_heads * c.top_k; g.N = n_grad_rows; g.D = c.input_dim; g.Dout = c.output_dim;
    g.act_dtype = c.act_dtype; g.table_dtype = c.table_dtype; g.activation = c.activation;
    g.status = h->status; g.sm_count = h->sm_count; g.hidden = h->hidden; g.grad_dtype = grad_table_dtype;
    // rows longer than 4 KB do not fit the register-resident kernel: the general kernel takes them (fp32 sums)
    const int row_bytes = (c.input_dim > c.output_dim ? c.input_dim : c.output_dim) * act_bytes(c.table_dtype);
    const bool general = h->hidden > 1 || row_bytes > 4096 || c.act_dtype == PEER_DTYPE_F16;
    if (general && grad_table_dtype != PEER_DTYPE_F32)
        return fail(h, PEER_ERR_UNSUPPORTED, "table gradients of rows longer than 4 KB are accumulated in fp32");
    if (general && g.hidden < 1) g.hidden = 1;
    cudaError_t e = general ? launch_gather_hidden_grad(g, static_cast<cudaStream_t>(stream))
                            : launch_gather_grad(g, static_cast<cudaStream_t>(stream));
    if (e == cudaErrorInvalidValue)
        return fail(h, PEER_ERR_UNSUPPORTED, "expert backward: row width %d/%d is not implemented for this dtype (bf16 up to 2048, fp32 up to 1024)",
                    c.input_dim, c.output_dim);
    CU_TRY(h, e);
    h->launches += 1;
    return PEER_OK;
}

extern "C" int peer_query_status(peer_handle_t h, void* stream) {
    if (!h) return PEER_ERR_INVALID_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int st = 0;
    CU_TRY(h, cudaMemcpyAsync(&st, h->status, sizeof(int), cudaMemcpyDeviceToHost, s));
    CU_TRY(h, cudaMemsetAsync(h->status, 0, sizeof(int), s));
    CU_TRY(h, cudaStreamSynchronize(s));
    if (st == STATUS_TIMEOUT) return fail(h, PEER_ERR_DEVICE_TIMEOUT, "a bounded device-side wait ran out");
    if (st == STATUS_BOUNDS) return fail(h, PEER_ERR_BOUNDS, "an expert id outside [0, num_experts) (or a grid position outside the key grid) was skipped");
    return PEER_OK;
}
