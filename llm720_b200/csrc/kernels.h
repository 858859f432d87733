// Internal launch interface between the C ABI (peer_api.cu) and the kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace peer {

// Largest number of (a, b) candidate pairs the combine step examines
// (pairs with (a+1)(b+1) <= k for k <= 32 number at most 119).
constexpr int MAX_PAIRS = 128;

struct QueryArgs {
    const void* x;        // [T, D] act dtype
    const void* w;        // [H*Q, D] act dtype
    const void* b;        // [H*Q] or null
    const void* ln_w;     // [Q] or null (=1)
    const void* ln_b;     // [Q] or null (=0)
    float* q_ln_out;      // optional [T, H, Q]: queries after LayerNorm
    float* q_hat_out;     // optional [T, H, Q]: halves L2-normalised
    int64_t T;
    int D, H, Q;
    int layer_norm, norm_query;
    int act_dtype;
};
cudaError_t launch_query_simt(const QueryArgs& a, cudaStream_t s);

// Tensor-core (tcgen05) query stage for bf16 layers.  Besides the optional fp32 outputs of
// QueryArgs it writes the normalised queries as three bf16 terms (hi, mid, lo), each a
// [T, H, Q] array, `split_stride` elements apart.
bool query_tc_supported(const QueryArgs& a);
cudaError_t query_tc_setup();
cudaError_t launch_query_tc(const QueryArgs& a, __nv_bfloat16* split_out, int64_t split_stride, int* status,
                            int sm_count, cudaStream_t s);

// Tensor-core (tcgen05) selection for bf16 layers: same results as launch_select_simt.
struct SelectTcArgs {
    const __nv_bfloat16* q_split;  // [3][term_rows, Q]: hi/mid/lo terms of the normalised queries
    int64_t term_rows;             // rows between the three term arrays (>= rows)
    const void* keys0;             // [n0, Q/2] bf16, as stored (not normalised)
    const void* keys1;             // [n1, Q/2]
    const float* invn0;            // [n0] 1/||key|| (or 1)
    const float* invn1;            // [n1]
    int64_t rows;                  // T * H
    int Q, n0, n1, kp0, kp1, k, mult0, mult1;
    int32_t* ids32; float* weights; int64_t* ids64; float* raw_scores;   // as in SelectArgs
    int32_t* prod_ids;        // optional [rows, k]: i0 * n1 + i1 whatever mult0/mult1 say
    int* status;
    int sm_count;
    int32_t* overflow_rows;        // [rows]: rows the kernel leaves to the exact kernel (clustered scores)
    int* overflow_count;           // device counter, zeroed by the caller before the launch
    unsigned long long* stats;     // optional [2], accumulated: row-halves whose candidate list continued in the
                                   // pool; rows handed to the exact kernel
    // optional (both or none; only for layers that normalise their queries): the first pass leaves out the
    // query's lo term.  eps0/1: device scalars, the most a score can lose by that (from launch_key_prep)
    const float* eps0; const float* eps1;
};
bool select_tc_supported(int act_dtype, int Q, int n0, int n1, int k, int kp0, int kp1);
cudaError_t select_tc_setup();
cudaError_t launch_select_tc(const SelectTcArgs& a, cudaStream_t s);
// Both bf16 sub-key tables in one launch: invn[j] = 1 / max(||key_j||, 1e-12) (or 1 when !do_norm), khat = the
// normalised keys in fp32, transposed [width, n] (what launch_normalize_rows writes with transpose_out), and with
// eps (a device pair, zeroed here) the error bounds of the select kernel's two-term first pass, one per table
cudaError_t launch_key_prep(const void* keys0, const void* keys1, int n0, int n1, int width, int do_norm, float* khat0,
                            float* khat1, float* invn0, float* invn1, float* eps, cudaStream_t s);

// rows of `width` elements -> fp32, each row divided by max(||row||, 1e-12) when do_norm;
// written [rows, width], or [width, rows] when transpose_out
cudaError_t launch_normalize_rows(const void* in, int in_dtype, int64_t rows, int width, int do_norm,
                                  int transpose_out, float* out, cudaStream_t s);
// [rows, Q] fp32 -> both halves of every row L2-normalised, as fp32 (`out`, optional) and/or as the three
// bf16 terms hi/mid/lo the tensor-core select kernel takes (`split`, optional; arrays split_stride apart)
cudaError_t launch_normalize_halves(const float* q, int64_t rows, int Q, int do_norm, float* out,
                                    cudaStream_t s, __nv_bfloat16* split = nullptr, int64_t split_stride = 0);

struct SelectArgs {
    const float* q_hat;   // [rows, Q] fp32, halves normalised
    const float* khat0;   // [Q/2, n0] fp32: normalised sub-keys, transposed
    const float* khat1;   // [Q/2, n1] fp32
    int64_t rows;         // T * H
    int Q, n0, n1;
    int kp0, kp1;         // candidates kept per half
    int k;                // final top-k
    int mult0, mult1;     // flat id = i0*mult0 + i1*mult1
    const uint16_t* pairs;// device [n_pairs]: (a << 8) | b, candidate pairs of the combine step
    int n_pairs;
    int32_t* ids32;       // optional [rows, k]
    float* weights;       // optional [rows, k] softmax over k
    int64_t* ids64;       // optional [rows, k]
    float* raw_scores;    // optional [rows, k]
    int32_t* prod_ids;    // optional [rows, k]: i0 * n1 + i1 whatever mult0/mult1 say
    // optional: process only the rows row_list[0 .. *row_count) (device memory), and/or take the
    // normalised queries as the sum of three bf16 terms split_stride elements apart
    const int32_t* row_list;
    const int* row_count;
    const __nv_bfloat16* q_split;
    int64_t split_stride;
};
cudaError_t launch_select_simt(const SelectArgs& a, cudaStream_t s);

struct GatherArgs {
    const void* x;            // [T, D] act dtype
    const int32_t* ids;       // [T, HK]
    const float* weights;     // [T, HK]
    const void* down;         // [N, D] table dtype
    const void* up;           // [N, Dout]
    const float* down_scale;  // [N] or null
    const float* up_scale;    // [N] or null
    void* out;                // [T, Dout] act dtype
    int64_t T;
    int HK;
    int64_t N;
    int D, Dout;
    int act_dtype, table_dtype, activation;
    int* status;              // device status word
    int sm_count;
    int hidden;               // neurons per expert (rows are [hidden, D] / [Dout, hidden] blocks); 0 or 1 = single
    const void* residual;     // optional [T, Dout] act dtype: added to the result (out = residual + y)
    int rows_l2_resident;     // hint: the ids address so few rows that they stay in L2 (reference id arithmetic)
    const int32_t* counts;    // optional [T]: how many of token t's HK entries are in use
    float* out_f32;           // optional fp32 output [T, Dout] (partial sums of a row-sharded table)
    // optional: ids / weights / counts are blocks as received from the ranks of an expert-parallel layer (route.cu):
    // token t's entries start at ids[(t / block_tokens) * block_stride + (t % block_tokens) * HK] (same for weights),
    // its count is counts[(t / block_tokens) * block_stride + t % block_tokens]; 0 = plain [T, HK] arrays
    int64_t block_tokens, block_stride;
    // optional tiered residency: row_map [N] int32 on the device; row_map[id] >= 0: the row is that slot of
    // cache_down / cache_up (HBM); < 0: it is read in place from down / up, which then point at host memory the GPU
    // can address (pinned, unified addressing)
    const int32_t* row_map;
    const void* cache_down;
    const void* cache_up;
};
cudaError_t launch_gather_eval(const GatherArgs& a, cudaStream_t s);

// Backward of the expert evaluation (gather_grad.cu): fp32 or bf16 layers with tables of the same dtype.
struct GatherGradArgs {
    const void* x;            // [T, D] act dtype
    const void* dy;           // [T, Dout] act dtype
    const int32_t* ids;       // [T, HK]
    const float* weights;     // [T, HK]
    const void* down;         // [N, D]
    const void* up;           // [N, Dout]
    void* d_down;             // [N, D] fp32 (or grad_dtype), accumulated into
    void* d_up;               // [N, Dout] fp32 (or grad_dtype), accumulated into
    float* dx;                // [T, D] fp32, written
    float* dweights;          // [T, HK] fp32, written
    int64_t T;
    int HK;
    int64_t N;
    int D, Dout;
    int act_dtype, table_dtype, activation;
    int* status;
    int sm_count;
    int hidden;               // neurons per expert; 0 or 1 = single
    int grad_dtype;           // dtype of d_down / d_up: PEER_DTYPE_F32, or the tables' own 16-bit type
};
cudaError_t launch_gather_grad(const GatherGradArgs& a, cudaStream_t s);

// Experts with several hidden neurons (gather_hidden.cu): forward and backward, fp32 or bf16 layers
// with tables of the same dtype.
cudaError_t launch_gather_hidden(const GatherArgs& a, cudaStream_t s);
cudaError_t launch_gather_hidden_grad(const GatherGradArgs& a, cudaStream_t s);

// Product-key selection over 1 to 4 key dimensions (select_nd.cu).
struct SelectNdArgs {
    const float* q_ln;        // [rows, Q] fp32 queries after LayerNorm
    const void* keys[4];      // [n[d], Q/nd] act dtype, as stored
    int n[4];
    int kp[4];                // candidates kept per dimension (<= 32)
    long long mult[4];        // flat id = sum_d index_d * mult[d]
    int nd, Q, k;
    int norm_keys, norm_query, act_dtype;
    int64_t rows;
    int32_t* ids32;           // optional [rows, k]
    float* weights;           // optional [rows, k] softmax
    int64_t* ids64;           // optional [rows, k]
    float* raw_scores;        // optional [rows, k]
    int32_t* prod_ids;        // optional [rows, k]: sum_d index_d * stride[d] (true row-major position in the key grid)
    long long stride[4];
};
cudaError_t launch_select_nd(const SelectNdArgs& a, cudaStream_t s);

// Backward of the selected scores and their softmax with respect to the queries (select_grad.cu)
struct SelectGradArgs {
    const float* q_ln;          // [rows, Q] fp32 queries after LayerNorm
    const void* keys[4];        // [n[d], Q/nd] act dtype, as stored
    int n[4];
    long long stride[4];        // true row-major strides of the key grid
    int nd, Q, k;
    int norm_keys, norm_query, act_dtype;
    int64_t rows;
    const int32_t* prod_ids;    // [rows, k] grid positions of the selected experts
    const float* scores;        // [rows, k] raw scores of the forward pass
    const float* grad_weights;  // [rows, k] dL/d softmax weights
    float* grad_q;              // [rows, Q] written
    int* status;                // device status word: STATUS_BOUNDS when a grid position lies outside the key grid
};
cudaError_t launch_select_grad(const SelectGradArgs& a, cudaStream_t s);

// Tuple routing of the expert-parallel layer (route.cu): `send` is [world] blocks of int32, each
// [local row ids: T x E | weight bits: T x E | counts: T] for one destination rank.
cudaError_t launch_route_tuples(const int32_t* ids, const float* weights, int64_t n_tokens, int entries_per_token,
                                int64_t rows_per_rank, int world, int32_t* send, cudaStream_t s);

// LayerNorm over the model dimension, fp32 parameters (block_ln.cu)
cudaError_t launch_block_ln(const void* x, int act_dtype, int64_t rows, int D, const float* w, const float* b, float eps,
                            void* out, cudaStream_t s);
// one-time per-process attribute set-up (dynamic shared memory opt-in)
cudaError_t select_simt_setup();

}  // namespace peer
