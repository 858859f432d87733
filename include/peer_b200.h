/*
 * peer_b200 — C ABI of the B200 (sm_100a) PEER forward library.
 *
 * Every entry point takes plain device (or, where stated, pinned host)
 * pointers and sizes; no C++ or framework types cross this boundary.  The
 * caller owns every tensor, including the output; the library owns only the
 * per-handle scratch it allocates in peer_create (normalised sub-keys,
 * normalised queries, the selected (id, weight) tuples, a status word) and
 * frees in peer_destroy.  All work is enqueued on the stream the caller
 * passes; no entry point other than create/destroy/forward_host/query_status
 * synchronises.
 *
 * Each declaration names the interface of wrmedford/llm720 that it replaces
 * (paths relative to that project).
 */
#ifndef PEER_B200_H
#define PEER_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PEER_B200_ABI_VERSION 2

/* Return codes.  Nothing in this library falls back to another code path:
 * an unsupported configuration is an error. */
enum {
    PEER_OK = 0,
    PEER_ERR_INVALID_ARG = 1,   /* null pointer, bad size, misaligned pointer        */
    PEER_ERR_UNSUPPORTED = 2,   /* configuration outside what the kernels implement  */
    PEER_ERR_CUDA = 3,          /* a CUDA runtime call or launch failed              */
    PEER_ERR_DEVICE_TIMEOUT = 4,/* a bounded device-side wait ran out                */
    PEER_ERR_BOUNDS = 5         /* an expert id outside [0, num_experts) was seen    */
};

enum { PEER_DTYPE_F32 = 0, PEER_DTYPE_BF16 = 1, PEER_DTYPE_E4M3 = 2, PEER_DTYPE_F16 = 3 };
enum { PEER_ACT_GELU = 0, PEER_ACT_RELU = 1 };
/* How the two per-dimension sub-key indices (i0, i1) become a flat expert id.
 * REFERENCE: i0 + i1, what llm/models/experts.py:203-230 computes (the first
 * dimension never receives its multiplier).  PRODUCT: i0 * n_keys1 + i1. */
enum { PEER_INDEX_REFERENCE = 0, PEER_INDEX_PRODUCT = 1 };

/* Mirrors the constructor of the reference module, PEER.__init__
 * (llm/models/experts.py:46-61), and of the native operator
 * PEEROperatorEnhanced (llm/models/kernels/peer_cutlass.h:13-23). */
typedef struct peer_config {
    int32_t abi_version;        /* PEER_B200_ABI_VERSION                              */
    int32_t input_dim;
    int32_t output_dim;
    int64_t num_experts;        /* = n_keys0 * n_keys1                                */
    int32_t top_k;              /* num_experts_per_tok, <= 32                         */
    int32_t num_heads;
    int32_t query_dim;          /* per head, even, <= 256                             */
    int32_t n_keys0, n_keys1;   /* product_key_dim[0], [1]                            */
    int32_t expert_hidden_size; /* neurons per expert, 1..16 (experts.py:337-352: down rows are
                                   [h, input_dim] blocks, up rows [output_dim, h] blocks)           */
    int32_t activation;         /* PEER_ACT_*                                         */
    int32_t norm_keys, norm_query, layer_norm; /* booleans (batch_norm_query = layer_norm) */
    int32_t act_dtype;          /* dtype of x, out, query weights, LN affine, sub-keys: F32, BF16 or F16 */
    int32_t table_dtype;        /* dtype of expert_down / expert_up: F32, BF16, E4M3 (with BF16 activations)
                                   or F16 (with F16 activations; fp16 layers run the CUDA-core kernels) */
    int32_t index_mode;         /* PEER_INDEX_*                                       */
    int64_t max_tokens;         /* scratch capacity; longer inputs are processed in slices */
    int32_t num_key_dims;       /* len(product_key_dim): 1..4; 0 is read as 2         */
    int32_t n_keys2, n_keys3;   /* product_key_dim[2], [3] (read when num_key_dims says so) */
} peer_config_t;

/* Tensors of one forward call; all row-major and contiguous.
 * Mirrors the argument list of the pybind entry `peer_forward`
 * (llm/models/kernels/peer_cutlass_wrapper.cpp:65-88). */
typedef struct peer_tensors {
    const void*  x;            /* [T, input_dim]                 act_dtype            */
    const void*  query_w;      /* [num_heads*query_dim, input_dim] act_dtype          */
    const void*  query_b;      /* [num_heads*query_dim] or NULL  act_dtype            */
    const void*  ln_w;         /* [query_dim] or NULL            act_dtype            */
    const void*  ln_b;         /* [query_dim] or NULL            act_dtype            */
    const void*  keys0;        /* [n_keys0, query_dim/2]         act_dtype            */
    const void*  keys1;        /* [n_keys1, query_dim/2]         act_dtype            */
    const void*  expert_down;  /* [num_experts, input_dim]       table_dtype          */
    const void*  expert_up;    /* [num_experts, output_dim]      table_dtype          */
    const float* down_scale;   /* [num_experts] (E4M3 tables) else NULL               */
    const float* up_scale;     /* [num_experts] (E4M3 tables) else NULL               */
    void*        out;          /* [T, output_dim]                act_dtype            */
    int64_t*     ids_out;      /* optional [T, num_heads, top_k]: selected expert ids */
    float*       scores_out;   /* optional [T, num_heads, top_k]: raw (pre-softmax) scores */
    const void*  keys2;        /* [n_keys2, query_dim/num_key_dims] (3-D, 4-D key grids) */
    const void*  keys3;        /* [n_keys3, query_dim/num_key_dims] (4-D key grids)      */
    int32_t*     product_ids_out; /* optional [T, num_heads, top_k] (peer_forward only): the selected experts'
                                  true positions in the key grid, sum_d index_d * stride_d, whatever
                                  index_mode says; the backward pass needs the per-dimension indices */
} peer_tensors_t;

typedef struct peer_op* peer_handle_t;

/* Replaces the PEEROperatorEnhanced constructor + allocate_weights
 * (llm/models/kernels/peer_cutlass.cu:1178-1305) and the process-global
 * operator of peer_cutlass_wrapper.cpp:17-63.  One handle per module per
 * device; not thread-safe.  Allocates the scratch on the current device. */
int peer_create(const peer_config_t* cfg, peer_handle_t* out_handle);

/* Replaces ~PEEROperatorEnhanced. */
int peer_destroy(peer_handle_t h);

/* Text of the last error on this handle (or, when h is NULL, of the calling
 * thread's last failed peer_create / handle-free call).  Replaces the exceptions thrown at
 * peer_cutlass_wrapper.cpp:90-96 and peer_cutlass.cu:1388-1394. */
const char* peer_last_error(peer_handle_t h);

/* The whole layer on device buffers: replaces PEER.forward /
 * PEER._forward_pytorch (llm/models/experts.py:288-384, 422-440) and
 * PEEROperatorEnhanced::forward (peer_cutlass.cu:1307-1395).
 * Asynchronous on `stream` (a cudaStream_t). */
int peer_forward(peer_handle_t h, const peer_tensors_t* t, int64_t n_tokens, void* stream);

/* The feed-forward half of the reference's TransformerBlock.forward (llm/models/foundation.py:
 * 196-205) in one call: out = hidden + PEER(LayerNorm(hidden)), with t->x = hidden [T, input_dim]
 * (act_dtype) and the block's ln_2 parameters ln_w, ln_b (fp32 [input_dim], either may be NULL) and
 * eps.  The normalised rows go to library scratch (allocated on the first call), the residual is
 * added where the expert stage writes its result.  input_dim must equal output_dim; t->out may not
 * alias t->x.  Asynchronous on `stream`. */
int peer_block_forward(peer_handle_t h, const peer_tensors_t* t, const float* ln_w, const float* ln_b,
                       float ln_eps, int64_t n_tokens, void* stream);

/* Tiered residency of the expert tables, for tables larger than the GPU's memory: the role of the reference's
 * HierarchicalExpertCache (llm/models/kernels/peer_cutlass.cu:110-536; docs/MEMORY_HIERARCHY.md:5-11: HBM cache
 * in front of pinned host memory), without its background thread and per-call table copies.  After this call
 * the handle's forwards (peer_forward, peer_block_forward, peer_forward_host*) take t->expert_down / t->expert_up
 * as the FULL tables in host memory that the GPU can address (pinned; with unified addressing the host pointer is
 * the device pointer), and read a row from there only when row_map[id] < 0; a row with row_map[id] = s >= 0 is
 * read from row s of cache_down / cache_up in HBM through the usual bulk-copy rings.  row_map: int32
 * [num_experts] on the device; the caches: table_dtype, rows of input_dim / output_dim.  Per-row FP8 scales stay
 * whole on the device.  The three arrays are the caller's and must stay valid; which rows to cache is the
 * caller's policy (peer_usage_histogram gives the counts).  row_map = NULL switches back.  bf16 and FP8 tables
 * of single-neuron experts; inference only. */
int peer_set_row_tier(peer_handle_t h, const int32_t* row_map, const void* cache_down, const void* cache_up);

/* Same, with t->x and t->out (and the optional ids/scores outputs) in HOST
 * memory (pinned for full speed): token slices are copied in, processed and
 * copied out on three internal streams so transfers overlap the kernels.
 * Returns after the last slice has landed in t->out.  The call runs on the library's own streams: work
 * the caller enqueued earlier on another stream (an in-place weight update, say) must have completed
 * before the call.  Replaces the
 * host-tensor call path of peer_forward_cutlass
 * (llm/models/kernels/peer_cutlass.py:135-234). */
int peer_forward_host(peer_handle_t h, const peer_tensors_t* t, int64_t n_tokens);

/* The same call split in two, so that consecutive batches overlap: _async enqueues the copies and
 * kernels of one batch and returns a ticket; _wait blocks until that batch's outputs are complete in
 * host memory.  t->x must stay unchanged and t->out untouched until the wait; a later batch may be
 * submitted before an earlier one is waited for (its first copy-in then overlaps the earlier batch's
 * last copy-out), each with its own output buffer.  Tickets are waited in any order; at most 8 may be
 * outstanding. */
int peer_forward_host_async(peer_handle_t h, const peer_tensors_t* t, int64_t n_tokens, int64_t* ticket);
int peer_forward_host_wait(peer_handle_t h, int64_t ticket);

/* Stage entry points (used by the parity tests and by callers that need one
 * stage only). */

/* Query projection + shared LayerNorm: experts.py:302-308.  Writes the
 * queries after LayerNorm, fp32 [T, num_heads, query_dim]. */
int peer_project_queries(peer_handle_t h, const peer_tensors_t* t, int64_t n_tokens,
                         float* queries_out, void* stream);

/* Product-key retrieval from given queries: PEER._get_expert_indices_pytorch
 * (experts.py:138-285).  queries fp32 [T, num_heads, query_dim] (after
 * LayerNorm, before the per-half L2 normalisation, exactly what the
 * reference function receives).  Writes ids int64 and raw scores fp32,
 * both [T, num_heads, top_k], sorted by descending score.  Runs the kernels peer_forward runs for
 * this handle: the tensor-core selection on bf16 layers whose shape it covers (the given queries are
 * normalised and split into bf16 terms first), the CUDA-core selection otherwise. */
int peer_select(peer_handle_t h, const float* queries, const void* keys0, const void* keys1,
                int64_t n_tokens, int64_t* ids_out, float* scores_out, void* stream);

/* Counters of the tensor-core selection kernel's rare paths, accumulated since the last read (the
 * read clears them; synchronises `stream`): *pooled_lists = (row, query half) pairs whose candidate
 * list outgrew its 32 slots and continued in the shared pool; *refined_rows = rows that lost a
 * candidate there and were redone by the exact CUDA-core kernel.  Both stay 0 on layers that run the
 * CUDA-core selection.  The results never depend on these paths (each is exact); the counters let a
 * test prove that a given input really exercised them.  The reference has one selection routine
 * (PEER._get_expert_indices_pytorch, experts.py:138-285) and nothing to count. */
int peer_select_stats(peer_handle_t h, int64_t* pooled_lists, int64_t* refined_rows, void* stream);

/* Same retrieval for a key grid of any dimensionality (1 to 4; experts.py:195-270: the dimensions
 * are folded in one at a time and all but the last fold keep the best 4*top_k sums).  `keys` is an
 * array of num_key_dims device pointers, table d being [n_keys_d, query_dim/num_key_dims]. */
int peer_select_nd(peer_handle_t h, const float* queries, const void* const* keys, int64_t n_tokens,
                   int64_t* ids_out, float* scores_out, void* stream);

/* Expert evaluation from given selections: experts.py:327-382 with the
 * softmax already applied.  ids int32 and weights fp32, both
 * [T, num_heads*top_k]; out[t] = sum_j w[t,j] * act(down[ids[t,j]] . x[t]) * up[ids[t,j]]. */
int peer_gather_eval(peer_handle_t h, const void* x, const int32_t* ids, const float* weights,
                     const void* expert_down, const void* expert_up, const float* down_scale,
                     const float* up_scale, void* out, int64_t n_tokens, void* stream);

/* Expert evaluation against a ROW SHARD of the tables (expert-parallel layers): the caller holds
 * rows [r0, r0 + n_local_rows) of expert_down / expert_up, `ids` are LOCAL row numbers, token t uses
 * its first counts[t] (<= entries_per_token) entries, and the result is the fp32 partial sum
 * out_f32[t] = sum_j w[t,j] * act(down[ids[t,j]] . x[t]) * up[ids[t,j]] that the ranks then reduce.
 * The reference has no sharded implementation of the layer (expert sharding is announced in
 * docs/paper/paper.tex:446 and listed as future work in docs/CUTLASS_KERNEL.md:181); this is the
 * per-rank piece of it, with the semantics of experts.py:332-382 restricted to the owned rows. */
int peer_gather_eval_partial(peer_handle_t h, const void* x, const int32_t* ids, const float* weights,
                             const int32_t* counts, int32_t entries_per_token, const void* expert_down,
                             const void* expert_up, const float* down_scale, const float* up_scale,
                             int64_t n_local_rows, float* out_f32, int64_t n_tokens, void* stream);

/* The other per-rank pieces of the expert-parallel layer (no counterpart in the reference, see above).
 *
 * peer_select_tokens: query projection + selection only (experts.py:302-327): flat expert ids int32
 * and softmax weights fp32, both [T, num_heads*top_k], into caller buffers - what this rank sends.
 * t->expert_down / expert_up / out are not read; t->ids_out / scores_out are filled when given.
 *
 * peer_route_tuples (sender): sorts the T*E tuples of this rank's T tokens (E = entries_per_token) by owner =
 * id / rows_per_rank into `send`: one block of int32 per destination rank, `world` blocks of
 * 2*T*E + T words each, laid out [local row ids: T x E | weight bits: T x E | counts: T].  Row t holds,
 * packed to the front in slot order, those of token t's tuples the destination owns (id - owner*rows_per_rank),
 * counts[t] how many; unused slots are (row 0, weight 0); ids outside [0, world*rows_per_rank) go nowhere.
 * One all-to-all of equal-size blocks then gives every rank `world` such blocks, and because a token's
 * tuples only ever come from the rank that owns the token, block b row t IS the list of global token
 * b*T + t: nothing is sorted or merged on the receiving side.  Deterministic; no handle; asynchronous.
 *
 * peer_gather_eval_routed (receiver): peer_gather_eval_partial reading those received blocks in place:
 * `recv` = int32 [world][2*T*E + T] as it arrives (T = tokens_per_rank, E = num_heads*top_k of the handle),
 * x = the activations of all world*T tokens [world*T, input_dim], out_f32 [world*T, output_dim]. */
int peer_select_tokens(peer_handle_t h, const peer_tensors_t* t, int64_t n_tokens, int32_t* ids_out,
                       float* weights_out, void* stream);
int peer_route_tuples(const int32_t* ids, const float* weights, int64_t n_tokens, int32_t entries_per_token,
                      int64_t rows_per_rank, int32_t world, int32_t* send, void* stream);
int peer_gather_eval_routed(peer_handle_t h, const void* x, const int32_t* recv, int32_t world,
                            int64_t tokens_per_rank, const void* expert_down, const void* expert_up,
                            const float* down_scale, const float* up_scale, int64_t n_local_rows,
                            float* out_f32, void* stream);

/* Direct exchange for the expert-parallel layer on the GPUs of one node: what the all-gather, the all-to-all
 * and the reduce-scatter around peer_select_tokens / peer_gather_eval_routed move, written by plain stores
 * into the peers' memory (NVLink) with step numbers as completion flags.  No counterpart in the reference
 * (it has no sharded PEER: docs/paper/paper.tex:446, docs/CUTLASS_KERNEL.md:181).
 *
 * peer_xchg_create allocates this rank's region on the current device (activations of all world*T tokens,
 * `world` tuple blocks in the format of peer_route_tuples, `world` slots of fp32 partial sums for this rank's
 * T tokens, each twice, and the flags); peer_xchg_export gives its 64-byte CUDA IPC handle; after the ranks
 * have exchanged the handles by any host-side means, peer_xchg_attach(handles of all ranks, 64 bytes each,
 * in rank order; the own entry is ignored) maps the peers' regions.  One step, all calls on one stream:
 *   peer_xchg_push_x(x of my T tokens)           -> starts the step; x goes to every rank
 *   peer_xchg_route(ids, weights [T, E])         -> tuples go to the owners of the rows (after peer_select_tokens)
 *   peer_xchg_wait_inputs(&x_all, &recv)         -> waits for all ranks' x and tuples; the pointers are what
 *                                                   peer_gather_eval_routed takes
 *   peer_xchg_combine(partial [world*T, D_out] fp32, out [T, D_out] act dtype)
 *                                                -> partial sums go to the tokens' ranks; out = their sum in
 *                                                   rank order (deterministic), cast to the activation dtype
 * peer_xchg_forward is that whole step in one call (t->x = my T tokens, t->expert_down / expert_up = my rows; the
 * scratch buffers are the caller's: ids and weights [T, E], partial sums fp32 [world*T, D_out]).
 * peer_xchg_counts (after peer_xchg_wait_inputs) copies out how many tuples each of the world*T tokens brought
 * to this rank.  Every rank must run the same steps in the same order.  Waits are bounded (two seconds): when a rank's data
 * does not arrive, the step's result is undefined and peer_xchg_status (synchronises the stream) returns
 * PEER_ERR_DEVICE_TIMEOUT; nothing hangs.  After such a timeout the ranks' step numbers no longer agree: destroy
 * the exchange on every rank and create it anew.  peer_xchg_destroy must be called by all ranks only after all of
 * them have finished their last step (a host barrier), since peers write into the region.  Errors: return
 * code + peer_last_error(NULL). */
typedef struct peer_xchg* peer_xchg_t;
int peer_xchg_create(int32_t world, int32_t rank, int64_t tokens_per_rank, int32_t entries_per_token,
                     int32_t input_dim, int32_t output_dim, int32_t act_dtype, peer_xchg_t* out);
int peer_xchg_export(peer_xchg_t h, unsigned char* handle64);
int peer_xchg_attach(peer_xchg_t h, const unsigned char* handles);
int peer_xchg_push_x(peer_xchg_t h, const void* x_local, void* stream);
int peer_xchg_route(peer_xchg_t h, const int32_t* ids, const float* weights, int64_t rows_per_rank, void* stream);
int peer_xchg_wait_inputs(peer_xchg_t h, const void** x_all, const int32_t** recv, void* stream);
int peer_xchg_combine(peer_xchg_t h, const float* partial, void* out, void* stream);
int peer_xchg_forward(peer_xchg_t x, peer_handle_t h, const peer_tensors_t* t, int32_t* ids_scratch,
                      float* weights_scratch, int64_t rows_per_rank, float* partial_scratch, void* out, void* stream);
int peer_xchg_counts(peer_xchg_t h, int32_t* counts_out, void* stream);
int peer_xchg_status(peer_xchg_t h, void* stream);
int peer_xchg_destroy(peer_xchg_t h);

/* Backward of peer_gather_eval: the gradients autograd derives for the expert evaluation of the
 * reference (llm/models/experts.py:332-382; exercised by tests/test_peer_integration.py:181-192 and
 * by the training step, llm/training/train.py:743-768).  Given grad_out = dL/dout [T, output_dim]
 * (act_dtype) and the forward's x, ids and weights:
 *   grad_x       [T, input_dim]      fp32, written:  sum_j dz_j * down[ids_j]
 *   grad_weights [T, num_heads*top_k] fp32, written: act(down[ids_j] . x) * (up[ids_j] . grad_out)
 *   grad_down    [num_experts, input_dim]  ACCUMULATED: += dz_j * x          (zero it first)
 *   grad_up      [num_experts, output_dim] ACCUMULATED: += w_j * act(.) * grad_out
 * with dz_j = w_j * (up[ids_j] . grad_out) * act'(down[ids_j] . x).  Tables must be in act_dtype.
 * grad_table_dtype: PEER_DTYPE_F32, or PEER_DTYPE_BF16 for a bf16 layer: the sums are then formed in
 * bf16, as the reference's bf16 training forms them (its embedding gradients are bf16 tensors), with
 * half the memory traffic and no cast afterwards. */
int peer_gather_eval_backward(peer_handle_t h, const void* x, const void* grad_out, const int32_t* ids,
                              const float* weights, const void* expert_down, const void* expert_up,
                              float* grad_x, float* grad_weights, void* grad_down, void* grad_up,
                              int32_t grad_table_dtype, int64_t n_tokens, void* stream);

/* The same with gradient tables of only n_grad_rows rows (grad_down [n_grad_rows, input_dim], grad_up
 * [n_grad_rows, output_dim]) for callers who know that every id lies below n_grad_rows: with the reference's
 * id arithmetic (i0 + i1, experts.py:203-230) ids stay below n_keys0 + n_keys1, so a few thousand rows of fp32
 * sums (L2-resident) replace two dense fp32 tables.  An id at or beyond n_grad_rows is skipped and recorded in
 * the status word like any id outside the table. */
int peer_gather_eval_backward_rows(peer_handle_t h, const void* x, const void* grad_out, const int32_t* ids,
                                   const float* weights, const void* expert_down, const void* expert_up,
                                   float* grad_x, float* grad_weights, void* grad_down, void* grad_up,
                                   int32_t grad_table_dtype, int64_t n_grad_rows, int64_t n_tokens, void* stream);

/* Backward of the score path: from grad_weights = dL/d(softmax weights) [T, num_heads, top_k] to
 * grad_queries = dL/d(queries after LayerNorm) [T, num_heads, query_dim] (fp32, written), through the
 * softmax, the selected scores and the per-slice query normalisation of experts.py:153-163, :327.
 * queries: the fp32 queries the forward selected from; product_ids: grid positions written by
 * peer_forward (product_ids_out); scores: the forward's raw scores.  The sub-keys get no gradient,
 * as in the reference (it reads them through .data, experts.py:154). */
int peer_select_backward(peer_handle_t h, const float* queries, const void* const* keys,
                         const int32_t* product_ids, const float* scores, const float* grad_weights,
                         int64_t n_tokens, float* grad_queries, void* stream);

/* Product-key retrieval (same result as peer_select) for callers that cannot allocate device
 * memory: no handle, no cudaMalloc anywhere on this path.  This entry point has no counterpart in
 * the reference; it exists for embedders that have given all GPU memory to their own pool, or that
 * run in a loop where an allocation's device-wide synchronisation is not acceptable.  The scratch
 * the kernels need sits in an 8 MiB array inside the library image (held by every GPU that loads
 * the library), so n_tokens*num_heads*query_dim*4 + (n_keys0+n_keys1)*query_dim*2 bytes must fit
 * in it; larger calls return PEER_ERR_UNSUPPORTED with both sizes in peer_last_error(NULL).
 * Of `cfg` only abi_version, num_heads, query_dim, n_keys0, n_keys1, top_k, norm_keys, norm_query,
 * act_dtype (dtype of the sub-keys) and index_mode are read.  The first call on each device does
 * a one-time set-up (address of the array, kernel attribute; serialised by a lock): make it at
 * start-up, before any stream capture.  Every later call only enqueues kernels on `stream`: it
 * reads no host memory and does not synchronise.  All calls share the array: calls whose kernels
 * may overlap on the GPU race. */
int peer_select_noalloc(const peer_config_t* cfg, const float* queries, const void* keys0,
                        const void* keys1, int64_t n_tokens, int64_t* ids_out, float* scores_out,
                        void* stream);

/* Expert-usage histogram on the device: counts[id] += 1 for every id in ids[0 .. n_ids) (int64, the
 * layout of ids_out / the module's _last_expert_indices).  Replaces the host loop of
 * ExpertUsageTracker.record_usage (llm/utils/experts/tracking.py:96-100).  No handle; ids outside
 * [0, num_experts) are not counted but added to *dropped when that pointer is given.  Asynchronous. */
int peer_usage_histogram(const int64_t* ids, int64_t n_ids, int64_t* counts, int64_t num_experts,
                         int64_t* dropped, void* stream);

/* Reads and clears the device status word (synchronises `stream`).  Returns
 * PEER_OK, PEER_ERR_DEVICE_TIMEOUT or PEER_ERR_BOUNDS.  The kernels never
 * trap: a bounded wait that runs out, or an expert id outside the table,
 * is recorded there and the offending access is skipped. */
int peer_query_status(peer_handle_t h, void* stream);

/* Inference with fixed weights: while `frozen` is set the caller promises that the sub-key tables it passes to this
 * handle do not change, and what the selection derives from them (1/||key||, the normalised copy, the first pass's
 * error bounds: one small launch per call otherwise) is computed by the first call and reused by every later call
 * that brings the same two key pointers on the same stream.  Other pointers, another stream, or setting the flag
 * again compute them anew.  Off by default: the reference's module reads its keys afresh in every forward
 * (llm/models/experts.py:153-163), which is what training needs.  Only for two-dimensional key grids. */
int peer_freeze_keys(peer_handle_t h, int frozen);

/* Per-stage device timing, for benchmarks: while enabled, every slice of
 * peer_forward / peer_forward_host records CUDA events on its stream around
 * the three stage launches (query, select, expert evaluation).  Enabling or
 * disabling discards pending measurements.  Replaces the cudaEvent timing of
 * the reference's smoke_test (llm/models/kernels/peer_cutlass.cu:1468-1483). */
int peer_stage_timing(peer_handle_t h, int enable);

/* Waits for the recorded slices and returns the summed milliseconds of the
 * three stages in ms3[0..2] and the number of slices in *n_slices; clears the
 * record. */
int peer_stage_times(peer_handle_t h, double* ms3, int64_t* n_slices);

/* Number of kernel launches this handle has enqueued since creation. */
int64_t peer_launch_count(peer_handle_t h);

/* Library ABI version (PEER_B200_ABI_VERSION it was built with). */
int peer_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* PEER_B200_H */
