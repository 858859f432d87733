// Tuple routing for the expert-parallel layer (tables split by rows over ranks).
//
// The reference has no sharded PEER (expert sharding is announced in
// docs/paper/paper.tex:446 and listed as future work in docs/CUTLASS_KERNEL.md:181);
// what is exchanged follows from its forward (llm/models/experts.py:332-382): each
// selected (token, expert id, softmax weight) must reach the rank that owns the
// expert's rows.
//
// Two kernels, both deterministic (no atomics decide an order, so the partial sums
// downstream are formed in the same order on every run):
//   route  (sender)   bucket this rank's tuples by owner = id / rows_per_rank into a
//                     fixed-shape buffer [world, cap, 3] of (global token, local row,
//                     weight bits); a bucket keeps the tuples in (token, slot) order
//                     and is padded with token -1;
//   pack   (receiver) turn the received buckets [world, cap, 3] into per-token lists
//                     (ids [T, list_cap], weights [T, list_cap], counts [T]) in
//                     (source rank, position) order, the input of
//                     peer_gather_eval_partial.
#include "common.cuh"
#include "kernels.h"

namespace peer {

namespace {

constexpr int ROUTE_THREADS = 1024;
constexpr int ROUTE_WARPS = ROUTE_THREADS / 32;
constexpr int MAX_WORLD = 64;

__global__ void __launch_bounds__(ROUTE_THREADS, 1)
route_kernel(const int32_t* __restrict__ ids, const float* __restrict__ weights, int64_t n, int HK, int token_offset,
             int64_t rows, int world, int64_t cap, int32_t* __restrict__ send) {
    __shared__ int s_base[MAX_WORLD];                 // tuples placed so far, per owner
    __shared__ int s_warp[ROUTE_WARPS][MAX_WORLD];    // per chunk: tuples of each warp per owner, then their offsets
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < world) s_base[tid] = 0;
    __syncthreads();
    for (int64_t c0 = 0; c0 < n; c0 += ROUTE_THREADS) {
        const int64_t i = c0 + tid;
        int owner = -1, local = 0, tok = 0;
        uint32_t wbits = 0;
        if (i < n) {
            const int64_t id = ids[i];
            if (id >= 0 && id < rows * world) {       // an id outside the table is not sent anywhere
                owner = static_cast<int>(id / rows);
                local = static_cast<int>(id - static_cast<int64_t>(owner) * rows);
                tok = token_offset + static_cast<int>(i / HK);
                wbits = __float_as_uint(weights[i]);
            }
        }
        int before = 0;                               // tuples of my owner in lower lanes of my warp
        for (int r = 0; r < world; ++r) {
            const unsigned m = __ballot_sync(FULL_MASK, owner == r);
            if (lane == 0) s_warp[warp][r] = __popc(m);
            if (owner == r) before = __popc(m & ((1u << lane) - 1u));
        }
        __syncthreads();
        if (tid < world) {                            // exclusive scan over the warps, continuing from earlier chunks
            int run = s_base[tid];
            for (int w = 0; w < ROUTE_WARPS; ++w) {
                const int c = s_warp[w][tid];
                s_warp[w][tid] = run;
                run += c;
            }
            s_base[tid] = run;
        }
        __syncthreads();
        if (owner >= 0) {
            const int64_t pos = s_warp[warp][owner] + before;
            if (pos < cap) {
                int32_t* dst = send + (static_cast<int64_t>(owner) * cap + pos) * 3;
                dst[0] = tok; dst[1] = local; dst[2] = static_cast<int32_t>(wbits);
            }
        }
        __syncthreads();
    }
    for (int r = 0; r < world; ++r)                   // padding: token -1
        for (int64_t pos = s_base[r] + tid; pos < cap; pos += ROUTE_THREADS) {
            int32_t* dst = send + (static_cast<int64_t>(r) * cap + pos) * 3;
            dst[0] = -1; dst[1] = 0; dst[2] = 0;
        }
}

constexpr int PACK_WARPS = 4;

__global__ void __launch_bounds__(PACK_WARPS * 32)
pack_kernel(const int32_t* __restrict__ recv, int world, int64_t cap, int64_t T, int list_cap,
            int32_t* __restrict__ ids_out, float* __restrict__ w_out, int32_t* __restrict__ counts) {
    const int lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * PACK_WARPS + (threadIdx.x >> 5);
    if (t >= T) return;                               // warp-uniform
    int n = 0;
    for (int b = 0; b < world; ++b) {
        const int32_t* bucket = recv + static_cast<int64_t>(b) * cap * 3;
        for (int64_t e0 = 0; e0 < cap; e0 += 32) {
            const int64_t e = e0 + lane;
            const int tok = e < cap ? bucket[e * 3] : -1;
            if (__ballot_sync(FULL_MASK, tok >= 0) == 0) break;       // the rest of this bucket is padding
            const unsigned m = __ballot_sync(FULL_MASK, tok == static_cast<int>(t));
            if (tok == static_cast<int>(t)) {
                const int pos = n + __popc(m & ((1u << lane) - 1u));
                if (pos < list_cap) {
                    ids_out[t * list_cap + pos] = bucket[e * 3 + 1];
                    w_out[t * list_cap + pos] = __int_as_float(bucket[e * 3 + 2]);
                }
            }
            n += __popc(m);
        }
    }
    const int used = n < list_cap ? n : list_cap;
    for (int j = used + lane; j < list_cap; j += 32) { ids_out[t * list_cap + j] = 0; w_out[t * list_cap + j] = 0.f; }
    if (lane == 0) counts[t] = used;
}

}  // namespace

cudaError_t launch_route_tuples(const int32_t* ids, const float* weights, int64_t n_tokens, int entries_per_token,
                                int token_offset, int64_t rows_per_rank, int world, int64_t bucket_cap, int32_t* send,
                                cudaStream_t s) {
    if (world < 1 || world > MAX_WORLD || rows_per_rank < 1 || entries_per_token < 1 || bucket_cap < 1)
        return cudaErrorInvalidValue;
    route_kernel<<<1, ROUTE_THREADS, 0, s>>>(ids, weights, n_tokens * entries_per_token, entries_per_token, token_offset,
                                             rows_per_rank, world, bucket_cap, send);
    return cudaGetLastError();
}

cudaError_t launch_pack_tuples(const int32_t* recv, int world, int64_t bucket_cap, int64_t n_tokens, int list_cap,
                               int32_t* ids_out, float* weights_out, int32_t* counts_out, cudaStream_t s) {
    if (world < 1 || bucket_cap < 1 || list_cap < 1) return cudaErrorInvalidValue;
    if (n_tokens == 0) return cudaSuccess;
    const unsigned blocks = static_cast<unsigned>((n_tokens + PACK_WARPS - 1) / PACK_WARPS);
    pack_kernel<<<blocks, PACK_WARPS * 32, 0, s>>>(recv, world, bucket_cap, n_tokens, list_cap, ids_out, weights_out,
                                                   counts_out);
    return cudaGetLastError();
}

}  // namespace peer
