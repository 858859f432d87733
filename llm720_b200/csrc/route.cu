// Tuple routing for the expert-parallel layer (tables split by rows over ranks).
//
// The reference has no sharded PEER (expert sharding is announced in
// docs/paper/paper.tex:446 and listed as future work in docs/CUTLASS_KERNEL.md:181);
// what is exchanged follows from its forward (llm/models/experts.py:332-382): each
// selected (token, expert id, softmax weight) must reach the rank that owns the
// expert's rows.
//
// Wire format.  Every rank sends every peer one fixed-shape block of int32:
//     [ local row ids : T x E | weight bits : T x E | counts : T ]
// (T = tokens of the sending rank, E = num_heads * top_k).  Row t of the first two
// parts holds, packed to the front and in slot order, those of token t's tuples
// whose expert the receiving peer owns; counts[t] says how many.  A token's tuples
// reach a peer only from the rank that owns the token, so what a rank receives
// from its `world` peers IS the per-token list of all world * T tokens: block b,
// row t belongs to global token b * T + t.  Nothing has to be sorted, merged or
// counted on the receiving side; the expert stage reads the blocks in place
// (launch_gather_eval with GatherArgs::block_tokens).
// One kernel, one warp per token, deterministic (ballots, no atomics).
#include "common.cuh"
#include "kernels.h"

namespace peer {

namespace {

constexpr int ROUTE_WARPS = 4;

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_kernel(const int32_t* __restrict__ ids, const float* __restrict__ weights, int64_t T, int E, int64_t rows,
             int world, int32_t* __restrict__ send) {
    const int lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * ROUTE_WARPS + (threadIdx.x >> 5);
    if (t >= T) return;                                   // warp-uniform
    const int64_t block = 2 * T * E + T;                  // int32 per destination
    for (int r = 0; r < world; ++r) {
        int32_t* b_ids = send + r * block + t * E;
        int32_t* b_w = send + r * block + T * E + t * E;
        int n = 0;
        for (int e0 = 0; e0 < E; e0 += 32) {
            const int e = e0 + lane;
            int64_t id = -1;
            float w = 0.f;
            if (e < E) { id = ids[t * E + e]; w = weights[t * E + e]; }
            const bool mine = id >= r * rows && id < (r + 1) * rows;      // an id outside the table goes nowhere
            const unsigned m = __ballot_sync(FULL_MASK, mine);
            if (mine) {
                const int pos = n + __popc(m & ((1u << lane) - 1u));
                b_ids[pos] = static_cast<int32_t>(id - r * rows);
                b_w[pos] = __float_as_int(w);
            }
            n += __popc(m);
        }
        for (int j = n + lane; j < E; j += 32) { b_ids[j] = 0; b_w[j] = 0; }   // unused slots: row 0, weight 0
        if (lane == 0) send[r * block + 2 * T * E + t] = n;
    }
}

}  // namespace

cudaError_t launch_route_tuples(const int32_t* ids, const float* weights, int64_t n_tokens, int entries_per_token,
                                int64_t rows_per_rank, int world, int32_t* send, cudaStream_t s) {
    if (world < 1 || rows_per_rank < 1 || entries_per_token < 1) return cudaErrorInvalidValue;
    if (n_tokens == 0) return cudaSuccess;
    const unsigned blocks = static_cast<unsigned>((n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS);
    route_kernel<<<blocks, ROUTE_WARPS * 32, 0, s>>>(ids, weights, n_tokens, entries_per_token, rows_per_rank, world, send);
    return cudaGetLastError();
}

}  // namespace peer
