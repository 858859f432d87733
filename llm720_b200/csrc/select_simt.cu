// Product-key selection on CUDA cores, exact fp32: sub-key scores for both
// query halves, per-half top-k', the k' x k' candidate sums, final top-k,
// softmax and the flat expert id, fused so that no score ever reaches HBM.
//
// Follows llm/models/experts.py:153-163 (scores), :168-192 (per-half top-k'),
// :203-259 (candidate sums, flat ids, final top-k) and :327 (softmax).
//
// Ordering rule wherever scores tie exactly: the smaller sub-key index (per
// half) or the smaller flat candidate position a*k'+b (final) comes first.
#include <float.h>
#include <limits.h>

#include "common.cuh"
#include "kernels.h"

namespace peer {

namespace {

constexpr int R = 32;          // (token, head) rows per CTA
constexpr int KT = 128;        // sub-keys per tile
constexpr int MAXHW = 128;     // largest half query width
constexpr int THREADS = 256;
constexpr size_t SMEM_BYTES = sizeof(float) * (MAXHW * R + MAXHW * KT);

// khatT0/1: normalised sub-keys stored TRANSPOSED, [Q/2][n], so that a tile of
// consecutive keys is read with coalesced loads.
__global__ void __launch_bounds__(THREADS, 2) select_simt_kernel(SelectArgs a) {
    extern __shared__ __align__(16) float smem[];
    float* qh = smem;                 // [hw][R]   query halves, transposed
    float* kt = smem + MAXHW * R;     // [hw][KT]  key tile, transposed

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hw = a.Q / 2;
    // Either all rows [0, rows), or only the rows named in row_list (the rows another kernel left over).
    const int64_t nrows = a.row_list ? static_cast<int64_t>(*a.row_count) : a.rows;
    for (int64_t blk = blockIdx.x; blk * R < nrows; blk += gridDim.x) {
    const int64_t row0 = blk * R;
    auto row_of = [&](int64_t i) -> int64_t {       // i-th row of this pass -> row of the layer, or -1
        if (i >= nrows) return -1;
        return a.row_list ? static_cast<int64_t>(a.row_list[i]) : i;
    };

    float lv[2][4];
    int li[2][4];

#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int n = half ? a.n1 : a.n0;
        const int kp = half ? a.kp1 : a.kp0;
        const float* __restrict__ khatT = half ? a.khat1 : a.khat0;
#pragma unroll
        for (int i = 0; i < 4; ++i) { lv[half][i] = -INFINITY; li[half][i] = INT_MAX; }

        __syncthreads();   // everyone is done with the previous half's qh
        {   // lane = row, warp = 16-wide slice of the half
            const int64_t r = row_of(row0 + lane);
            for (int c0 = warp * 16; c0 < hw; c0 += 8 * 16) {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int c = c0 + e;
                    if (c < hw) {
                        float qv = 0.f;
                        if (r >= 0) {
                            const int64_t o = r * a.Q + half * hw + c;
                            if (a.q_split)      // hi + mid + lo bf16 terms: the fp32 value exactly
                                qv = (__bfloat162float(a.q_split[o]) + __bfloat162float(a.q_split[o + a.split_stride])) +
                                     __bfloat162float(a.q_split[o + 2 * a.split_stride]);
                            else
                                qv = a.q_hat[o];
                        }
                        qh[c * R + lane] = qv;
                    }
                }
            }
        }

        for (int base = 0; base < n; base += KT) {
            __syncthreads();   // previous tile consumed (and qh stores ordered before use)
            if ((n & 3) == 0) {
                for (int idx = tid; idx < hw * (KT / 4); idx += THREADS) {
                    const int kk = idx / (KT / 4), c = (idx % (KT / 4)) * 4;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (base + c < n)
                        v = *reinterpret_cast<const float4*>(khatT + static_cast<int64_t>(kk) * n + base + c);
                    *reinterpret_cast<float4*>(kt + kk * KT + c) = v;
                }
            } else {
                for (int idx = tid; idx < hw * KT; idx += THREADS) {
                    const int kk = idx / KT, c = idx % KT;
                    kt[kk * KT + c] = (base + c < n) ? khatT[static_cast<int64_t>(kk) * n + base + c] : 0.f;
                }
            }
            __syncthreads();

            float acc[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 4
            for (int kk = 0; kk < hw; ++kk) {
                const float4 q4 = *reinterpret_cast<const float4*>(qh + kk * R + warp * 4);
                const float q[4] = {q4.x, q4.y, q4.z, q4.w};
                float b[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = kt[kk * KT + lane + 32 * j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(q[i], b[j], acc[i][j]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int key = base + lane + 32 * j;
                    warp_list_offer(lv[half][i], li[half][i], acc[i][j], key, key < n, kp, lane);
                }
        }
    }

    // Combine: candidate (a, b) has score s0[a] + s1[b]; only pairs with
    // (a+1)(b+1) <= k can reach the top k because both lists are sorted.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = row_of(row0 + warp * 4 + i);
        if (r < 0) continue;   // warp-uniform
        float fv = -INFINITY;
        int fi = INT_MAX;
        for (int p = 0; p < a.n_pairs; ++p) {
            const int pr = a.pairs[p];
            const int pa = pr >> 8, pb = pr & 255;
            const float cv = __shfl_sync(FULL_MASK, lv[0][i], pa) + __shfl_sync(FULL_MASK, lv[1][i], pb);
            warp_list_insert(fv, fi, cv, pa * a.kp1 + pb, a.k, lane);
        }
        const bool live = lane < a.k;
        const int pa = live ? fi / a.kp1 : 0, pb = live ? fi % a.kp1 : 0;
        const int i0 = __shfl_sync(FULL_MASK, li[0][i], pa);
        const int i1 = __shfl_sync(FULL_MASK, li[1][i], pb);
        const int64_t id = static_cast<int64_t>(i0) * a.mult0 + static_cast<int64_t>(i1) * a.mult1;
        const float top = __shfl_sync(FULL_MASK, fv, 0);
        const float e = live ? expf(fv - top) : 0.f;
        const float w = e / warp_sum(e);
        if (live) {
            const int64_t o = r * a.k + lane;
            if (a.ids32) a.ids32[o] = static_cast<int32_t>(id);
            if (a.weights) a.weights[o] = w;
            if (a.ids64) a.ids64[o] = id;
            if (a.raw_scores) a.raw_scores[o] = fv;
            if (a.prod_ids) a.prod_ids[o] = i0 * a.n1 + i1;
        }
    }
    }
}

}  // namespace

cudaError_t select_simt_setup() {
    return cudaFuncSetAttribute(select_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(SMEM_BYTES));
}

cudaError_t launch_select_simt(const SelectArgs& a, cudaStream_t s) {
    if (a.rows == 0) return cudaSuccess;
    // with a row list the number of rows is only known on the device: a small fixed grid loops over it
    const unsigned grid = a.row_list ? 296u : static_cast<unsigned>((a.rows + R - 1) / R);
    select_simt_kernel<<<grid, THREADS, SMEM_BYTES, s>>>(a);
    return cudaGetLastError();
}

}  // namespace peer
