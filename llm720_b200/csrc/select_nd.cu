// Product-key selection for any number of key dimensions (1 to 4), exact fp32,
// one warp per (token, head) row.  This is the general form of
// llm/models/experts.py:138-285: per-dimension cosine scores (:149-163),
// top-k' per dimension (:168-192), then the dimensions are folded in one at a
// time: all sums of a kept candidate and a dimension's candidate are formed,
// and the best min(4k, count) of them (the last fold: the best k) are kept
// (:214-265); when a fold keeps every sum they stay in their flattened order,
// exactly as the reference leaves them.  The two-dimensional layers of the
// benchmark configurations use the specialised kernels (select_tc.cu,
// select_simt.cu); this one covers 1-D, 3-D and 4-D keys and odd widths, e.g.
// the reference's own test layer with query_dim 30 over a 4x4x4 grid
// (tests/test_peer_integration.py:92-111).
//
// Flat ids: dimension d contributes index * mult[d]; the caller passes
// mult[0] = 1 for the reference's index arithmetic (the first dimension never
// receives its multiplier, experts.py:203-204) or the true stride.
// Ties: smaller sub-key index first (per dimension), smaller flattened
// candidate position first (folds).
#include <float.h>
#include <limits.h>

#include "common.cuh"
#include "kernels.h"

namespace peer {

namespace {

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int MAX_W = 256;      // widest per-dimension query slice
constexpr int MAX_KEEP = 128;   // 4 * top_k
constexpr float NORM_EPS = 1e-12f;

__device__ __forceinline__ int f2key(float x) { const int i = __float_as_int(x); return i ^ ((i >> 31) & 0x7fffffff); }
__device__ __forceinline__ float key2f(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7fffffff)); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL_MASK, v, o));
    return v;
}

struct WarpScratch {
    float q[MAX_W];
    float top_s[4][32];
    int top_i[4][32];
    float run_s[2][MAX_KEEP];
    long long run_i[2][MAX_KEEP];
    int run_p[2][MAX_KEEP];         // the same candidates' true positions in the key grid
};

template <typename T>
__global__ void __launch_bounds__(THREADS) select_nd_kernel(const SelectNdArgs a) {
    __shared__ WarpScratch scratch[WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    WarpScratch& w = scratch[warp];
    const int width = a.Q / a.nd;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * WARPS + warp; row < a.rows;
         row += static_cast<int64_t>(gridDim.x) * WARPS) {
        // ---- per dimension: normalised query slice, scores, top-k'
        for (int d = 0; d < a.nd; ++d) {
            __syncwarp();
            float ss = 0.f;
            for (int c = lane; c < width; c += 32) {
                const float v = a.q_ln[row * a.Q + d * width + c];
                w.q[c] = v;
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
            const float qs = a.norm_query ? 1.0f / fmaxf(sqrtf(ss), NORM_EPS) : 1.0f;
            __syncwarp();
            for (int c = lane; c < width; c += 32) w.q[c] *= qs;
            __syncwarp();
            const T* __restrict__ keys = static_cast<const T*>(a.keys[d]);
            float lv = -INFINITY;
            int li = INT_MAX;
            for (int base = 0; base < a.n[d]; base += 32) {
                const int j = base + lane;
                float dot = 0.f, kk = 0.f;
                if (j < a.n[d]) {
                    const T* kr = keys + static_cast<int64_t>(j) * width;
                    for (int c = 0; c < width; ++c) {
                        const float kv = to_f32<T>(kr[c]);
                        dot = fmaf(w.q[c], kv, dot);
                        kk = fmaf(kv, kv, kk);
                    }
                    if (a.norm_keys) dot *= 1.0f / fmaxf(sqrtf(kk), NORM_EPS);
                }
                warp_list_offer(lv, li, dot, j, j < a.n[d], a.kp[d], lane);
            }
            w.top_s[d][lane] = lv;
            w.top_i[d][lane] = li;
        }
        __syncwarp();

        // ---- fold the dimensions
        int cur = 0, len;
        if (a.nd == 1) {
            len = min(a.k, a.kp[0]);                       // already sorted: the best k of the one list
            // mult[0] == 0: the reference's 1-D result, positions inside the candidate list (experts.py:197-200)
            for (int c = lane; c < len; c += 32) {
                w.run_s[0][c] = w.top_s[0][c];
                w.run_i[0][c] = a.mult[0] == 0 ? c : static_cast<long long>(w.top_i[0][c]) * a.mult[0];
                w.run_p[0][c] = w.top_i[0][c];
            }
        } else {
            len = a.kp[0];
            for (int c = lane; c < len; c += 32) {
                w.run_s[0][c] = w.top_s[0][c];
                w.run_i[0][c] = static_cast<long long>(w.top_i[0][c]) * a.mult[0];
                w.run_p[0][c] = static_cast<int>(w.top_i[0][c] * a.stride[0]);
            }
            for (int d = 1; d < a.nd; ++d) {
                __syncwarp();
                const int kp = a.kp[d];
                const int count = len * kp;
                int keep = d < a.nd - 1 ? min(4 * a.k, count) : min(a.k, count);
                keep = max(keep, 1);
                const int nxt = cur ^ 1;
                if (keep == count) {                       // every sum is kept, in flattened order
                    for (int c = lane; c < count; c += 32) {
                        w.run_s[nxt][c] = w.run_s[cur][c / kp] + w.top_s[d][c % kp];
                        w.run_i[nxt][c] = w.run_i[cur][c / kp] + static_cast<long long>(w.top_i[d][c % kp]) * a.mult[d];
                        w.run_p[nxt][c] = w.run_p[cur][c / kp] + static_cast<int>(w.top_i[d][c % kp] * a.stride[d]);
                    }
                } else {
                    int last_key = INT_MAX, last_pos = -1;   // nothing taken yet
                    bool first = true;
                    for (int it = 0; it < keep; ++it) {
                        int best_key = INT_MIN, best_pos = INT_MAX;
                        for (int c = lane; c < count; c += 32) {
                            const int key = f2key(w.run_s[cur][c / kp] + w.top_s[d][c % kp]);
                            const bool eligible = first || key < last_key || (key == last_key && c > last_pos);
                            if (eligible && (key > best_key || (key == best_key && c < best_pos))) { best_key = key; best_pos = c; }
                        }
                        const int m = __reduce_max_sync(FULL_MASK, best_key);
                        const int pos = __reduce_min_sync(FULL_MASK, best_key == m ? best_pos : INT_MAX);
                        if (lane == 0) {
                            w.run_s[nxt][it] = key2f(m);
                            w.run_i[nxt][it] = w.run_i[cur][pos / kp] + static_cast<long long>(w.top_i[d][pos % kp]) * a.mult[d];
                            w.run_p[nxt][it] = w.run_p[cur][pos / kp] + static_cast<int>(w.top_i[d][pos % kp] * a.stride[d]);
                        }
                        last_key = m; last_pos = pos; first = false;
                    }
                }
                len = keep;
                cur = nxt;
            }
        }
        __syncwarp();
        const int kout = min(a.k, len);                     // experts.py:267-270
        // ---- softmax over the kept scores, outputs (k_out entries per row; the caller sizes by it)
        float mx = -INFINITY;
        for (int c = lane; c < kout; c += 32) mx = fmaxf(mx, w.run_s[cur][c]);
        mx = warp_max(mx);
        float es = 0.f;
        for (int c = lane; c < kout; c += 32) es += expf(w.run_s[cur][c] - mx);
        es = warp_sum(es);
        for (int c = lane; c < kout; c += 32) {
            const int64_t o = row * kout + c;
            const float sc = w.run_s[cur][c];
            const long long id = w.run_i[cur][c];
            if (a.ids32) a.ids32[o] = static_cast<int32_t>(id);
            if (a.weights) a.weights[o] = expf(sc - mx) / es;
            if (a.ids64) a.ids64[o] = id;
            if (a.raw_scores) a.raw_scores[o] = sc;
            if (a.prod_ids) a.prod_ids[o] = w.run_p[cur][c];
        }
    }
}

}  // namespace

cudaError_t launch_select_nd(const SelectNdArgs& a, cudaStream_t s) {
    if (a.rows == 0) return cudaSuccess;
    if (a.nd < 1 || a.nd > 4 || a.Q % a.nd || a.Q / a.nd > MAX_W || 4 * a.k > MAX_KEEP) return cudaErrorInvalidValue;
    for (int d = 0; d < a.nd; ++d)
        if (a.kp[d] < 1 || a.kp[d] > 32 || a.n[d] < 1) return cudaErrorInvalidValue;
    int64_t blocks = (a.rows + WARPS - 1) / WARPS;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (a.act_dtype == PEER_DTYPE_F32) select_nd_kernel<float><<<static_cast<unsigned>(blocks), THREADS, 0, s>>>(a);
    else if (a.act_dtype == PEER_DTYPE_BF16) select_nd_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), THREADS, 0, s>>>(a);
    else if (a.act_dtype == PEER_DTYPE_F16) select_nd_kernel<__half><<<static_cast<unsigned>(blocks), THREADS, 0, s>>>(a);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace peer
