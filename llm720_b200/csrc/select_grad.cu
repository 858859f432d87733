// Backward of the score path of the selection: given dL/dw for the softmax
// weights w = softmax(s) of the k selected experts of a (token, head) row, with
//     s_j = sum_d  qhat_d . khat_d[i_dj],     qhat_d = q_d / max(||q_d||, eps),
// (llm/models/experts.py:153-163, :327), the gradient with respect to the
// queries q after LayerNorm:
//     ds_j    = w_j * (dw_j - sum_i w_i dw_i)
//     dqhat_d = sum_j ds_j * khat_d[i_dj]
//     dq_d    = (dqhat_d - qhat_d * (qhat_d . dqhat_d)) / ||q_d||        (norm_query)
// The indices are constants of the forward pass and the sub-keys receive no
// gradient (the reference reads them through .data, experts.py:154).  One warp
// per row; the 2k (or nd*k) selected key rows are the only table reads.
#include "common.cuh"
#include "kernels.h"

namespace peer {

namespace {

constexpr int WARPS = 4;
constexpr float NORM_EPS = 1e-12f;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) select_grad_kernel(const SelectGradArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int width = a.Q / a.nd;
    long long total = 1;
    for (int d = 0; d < a.nd; ++d) total *= a.n[d];
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * WARPS + warp; row < a.rows;
         row += static_cast<int64_t>(gridDim.x) * WARPS) {
        // softmax weights and ds, one selected expert per lane
        const bool live = lane < a.k;
        const float s = live ? a.scores[row * a.k + lane] : -INFINITY;
        float mx = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL_MASK, mx, o));
        const float e = live ? expf(s - mx) : 0.f;
        const float w = e / warp_sum(e);
        const float dw = live ? a.grad_weights[row * a.k + lane] : 0.f;
        float ds = w * (dw - warp_sum(w * dw));
        int pid = live ? a.prod_ids[row * a.k + lane] : 0;
        // a grid position outside the key grid is recorded and contributes nothing; it is never used as an address
        if (pid < 0 || pid >= total) {
            if (a.status) atomicMax(a.status, STATUS_BOUNDS);
            pid = 0;
            ds = 0.f;
        }
        for (int d = 0; d < a.nd; ++d) {
            const int my_idx = static_cast<int>((pid / a.stride[d]) % a.n[d]);
            const T* __restrict__ keys = static_cast<const T*>(a.keys[d]);
            // scale of every selected key row: ds_j / max(||k_j||, eps)
            float my_scale = ds;
            if (a.norm_keys) {
                for (int j = 0; j < a.k; ++j) {
                    const int ij = __shfl_sync(FULL_MASK, my_idx, j);
                    const T* kr = keys + static_cast<int64_t>(ij) * width;
                    float ss = 0.f;
                    for (int c = lane; c < width; c += 32) { const float v = to_f32<T>(kr[c]); ss = fmaf(v, v, ss); }
                    ss = warp_sum(ss);
                    if (lane == j) my_scale = ds / fmaxf(sqrtf(ss), NORM_EPS);
                }
            }
            const float* qrow = a.q_ln + row * a.Q + d * width;
            float qq = 0.f;
            for (int c = lane; c < width; c += 32) { const float v = qrow[c]; qq = fmaf(v, v, qq); }
            const float qn = fmaxf(sqrtf(warp_sum(qq)), NORM_EPS);
            // pass 1: dqhat and its projection on qhat; pass 2 recomputes dqhat (cheap) to write dq
            float proj = 0.f;
            for (int pass = 0; pass < 2; ++pass) {
                for (int c0 = 0; c0 < width; c0 += 32) {
                    const int c = c0 + lane;
                    float g = 0.f;
                    for (int j = 0; j < a.k; ++j) {
                        const int ij = __shfl_sync(FULL_MASK, my_idx, j);
                        const float sj = __shfl_sync(FULL_MASK, my_scale, j);
                        if (c < width) g = fmaf(sj, to_f32<T>(keys[static_cast<int64_t>(ij) * width + c]), g);
                    }
                    if (c < width) {
                        if (!a.norm_query) {
                            if (pass == 1) a.grad_q[row * a.Q + d * width + c] = g;
                        } else if (pass == 0) {
                            proj = fmaf(qrow[c] / qn, g, proj);
                        } else {
                            a.grad_q[row * a.Q + d * width + c] = (g - (qrow[c] / qn) * proj) / qn;
                        }
                    }
                }
                if (pass == 0) proj = warp_sum(proj);
            }
        }
    }
}

}  // namespace

cudaError_t launch_select_grad(const SelectGradArgs& a, cudaStream_t s) {
    if (a.rows == 0) return cudaSuccess;
    if (a.nd < 1 || a.nd > 4 || a.k < 1 || a.k > 32 || a.Q % a.nd) return cudaErrorInvalidValue;
    int64_t blocks = (a.rows + WARPS - 1) / WARPS;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (a.act_dtype == PEER_DTYPE_F32) select_grad_kernel<float><<<static_cast<unsigned>(blocks), WARPS * 32, 0, s>>>(a);
    else if (a.act_dtype == PEER_DTYPE_BF16) select_grad_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), WARPS * 32, 0, s>>>(a);
    else if (a.act_dtype == PEER_DTYPE_F16) select_grad_kernel<__half><<<static_cast<unsigned>(blocks), WARPS * 32, 0, s>>>(a);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace peer
