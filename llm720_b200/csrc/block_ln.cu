// LayerNorm over the model dimension in front of the layer: the `ln_2` of the
// reference's TransformerBlock (llm/models/foundation.py:118, 196-199;
// nn.LayerNorm with fp32 parameters, biased variance, eps inside the square
// root).  One warp per token row; statistics in fp32; output in the layer's
// dtype, which is what the query projection and the expert stage then read.
#include "common.cuh"
#include "kernels.h"

namespace peer {

namespace {

template <typename T>
__global__ void block_ln_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                float eps, int64_t rows, int D, T* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (r >= rows) return;
    const T* xr = x + r * D;
    float s = 0.f;
    for (int c = lane; c < D; c += 32) s += to_f32<T>(xr[c]);
    const float mean = warp_sum(s) / static_cast<float>(D);
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) { const float d = to_f32<T>(xr[c]) - mean; ss = fmaf(d, d, ss); }
    const float rstd = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(D) + eps);
    for (int c = lane; c < D; c += 32) {
        float v = (to_f32<T>(xr[c]) - mean) * rstd;
        if (w) v *= w[c];
        if (b) v += b[c];
        out[r * D + c] = from_f32<T>(v);
    }
}

}  // namespace

cudaError_t launch_block_ln(const void* x, int act_dtype, int64_t rows, int D, const float* w, const float* b, float eps,
                            void* out, cudaStream_t s) {
    if (rows == 0) return cudaSuccess;
    const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
    if (act_dtype == PEER_DTYPE_F32)
        block_ln_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), w, b, eps, rows, D, static_cast<float*>(out));
    else if (act_dtype == PEER_DTYPE_BF16)
        block_ln_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), w, b, eps, rows, D,
                                                              static_cast<__nv_bfloat16*>(out));
    else if (act_dtype == PEER_DTYPE_F16)
        block_ln_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const __half*>(x), w, b, eps, rows, D, static_cast<__half*>(out));
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace peer
