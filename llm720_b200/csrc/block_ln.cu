// LayerNorm over the model dimension in front of the layer: the `ln_2` of the
// reference's TransformerBlock (llm/models/foundation.py:118, 196-199;
// nn.LayerNorm with fp32 parameters, biased variance, eps inside the square
// root).  One warp per token row; statistics in fp32; output in the layer's
// dtype, which is what the query projection and the expert stage then read.
// Rows that are a whole number of 512-byte warp loads (d_model 2048 or 4096 in
// bf16) stay in registers between the passes; other widths take the plain loop.
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

// Rows of NCH * 32 sixteen-byte chunks (2-byte types: NCH * 256 elements): the row is read once with 16-byte
// loads, stays in registers for both statistics passes and is written with 16-byte stores.
template <typename T, int NCH>
__global__ void __launch_bounds__(256) block_ln_vec_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                           const float* __restrict__ b, float eps, int64_t rows, int D,
                                                           T* __restrict__ out) {
    constexpr int EPC = 16 / sizeof(T);
    const int lane = threadIdx.x & 31;
    const int64_t r = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (r >= rows) return;
    const uint4* xr = reinterpret_cast<const uint4*>(x + r * D);
    float v[NCH * EPC];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const uint4 raw = __ldg(xr + lane + 32 * i);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int q = 0; q < EPC; ++q) { v[i * EPC + q] = to_f32<T>(e[q]); s += v[i * EPC + q]; }
    }
    const float mean = warp_sum(s) / static_cast<float>(D);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NCH * EPC; ++i) { const float d = v[i] - mean; ss = fmaf(d, d, ss); }
    const float rstd = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(D) + eps);
    uint4* orow = reinterpret_cast<uint4*>(out + r * D);
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c0 = (lane + 32 * i) * EPC;
        uint4 o;
        T* e = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int q = 0; q < EPC; ++q) {
            float y = (v[i * EPC + q] - mean) * rstd;
            if (w) y *= __ldg(w + c0 + q);
            if (b) y += __ldg(b + c0 + q);
            e[q] = from_f32<T>(y);
        }
        orow[lane + 32 * i] = o;
    }
}

template <typename T>
cudaError_t launch_t(const T* x, const float* w, const float* b, float eps, int64_t rows, int D, T* out, cudaStream_t s) {
    const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
    constexpr int EPC = 16 / sizeof(T);
    const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
    const int per_lane = D / (32 * EPC);
    if (aligned && D % (32 * EPC) == 0) {
        if (per_lane == 1) { block_ln_vec_kernel<T, 1><<<blocks, 256, 0, s>>>(x, w, b, eps, rows, D, out); return cudaGetLastError(); }
        if (per_lane == 2) { block_ln_vec_kernel<T, 2><<<blocks, 256, 0, s>>>(x, w, b, eps, rows, D, out); return cudaGetLastError(); }
        if (per_lane == 4) { block_ln_vec_kernel<T, 4><<<blocks, 256, 0, s>>>(x, w, b, eps, rows, D, out); return cudaGetLastError(); }
        if (per_lane == 8) { block_ln_vec_kernel<T, 8><<<blocks, 256, 0, s>>>(x, w, b, eps, rows, D, out); return cudaGetLastError(); }
        if (per_lane == 16 && sizeof(T) == 2) { block_ln_vec_kernel<T, 16><<<blocks, 256, 0, s>>>(x, w, b, eps, rows, D, out); return cudaGetLastError(); }
    }
    block_ln_kernel<T><<<blocks, 256, 0, s>>>(x, w, b, eps, rows, D, out);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_block_ln(const void* x, int act_dtype, int64_t rows, int D, const float* w, const float* b, float eps,
                            void* out, cudaStream_t s) {
    if (rows == 0) return cudaSuccess;
    if (act_dtype == PEER_DTYPE_F32)
        return launch_t<float>(static_cast<const float*>(x), w, b, eps, rows, D, static_cast<float*>(out), s);
    if (act_dtype == PEER_DTYPE_BF16)
        return launch_t<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(x), w, b, eps, rows, D, static_cast<__nv_bfloat16*>(out), s);
    if (act_dtype == PEER_DTYPE_F16)
        return launch_t<__half>(static_cast<const __half*>(x), w, b, eps, rows, D, static_cast<__half*>(out), s);
    return cudaErrorInvalidValue;
}

}  // namespace peer
