// Query stage on CUDA cores: q = x W^T + b, LayerNorm over the head's query
// dimension, per-half L2 normalisation.  Exact fp32 arithmetic; used for fp32
// layers and as the reference the tensor-core path is checked against.
//
// Follows llm/models/experts.py:302-308 (projection, LayerNorm shared by all
// heads) and :156-159 (F.normalize of each query half, eps 1e-12).
#include "common.cuh"
#include "kernels.h"

namespace peer {

namespace {

constexpr int BM = 64;       // tokens per CTA
constexpr int BK = 16;       // reduction slice
constexpr int APAD = 4;
constexpr int THREADS = 256;
constexpr float LN_EPS = 1e-5f;
constexpr float NORM_EPS = 1e-12f;

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    v[0] = bf16_lo(t.x); v[1] = bf16_hi(t.x); v[2] = bf16_lo(t.y); v[3] = bf16_hi(t.y);
}

template <>
__device__ __forceinline__ void load4<__half>(const __half* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

// One CTA: BM tokens x one head.  Warp w owns token rows w*8..w*8+7 whole
// (columns lane + 32*j), so the LayerNorm and the half norms are warp
// reductions and nothing is staged through shared memory.
template <typename T, int TN>
__global__ void __launch_bounds__(THREADS)
query_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                  const T* __restrict__ ln_w, const T* __restrict__ ln_b,
                  float* __restrict__ q_ln_out, float* __restrict__ q_hat_out,
                  int64_t Ttok, int D, int H, int Q, int layer_norm, int norm_query) {
    constexpr int QP = 32 * TN;
    __shared__ __align__(16) float As[BK][BM + APAD];
    __shared__ __align__(16) float Bs[BK][QP];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t m0 = static_cast<int64_t>(blockIdx.x) * BM;
    const int h = blockIdx.y;

    float acc[8][TN];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    const int ar = tid >> 2, ak = (tid & 3) * 4;     // A loader: row, k offset
    for (int k0 = 0; k0 < D; k0 += BK) {
        {   // x tile, stored transposed
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            const int64_t r = m0 + ar;
            if (r < Ttok && k0 + ak < D) load4<T>(x + r * D + k0 + ak, v);
#pragma unroll
            for (int e = 0; e < 4; ++e) As[ak + e][ar] = v[e];
        }
        for (int c = tid; c < QP; c += THREADS) {    // weight tile
#pragma unroll
            for (int kq = 0; kq < BK; kq += 4) {
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (c < Q && k0 + kq < D)
                    load4<T>(w + (static_cast<int64_t>(h) * Q + c) * D + k0 + kq, v);
#pragma unroll
                for (int e = 0; e < 4; ++e) Bs[kq + e][c] = v[e];
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[kk][warp * 8]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[kk][warp * 8 + 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            float b[TN];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[kk][lane + 32 * j];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

    // Epilogue: bias, LayerNorm, half norms.
    float bj[TN], gj[TN], oj[TN];
#pragma unroll
    for (int j = 0; j < TN; ++j) {
        const int c = lane + 32 * j;
        const bool ok = c < Q;
        bj[j] = (ok && bias) ? to_f32<T>(bias[h * Q + c]) : 0.f;
        gj[j] = (ok && ln_w) ? to_f32<T>(ln_w[c]) : 1.f;
        oj[j] = (ok && ln_b) ? to_f32<T>(ln_b[c]) : 0.f;
    }
    const int half = Q / 2;
    const float invQ = 1.0f / static_cast<float>(Q);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t r = m0 + warp * 8 + i;
        float v[TN];
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const bool ok = lane + 32 * j < Q;
            v[j] = ok ? acc[i][j] + bj[j] : 0.f;
            s += v[j];
        }
        if (layer_norm) {
            const float mean = warp_sum(s) * invQ;
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const float d = (lane + 32 * j < Q) ? v[j] - mean : 0.f;
                ss = fmaf(d, d, ss);
            }
            const float rstd = 1.0f / sqrtf(warp_sum(ss) * invQ + LN_EPS);
#pragma unroll
            for (int j = 0; j < TN; ++j)
                v[j] = (lane + 32 * j < Q) ? (v[j] - mean) * rstd * gj[j] + oj[j] : 0.f;
        }
        if (r < Ttok && q_ln_out) {
#pragma unroll
            for (int j = 0; j < TN; ++j)
                if (lane + 32 * j < Q) q_ln_out[(r * H + h) * Q + lane + 32 * j] = v[j];
        }
        if (q_hat_out) {
            if (norm_query) {
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    const int c = lane + 32 * j;
                    if (c < half) s0 = fmaf(v[j], v[j], s0);
                    else if (c < Q) s1 = fmaf(v[j], v[j], s1);
                }
                const float n0 = fmaxf(sqrtf(warp_sum(s0)), NORM_EPS);
                const float n1 = fmaxf(sqrtf(warp_sum(s1)), NORM_EPS);
#pragma unroll
                for (int j = 0; j < TN; ++j) v[j] = v[j] / ((lane + 32 * j < half) ? n0 : n1);
            }
            if (r < Ttok) {
#pragma unroll
                for (int j = 0; j < TN; ++j)
                    if (lane + 32 * j < Q) q_hat_out[(r * H + h) * Q + lane + 32 * j] = v[j];
            }
        }
    }
}

// warp per row: out = in / max(||in||, eps)  (or a plain widening copy)
template <typename T>
__global__ void normalize_rows_kernel(const T* __restrict__ in, int64_t rows, int width, int do_norm,
                                      int transpose_out, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (r >= rows) return;
    float ss = 0.f;
    for (int c = lane; c < width; c += 32) {
        const float v = to_f32<T>(in[r * width + c]);
        ss = fmaf(v, v, ss);
    }
    const float n = do_norm ? fmaxf(sqrtf(warp_sum(ss)), NORM_EPS) : 1.0f;
    for (int c = lane; c < width; c += 32) {
        const float v = to_f32<T>(in[r * width + c]);
        const float y = do_norm ? v / n : v;
        if (transpose_out) out[c * rows + r] = y;
        else out[r * width + c] = y;
    }
}

// out (optional): the normalised values in fp32.  split (optional): the same values as three bf16 terms
// (hi + mid + lo carry the 24 bits of the fp32 value), the three arrays split_stride elements apart: the
// operand format of the tensor-core select kernel.
__global__ void normalize_halves_kernel(const float* __restrict__ q, int64_t rows, int Q, int do_norm,
                                        float* __restrict__ out, __nv_bfloat16* __restrict__ split,
                                        int64_t split_stride) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (r >= rows) return;
    const int half = Q / 2;
    float s0 = 0.f, s1 = 0.f;
    for (int c = lane; c < Q; c += 32) {
        const float v = q[r * Q + c];
        if (c < half) s0 = fmaf(v, v, s0); else s1 = fmaf(v, v, s1);
    }
    const float n0 = do_norm ? fmaxf(sqrtf(warp_sum(s0)), NORM_EPS) : 1.0f;
    const float n1 = do_norm ? fmaxf(sqrtf(warp_sum(s1)), NORM_EPS) : 1.0f;
    for (int c = lane; c < Q; c += 32) {
        const float v = q[r * Q + c];
        const float y = do_norm ? v / (c < half ? n0 : n1) : v;
        if (out) out[r * Q + c] = y;
        if (split) {
            float rem = y;
            const __nv_bfloat16 hi = __float2bfloat16_rn(rem); rem -= __bfloat162float(hi);
            const __nv_bfloat16 mid = __float2bfloat16_rn(rem); rem -= __bfloat162float(mid);
            split[r * Q + c] = hi;
            split[split_stride + r * Q + c] = mid;
            split[2 * split_stride + r * Q + c] = __float2bfloat16_rn(rem);
        }
    }
}

template <typename T>
cudaError_t launch_query_t(const QueryArgs& a, cudaStream_t s) {
    const dim3 grid(static_cast<unsigned>((a.T + BM - 1) / BM), a.H);
    const T* x = static_cast<const T*>(a.x);
    const T* w = static_cast<const T*>(a.w);
    const T* b = static_cast<const T*>(a.b);
    const T* g = static_cast<const T*>(a.ln_w);
    const T* o = static_cast<const T*>(a.ln_b);
#define PEER_Q_LAUNCH(TN)                                                                         \
    query_simt_kernel<T, TN><<<grid, THREADS, 0, s>>>(x, w, b, g, o, a.q_ln_out, a.q_hat_out, a.T, \
                                                      a.D, a.H, a.Q, a.layer_norm, a.norm_query)
    if (a.Q <= 32) PEER_Q_LAUNCH(1);
    else if (a.Q <= 64) PEER_Q_LAUNCH(2);
    else if (a.Q <= 128) PEER_Q_LAUNCH(4);
    else PEER_Q_LAUNCH(8);
#undef PEER_Q_LAUNCH
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_query_simt(const QueryArgs& a, cudaStream_t s) {
    if (a.T == 0) return cudaSuccess;
    if (a.act_dtype == PEER_DTYPE_F32) return launch_query_t<float>(a, s);
    if (a.act_dtype == PEER_DTYPE_F16) return launch_query_t<__half>(a, s);
    return launch_query_t<__nv_bfloat16>(a, s);
}

cudaError_t launch_normalize_rows(const void* in, int in_dtype, int64_t rows, int width, int do_norm,
                                  int transpose_out, float* out, cudaStream_t s) {
    if (rows == 0) return cudaSuccess;
    const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
    if (in_dtype == PEER_DTYPE_F32)
        normalize_rows_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(in), rows, width,
                                                            do_norm, transpose_out, out);
    else if (in_dtype == PEER_DTYPE_F16)
        normalize_rows_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const __half*>(in), rows, width, do_norm,
                                                             transpose_out, out);
    else
        normalize_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(
            static_cast<const __nv_bfloat16*>(in), rows, width, do_norm, transpose_out, out);
    return cudaGetLastError();
}

cudaError_t launch_normalize_halves(const float* q, int64_t rows, int Q, int do_norm, float* out,
                                    cudaStream_t s, __nv_bfloat16* split, int64_t split_stride) {
    if (rows == 0) return cudaSuccess;
    const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
    normalize_halves_kernel<<<blocks, 256, 0, s>>>(q, rows, Q, do_norm, out, split, split_stride);
    return cudaGetLastError();
}

}  // namespace peer
