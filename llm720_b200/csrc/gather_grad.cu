// Backward of the expert evaluation
//     y[t] = sum_j w[t,j] * act(u_j . x[t]) * v_j          (u_j, v_j = rows ids[t,j] of the tables)
// for a given dy[t]:
//     g_j      = v_j . dy[t]
//     dw[t,j]  = act(z_j) * g_j                             z_j = u_j . x[t]
//     dz_j     = w[t,j] * g_j * act'(z_j)
//     dx[t]    = sum_j dz_j * u_j
//     dU[id_j] += dz_j * x[t]                               (sparse rows of a dense fp32 table)
//     dV[id_j] += w[t,j] * act(z_j) * dy[t]
//
// These are the gradients autograd derives for llm/models/experts.py:332-382
// (embedding lookups, two batched matmuls, activation, score weighting, the
// sums over slots and heads); the reference test that exercises them is
// tests/test_peer_integration.py:181-192.
//
// One warp owns one token: x[t], dy[t] and the dx accumulator stay in its
// registers; the rows are read with 16-byte loads and the table gradients are
// accumulated with vector reductions (red.global.add.v4.f32) into fp32 tables,
// so tokens that share an expert need no sorting or locking.  Rows are read
// twice (dot products, then the updates); the second read hits L1/L2.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace peer {

namespace {

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void red_add_v4_bf16x2(void* addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// one 16-byte chunk of a row (table or activation storage) as fp32 values
template <typename T> struct Chunk16;
template <> struct Chunk16<float> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void decode(const uint4& c, float (&f)[N]) {
        f[0] = __uint_as_float(c.x); f[1] = __uint_as_float(c.y); f[2] = __uint_as_float(c.z); f[3] = __uint_as_float(c.w);
    }
};
template <> struct Chunk16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void decode(const uint4& c, float (&f)[N]) {
        f[0] = bf16_lo(c.x); f[1] = bf16_hi(c.x); f[2] = bf16_lo(c.y); f[3] = bf16_hi(c.y);
        f[4] = bf16_lo(c.z); f[5] = bf16_hi(c.z); f[6] = bf16_lo(c.w); f[7] = bf16_hi(c.w);
    }
};

// sum of the 8 products of two 16-byte chunks of bf16 values, added to d: mixed-precision FMAs take the bf16
// operands as they are stored (a bf16 x bf16 product is exact in fp32, so this equals widening first)
__device__ __forceinline__ void dot8_bf16(const uint4& a, const uint4& b, float& d) {
    asm("{\n\t"
        ".reg .b16 a0, a1, b0, b1;\n\t"
        "mov.b32 {a0, a1}, %1;\n\tmov.b32 {b0, b1}, %5;\n\t"
        "fma.rn.f32.bf16 %0, a0, b0, %0;\n\tfma.rn.f32.bf16 %0, a1, b1, %0;\n\t"
        "mov.b32 {a0, a1}, %2;\n\tmov.b32 {b0, b1}, %6;\n\t"
        "fma.rn.f32.bf16 %0, a0, b0, %0;\n\tfma.rn.f32.bf16 %0, a1, b1, %0;\n\t"
        "mov.b32 {a0, a1}, %3;\n\tmov.b32 {b0, b1}, %7;\n\t"
        "fma.rn.f32.bf16 %0, a0, b0, %0;\n\tfma.rn.f32.bf16 %0, a1, b1, %0;\n\t"
        "mov.b32 {a0, a1}, %4;\n\tmov.b32 {b0, b1}, %8;\n\t"
        "fma.rn.f32.bf16 %0, a0, b0, %0;\n\tfma.rn.f32.bf16 %0, a1, b1, %0;\n\t"
        "}"
        : "+f"(d)
        : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w));
}

__device__ __forceinline__ float act_value(float z, int activation) {
    return activation == PEER_ACT_GELU ? gelu_erf(z) : fmaxf(z, 0.f);
}
__device__ __forceinline__ float act_slope(float z, int activation) {
    if (activation != PEER_ACT_GELU) return z > 0.f ? 1.f : 0.f;
    // d/dz [ z * Phi(z) ] = Phi(z) + z * phi(z)
    const float cdf = 0.5f * (1.0f + erff(z * 0.70710678118654752440f));
    const float pdf = 0.39894228040143267794f * expf(-0.5f * z * z);
    return cdf + z * pdf;
}

struct GradParams {
    const void* x; const void* dy; const int32_t* ids; const float* weights;
    const char* down; const char* up;
    void* d_down; void* d_up; float* dx; float* dweights;
    int64_t T; int HK; int64_t N; int D, Dout; int activation; int* status;
    int nch_u, nch_v;          // 16-byte chunks per down / up row (table storage)
};

// XT = TT here (fp32 layer with fp32 tables, bf16 layer with bf16 tables), so a 16-byte chunk of x or
// dy covers the same elements as a 16-byte chunk of a table row.
// LP: the table gradients are accumulated in the tables' own 16-bit type (what the reference's bf16 training
// does: its embedding gradients are bf16) instead of fp32: half the read-modify-write bytes, no cast afterwards.
template <typename XT, int CH, bool LP>
__global__ void __launch_bounds__(THREADS) gather_grad_kernel(const GradParams p) {
    constexpr int EPC = Chunk16<XT>::N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row_u = static_cast<uint32_t>(p.nch_u) * 16u, row_v = static_cast<uint32_t>(p.nch_v) * 16u;
    const char* __restrict__ xg = static_cast<const char*>(p.x);
    const char* __restrict__ dyg = static_cast<const char*>(p.dy);
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * WARPS;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * WARPS + warp; t < p.T; t += nwarps) {
        uint4 xc[CH], dyc[CH];                   // the token's rows in storage form
        float dxa[CH * EPC];
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int c = lane + 32 * i;
            xc[i] = c < p.nch_u ? __ldg(reinterpret_cast<const uint4*>(xg + t * row_u) + c) : make_uint4(0u, 0u, 0u, 0u);
            dyc[i] = c < p.nch_v ? __ldg(reinterpret_cast<const uint4*>(dyg + t * row_v) + c) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int q = 0; q < EPC; ++q) dxa[i * EPC + q] = 0.f;
        }
        for (int e = 0; e < p.HK; ++e) {
            const int32_t id = __ldg(p.ids + t * p.HK + e);
            const float w = __ldg(p.weights + t * p.HK + e);
            if (static_cast<uint32_t>(id) >= static_cast<uint64_t>(p.N)) {      // recorded and skipped
                if (lane == 0) { atomicMax(p.status, STATUS_BOUNDS); p.dweights[t * p.HK + e] = 0.f; }
                continue;
            }
            const uint4* __restrict__ ur = reinterpret_cast<const uint4*>(p.down + static_cast<int64_t>(id) * row_u);
            const uint4* __restrict__ vr = reinterpret_cast<const uint4*>(p.up + static_cast<int64_t>(id) * row_v);
            float z = 0.f, g = 0.f;
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const int c = lane + 32 * i;
                if constexpr (sizeof(XT) == 2) {
                    if (c < p.nch_u) dot8_bf16(__ldg(ur + c), xc[i], z);
                    if (c < p.nch_v) dot8_bf16(__ldg(vr + c), dyc[i], g);
                } else {
                    float a[EPC], b[EPC];
                    if (c < p.nch_u) {
                        Chunk16<XT>::decode(__ldg(ur + c), a);
                        Chunk16<XT>::decode(xc[i], b);
#pragma unroll
                        for (int q = 0; q < EPC; ++q) z = fmaf(a[q], b[q], z);
                    }
                    if (c < p.nch_v) {
                        Chunk16<XT>::decode(__ldg(vr + c), a);
                        Chunk16<XT>::decode(dyc[i], b);
#pragma unroll
                        for (int q = 0; q < EPC; ++q) g = fmaf(a[q], b[q], g);
                    }
                }
            }
            z = warp_sum(z);
            g = warp_sum(g);
            const float av = act_value(z, p.activation);
            if (lane == 0) p.dweights[t * p.HK + e] = av * g;
            const float cv = w * av;
            const float dz = w * g * act_slope(z, p.activation);
            using GT = typename std::conditional<LP, XT, float>::type;
            GT* __restrict__ du = static_cast<GT*>(p.d_down) + static_cast<int64_t>(id) * p.D;
            GT* __restrict__ dv = static_cast<GT*>(p.d_up) + static_cast<int64_t>(id) * p.Dout;
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const int c = lane + 32 * i;
                float a[EPC], b[EPC];
                if (c < p.nch_v) {
                    Chunk16<XT>::decode(dyc[i], b);
                    if constexpr (LP && sizeof(XT) == 2) {
                        red_add_v4_bf16x2(dv + c * EPC, pack2(cv * b[0], cv * b[1]), pack2(cv * b[2], cv * b[3]),
                                          pack2(cv * b[4], cv * b[5]), pack2(cv * b[6], cv * b[7]));
                    } else {
#pragma unroll
                        for (int q = 0; q < EPC; q += 4)
                            red_add_v4(reinterpret_cast<float*>(dv) + c * EPC + q, cv * b[q], cv * b[q + 1], cv * b[q + 2], cv * b[q + 3]);
                    }
                }
                if (c < p.nch_u) {
                    Chunk16<XT>::decode(__ldg(ur + c), a);
                    Chunk16<XT>::decode(xc[i], b);
#pragma unroll
                    for (int q = 0; q < EPC; ++q) dxa[i * EPC + q] = fmaf(dz, a[q], dxa[i * EPC + q]);
                    if constexpr (LP && sizeof(XT) == 2) {
                        red_add_v4_bf16x2(du + c * EPC, pack2(dz * b[0], dz * b[1]), pack2(dz * b[2], dz * b[3]),
                                          pack2(dz * b[4], dz * b[5]), pack2(dz * b[6], dz * b[7]));
                    } else {
#pragma unroll
                        for (int q = 0; q < EPC; q += 4)
                            red_add_v4(reinterpret_cast<float*>(du) + c * EPC + q, dz * b[q], dz * b[q + 1], dz * b[q + 2], dz * b[q + 3]);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int c = lane + 32 * i;
            if (c < p.nch_u) {
#pragma unroll
                for (int q = 0; q < EPC; q += 4)
                    *reinterpret_cast<float4*>(p.dx + t * p.D + c * EPC + q) =
                        make_float4(dxa[i * EPC + q], dxa[i * EPC + q + 1], dxa[i * EPC + q + 2], dxa[i * EPC + q + 3]);
            }
        }
    }
}

template <typename XT, int CH, bool LP>
cudaError_t launch_t(const GradParams& p, int sm_count, cudaStream_t s) {
    int64_t ctas = (p.T + WARPS - 1) / WARPS;
    const int64_t cap = static_cast<int64_t>(sm_count) * 4;      // a few CTAs per SM, grid-stride over tokens
    if (ctas > cap) ctas = cap;
    gather_grad_kernel<XT, CH, LP><<<static_cast<unsigned>(ctas), THREADS, 0, s>>>(p);
    return cudaGetLastError();
}

template <typename XT, bool LP>
cudaError_t launch_ch(const GradParams& p, int sm_count, cudaStream_t s) {
    const int max_ch = p.nch_u > p.nch_v ? p.nch_u : p.nch_v;
    const int need = (max_ch + 31) / 32;
    if (need <= 1) return launch_t<XT, 1, LP>(p, sm_count, s);
    if (need <= 2) return launch_t<XT, 2, LP>(p, sm_count, s);
    if (need <= 4) return launch_t<XT, 4, LP>(p, sm_count, s);
    if (need <= 8) return launch_t<XT, 8, LP>(p, sm_count, s);
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_gather_grad(const GatherGradArgs& a, cudaStream_t s) {
    if (a.T == 0) return cudaSuccess;
    if (a.act_dtype != a.table_dtype) return cudaErrorInvalidValue;
    const int tb = a.table_dtype == PEER_DTYPE_F32 ? 4 : 2;
    if ((a.D * tb) % 16 || (a.Dout * tb) % 16) return cudaErrorInvalidValue;
    GradParams p;
    p.x = a.x; p.dy = a.dy; p.ids = a.ids; p.weights = a.weights;
    p.down = static_cast<const char*>(a.down); p.up = static_cast<const char*>(a.up);
    p.d_down = a.d_down; p.d_up = a.d_up; p.dx = a.dx; p.dweights = a.dweights;
    p.T = a.T; p.HK = a.HK; p.N = a.N; p.D = a.D; p.Dout = a.Dout; p.activation = a.activation; p.status = a.status;
    p.nch_u = a.D * tb / 16; p.nch_v = a.Dout * tb / 16;
    if (a.act_dtype == PEER_DTYPE_F32) return launch_ch<float, false>(p, a.sm_count, s);       // fp32 either way
    if (a.act_dtype == PEER_DTYPE_BF16)
        return a.grad_dtype == PEER_DTYPE_BF16 ? launch_ch<__nv_bfloat16, true>(p, a.sm_count, s)
                                               : launch_ch<__nv_bfloat16, false>(p, a.sm_count, s);
    return cudaErrorInvalidValue;
}

}  // namespace peer
