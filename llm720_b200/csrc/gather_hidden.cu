// Expert evaluation and its backward for experts with more than one hidden
// neuron (expert_hidden_size = h > 1), llm/models/experts.py:337-382: the down
// row of an expert is an [h, D] block, the up row a [D_out, h] block,
//     hid_m = act(down[m, :] . x),   y += w * sum_m hid_m * up[:, m].
// The benchmark configurations use single-neuron experts and the specialised
// kernels (gather_eval.cu, gather_grad.cu); this general form covers the
// layers the reference's own tests build (h = 8, tests/test_peer_integration.py:
// 24-111).  One warp per token; the output (forward) or dx (backward) row is
// accumulated in shared memory; element loads are coalesced across the warp
// (consecutive lanes read consecutive elements of a down row, or consecutive
// [h]-element groups of the up block).
#include "common.cuh"
#include "kernels.h"

namespace peer {

namespace {

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int MAX_H = 16;

__device__ __forceinline__ float act_value(float z, int activation) {
    return activation == PEER_ACT_GELU ? gelu_erf(z) : fmaxf(z, 0.f);
}
__device__ __forceinline__ float act_slope(float z, int activation) {
    if (activation != PEER_ACT_GELU) return z > 0.f ? 1.f : 0.f;
    const float cdf = 0.5f * (1.0f + erff(z * 0.70710678118654752440f));
    const float pdf = 0.39894228040143267794f * expf(-0.5f * z * z);
    return cdf + z * pdf;
}

template <typename T>
__global__ void __launch_bounds__(THREADS) gather_hidden_kernel(const GatherArgs a) {
    extern __shared__ float acc_all[];                  // [WARPS][Dout]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* acc = acc_all + static_cast<size_t>(warp) * a.Dout;
    const int h = a.hidden;
    const T* __restrict__ xg = static_cast<const T*>(a.x);
    const T* __restrict__ down = static_cast<const T*>(a.down);
    const T* __restrict__ up = static_cast<const T*>(a.up);
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * WARPS + warp; t < a.T; t += static_cast<int64_t>(gridDim.x) * WARPS) {
        __syncwarp();
        for (int o = lane; o < a.Dout; o += 32) acc[o] = 0.f;
        const T* xr = xg + t * a.D;
        for (int e = 0; e < a.HK; ++e) {
            const int32_t id = __ldg(a.ids + t * a.HK + e);
            const float w = __ldg(a.weights + t * a.HK + e);
            if (static_cast<uint32_t>(id) >= static_cast<uint64_t>(a.N)) {
                if (lane == 0) atomicMax(a.status, STATUS_BOUNDS);
                continue;
            }
            const T* ub = down + static_cast<int64_t>(id) * h * a.D;
            const T* vb = up + static_cast<int64_t>(id) * h * a.Dout;
            float hid[MAX_H];
#pragma unroll
            for (int m = 0; m < MAX_H; ++m) {
                hid[m] = 0.f;
                if (m < h) {
                    float z = 0.f;
                    for (int i = lane; i < a.D; i += 32) z = fmaf(to_f32<T>(ub[m * a.D + i]), to_f32<T>(xr[i]), z);
                    hid[m] = w * act_value(warp_sum(z), a.activation);
                }
            }
            for (int o = lane; o < a.Dout; o += 32) {
                float s = 0.f;
#pragma unroll
                for (int m = 0; m < MAX_H; ++m)
                    if (m < h) s = fmaf(hid[m], to_f32<T>(vb[o * h + m]), s);
                acc[o] += s;
            }
        }
        if (a.out_f32) {
            for (int o = lane; o < a.Dout; o += 32) a.out_f32[t * a.Dout + o] = acc[o];
        } else {
            T* og = static_cast<T*>(a.out);
            const T* rs = static_cast<const T*>(a.residual);
            for (int o = lane; o < a.Dout; o += 32)
                og[t * a.Dout + o] = from_f32<T>(acc[o] + (rs ? to_f32<T>(rs[t * a.Dout + o]) : 0.f));
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(THREADS) gather_hidden_grad_kernel(const GatherGradArgs a) {
    extern __shared__ float dx_all[];                   // [WARPS][D]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* dxs = dx_all + static_cast<size_t>(warp) * a.D;
    const int h = a.hidden;
    const T* __restrict__ xg = static_cast<const T*>(a.x);
    const T* __restrict__ dyg = static_cast<const T*>(a.dy);
    const T* __restrict__ down = static_cast<const T*>(a.down);
    const T* __restrict__ up = static_cast<const T*>(a.up);
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * WARPS + warp; t < a.T; t += static_cast<int64_t>(gridDim.x) * WARPS) {
        __syncwarp();
        for (int i = lane; i < a.D; i += 32) dxs[i] = 0.f;
        const T* xr = xg + t * a.D;
        const T* dyr = dyg + t * a.Dout;
        for (int e = 0; e < a.HK; ++e) {
            const int32_t id = __ldg(a.ids + t * a.HK + e);
            const float w = __ldg(a.weights + t * a.HK + e);
            if (static_cast<uint32_t>(id) >= static_cast<uint64_t>(a.N)) {
                if (lane == 0) { atomicMax(a.status, STATUS_BOUNDS); a.dweights[t * a.HK + e] = 0.f; }
                continue;
            }
            const T* ub = down + static_cast<int64_t>(id) * h * a.D;
            const T* vb = up + static_cast<int64_t>(id) * h * a.Dout;
            float* du = static_cast<float*>(a.d_down) + static_cast<int64_t>(id) * h * a.D;
            float* dv = static_cast<float*>(a.d_up) + static_cast<int64_t>(id) * h * a.Dout;
            float z[MAX_H], g[MAX_H];
#pragma unroll
            for (int m = 0; m < MAX_H; ++m) {
                z[m] = 0.f; g[m] = 0.f;
                if (m < h) {
                    float s = 0.f;
                    for (int i = lane; i < a.D; i += 32) s = fmaf(to_f32<T>(ub[m * a.D + i]), to_f32<T>(xr[i]), s);
                    z[m] = warp_sum(s);
                }
            }
            for (int o = lane; o < a.Dout; o += 32) {
                const float dyo = to_f32<T>(dyr[o]);
#pragma unroll
                for (int m = 0; m < MAX_H; ++m)
                    if (m < h) g[m] = fmaf(to_f32<T>(vb[o * h + m]), dyo, g[m]);
            }
            float dwe = 0.f;
            float cv[MAX_H], dz[MAX_H];
#pragma unroll
            for (int m = 0; m < MAX_H; ++m) {
                cv[m] = 0.f; dz[m] = 0.f;
                if (m < h) {
                    g[m] = warp_sum(g[m]);
                    const float av = act_value(z[m], a.activation);
                    dwe = fmaf(av, g[m], dwe);
                    cv[m] = w * av;
                    dz[m] = w * g[m] * act_slope(z[m], a.activation);
                }
            }
            if (lane == 0) a.dweights[t * a.HK + e] = dwe;
            for (int o = lane; o < a.Dout; o += 32) {
                const float dyo = to_f32<T>(dyr[o]);
#pragma unroll
                for (int m = 0; m < MAX_H; ++m)
                    if (m < h) atomicAdd(dv + o * h + m, cv[m] * dyo);
            }
            for (int i = lane; i < a.D; i += 32) {
                const float xi = to_f32<T>(xr[i]);
                float s = 0.f;
#pragma unroll
                for (int m = 0; m < MAX_H; ++m)
                    if (m < h) {
                        s = fmaf(dz[m], to_f32<T>(ub[m * a.D + i]), s);
                        atomicAdd(du + m * a.D + i, dz[m] * xi);
                    }
                dxs[i] += s;
            }
        }
        for (int i = lane; i < a.D; i += 32) a.dx[t * a.D + i] = dxs[i];
    }
}

template <typename K>
cudaError_t opt_in(K kernel, size_t smem) {
    if (smem <= 48 * 1024) return cudaSuccess;
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
}

unsigned grid_for(int64_t T, int sm_count) {
    int64_t b = (T + WARPS - 1) / WARPS;
    const int64_t cap = static_cast<int64_t>(sm_count) * 8;
    return static_cast<unsigned>(b < cap ? b : cap);
}

}  // namespace

cudaError_t launch_gather_hidden(const GatherArgs& a, cudaStream_t s) {
    if (a.T == 0) return cudaSuccess;
    if (a.hidden < 1 || a.hidden > MAX_H || a.act_dtype != a.table_dtype || a.counts) return cudaErrorInvalidValue;
    const size_t smem = sizeof(float) * WARPS * a.Dout;
    cudaError_t e;
    if (a.act_dtype == PEER_DTYPE_F32) {
        if ((e = opt_in(gather_hidden_kernel<float>, smem)) != cudaSuccess) return e;
        gather_hidden_kernel<float><<<grid_for(a.T, a.sm_count), THREADS, smem, s>>>(a);
    } else if (a.act_dtype == PEER_DTYPE_BF16) {
        if ((e = opt_in(gather_hidden_kernel<__nv_bfloat16>, smem)) != cudaSuccess) return e;
        gather_hidden_kernel<__nv_bfloat16><<<grid_for(a.T, a.sm_count), THREADS, smem, s>>>(a);
    } else if (a.act_dtype == PEER_DTYPE_F16) {
        if ((e = opt_in(gather_hidden_kernel<__half>, smem)) != cudaSuccess) return e;
        gather_hidden_kernel<__half><<<grid_for(a.T, a.sm_count), THREADS, smem, s>>>(a);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_gather_hidden_grad(const GatherGradArgs& a, cudaStream_t s) {
    if (a.T == 0) return cudaSuccess;
    if (a.hidden < 1 || a.hidden > MAX_H || a.act_dtype != a.table_dtype || a.grad_dtype != PEER_DTYPE_F32)
        return cudaErrorInvalidValue;
    const size_t smem = sizeof(float) * WARPS * a.D;
    cudaError_t e;
    if (a.act_dtype == PEER_DTYPE_F32) {
        if ((e = opt_in(gather_hidden_grad_kernel<float>, smem)) != cudaSuccess) return e;
        gather_hidden_grad_kernel<float><<<grid_for(a.T, a.sm_count), THREADS, smem, s>>>(a);
    } else if (a.act_dtype == PEER_DTYPE_BF16) {
        if ((e = opt_in(gather_hidden_grad_kernel<__nv_bfloat16>, smem)) != cudaSuccess) return e;
        gather_hidden_grad_kernel<__nv_bfloat16><<<grid_for(a.T, a.sm_count), THREADS, smem, s>>>(a);
    } else if (a.act_dtype == PEER_DTYPE_F16) {
        if ((e = opt_in(gather_hidden_grad_kernel<__half>, smem)) != cudaSuccess) return e;
        gather_hidden_grad_kernel<__half><<<grid_for(a.T, a.sm_count), THREADS, smem, s>>>(a);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace peer
