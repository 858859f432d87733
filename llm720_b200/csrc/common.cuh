// Shared device helpers for the PEER kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "../../include/peer_b200.h"

namespace peer {

constexpr unsigned FULL_MASK = 0xffffffffu;

// Device status word values (0 = fine).  Written with atomicMax so the most
// severe condition survives.
constexpr int STATUS_OK = 0;
constexpr int STATUS_BOUNDS = 1;
constexpr int STATUS_TIMEOUT = 2;

// Upper bound on the polls of one mbarrier wait.  Each poll is a try_wait
// that itself blocks for a hardware-defined slice, so this is far more than
// any real copy needs and still ends in well under a second.
constexpr uint32_t WAIT_POLL_LIMIT = 1u << 20;

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL_MASK, v, o);
    return v;
}

__device__ __forceinline__ float gelu_erf(float z) {
    // exact (erf) GELU, the default of torch.nn.functional.gelu
    return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
}

// ---------------------------------------------------------------------------
// Warp-distributed sorted list: lane j (j < cap) holds the j-th best
// (value, index) pair.  Order: larger value first; equal values -> smaller
// index first.  An empty slot holds (-inf, INT_MAX).
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool ranks_before(float v1, int i1, float v2, int i2) {
    return (v1 > v2) || (v1 == v2 && i1 < i2);
}

// Insert the warp-uniform candidate (cv, ci); no-op when it does not make the list.
__device__ __forceinline__ void warp_list_insert(float& val, int& idx, float cv, int ci, int cap,
                                                 int lane) {
    const bool ahead = (lane < cap) && ranks_before(val, idx, cv, ci);
    const int pos = __popc(__ballot_sync(FULL_MASK, ahead));
    const float upv = __shfl_up_sync(FULL_MASK, val, 1);
    const int upi = __shfl_up_sync(FULL_MASK, idx, 1);
    if (pos < cap) {
        if (lane == pos) { val = cv; idx = ci; }
        else if (lane > pos && lane < cap) { val = upv; idx = upi; }
    }
}

// Offer one candidate per lane (lanes with `valid` false offer nothing).
__device__ __forceinline__ void warp_list_offer(float& val, int& idx, float cv, int ci, bool valid,
                                                int cap, int lane) {
    const float tv = __shfl_sync(FULL_MASK, val, cap - 1);
    const int ti = __shfl_sync(FULL_MASK, idx, cap - 1);
    unsigned m = __ballot_sync(FULL_MASK, valid && ranks_before(cv, ci, tv, ti));
    while (m) {
        const int src = __ffs(m) - 1;
        m &= m - 1;
        const float bv = __shfl_sync(FULL_MASK, cv, src);
        const int bi = __shfl_sync(FULL_MASK, ci, src);
        warp_list_insert(val, idx, bv, bi, cap, lane);
    }
}

// ---------------------------------------------------------------------------
// mbarrier + 1-D bulk copy (global -> this CTA's shared memory), sm_90+ PTX.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and records STATUS_TIMEOUT) if the phase did
// not complete within WAIT_POLL_LIMIT polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
    for (uint32_t i = 0; i < WAIT_POLL_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicMax(status, STATUS_TIMEOUT);
    return false;
}
// The same wait with a suspend-time hint of a microsecond: the thread sleeps in the barrier unit instead of
// polling.  For the tensor-core kernels, where waiting roles (producer, MMA issuer, scan warps between chunks)
// would otherwise spend issue slots the working warps need (query 2 %, selection 3 % faster); the expert stage
// keeps the plain form, its warps want to be back as soon as a row lands (1-2 % slower with the hint).
__device__ __forceinline__ bool mbar_wait_hint(uint32_t bar, uint32_t parity, int* status) {
    for (uint32_t i = 0; i < WAIT_POLL_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");
        if (ok) return true;
    }
    atomicMax(status, STATUS_TIMEOUT);
    return false;
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// dst/src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}

}  // namespace peer
