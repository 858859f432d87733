// Expert evaluation: for every token, stream the selected experts' down rows
// u_i and up rows v_i out of HBM, compute act(u_i . x) and accumulate
// w_i * act(u_i . x) * v_i.  Nothing but the output row is written.
//
// Replaces llm/models/experts.py:332-382 (embedding lookups that materialise
// two [T,H,k,D] tensors, two batched matmuls, the score weighting and both
// reductions) with one pass over the selected rows.
//
// Organisation: one WARP owns one token.  The token's activation row and its
// fp32 output accumulator live in that warp's registers for the whole token,
// so no cross-warp reduction or CTA barrier is ever needed.  Each warp has a
// private ring of row buffers in shared memory that lane 0 keeps full with
// 1-D bulk copies (cp.async.bulk, completion on an mbarrier); u_0, v_0, u_1,
// v_1 ... are issued STAGES rows ahead of their use, which is what keeps
// enough bytes in flight (about 190 KB per SM) to cover HBM latency.
// Every wait is bounded; a wait that runs out records STATUS_TIMEOUT and the
// warp stops, it never spins forever.
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace peer {

namespace {

constexpr int MAX_STAGES = 12;
constexpr int MAX_SMEM = 227 * 1024;

// Warps per CTA (one CTA per SM) and ring bytes per warp.  Rows of a 16-bit or 32-bit table keep the memory
// system busy with 8 warps; FP8 rows carry half the bytes per decoded element, so that instance is bound by
// the time one warp needs for a row pair's instructions and runs 16 warps (all that 128 registers per thread
// allow) with smaller rings and packed f16 activations.
// W10 (bf16 rows of 4 KB only): ten warps on 20 KB rings, for layers whose selected rows stay L2-resident (the
// reference's id arithmetic addresses at most n0 + n1 - 1 rows): there the stage is bound by instruction issue, not
// by memory, and more warps help; with rows streaming from HBM eight warps on deeper rings are faster.
template <typename TT, int CH, bool W10, bool TIER = false> struct WarpCfg {
    static constexpr bool MANY = sizeof(TT) == 1 && CH <= 4;      // rows up to 2048 elements: registers allow 16 warps
    static constexpr bool TEN = W10 && sizeof(TT) == 2 && CH == 8;
    static constexpr int WARPS = MANY ? (TIER ? 14 : 16) : (TEN ? 10 : 8);   // TIER: its slot map needs the shared memory of two warps
    static constexpr int RING_BYTES = MANY ? 12 * 1024 : (TEN ? 20 * 1024 : 24 * 1024);
};

template <typename TT, int CH, bool W10, bool TIER = false> struct RingCfg {
    static constexpr int SLOT = CH * 512;   // bytes: one row of up to CH 16-byte chunks per lane
    static constexpr int ST0 = WarpCfg<TT, CH, W10, TIER>::RING_BYTES / SLOT;
    static constexpr int STAGES = ST0 > MAX_STAGES ? MAX_STAGES : (ST0 < 2 ? 2 : ST0);
};

// ---- 16-byte chunk decoders: table storage -> fp32 -------------------------
template <typename TT> struct Chunk;
template <> struct Chunk<float> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void decode(const uint4& c, float (&f)[N]) {
        f[0] = __uint_as_float(c.x); f[1] = __uint_as_float(c.y);
        f[2] = __uint_as_float(c.z); f[3] = __uint_as_float(c.w);
    }
};
template <> struct Chunk<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void decode(const uint4& c, float (&f)[N]) {
        f[0] = bf16_lo(c.x); f[1] = bf16_hi(c.x); f[2] = bf16_lo(c.y); f[3] = bf16_hi(c.y);
        f[4] = bf16_lo(c.z); f[5] = bf16_hi(c.z); f[6] = bf16_lo(c.w); f[7] = bf16_hi(c.w);
    }
};
template <> struct Chunk<__nv_fp8_e4m3> {
    static constexpr int N = 16;
    __device__ static __forceinline__ void pair(uint32_t two_bytes, float& a, float& b) {
        const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two_bytes), __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
        a = f.x; b = f.y;
    }
    __device__ static __forceinline__ void decode(const uint4& c, float (&f)[N]) {
        pair(c.x & 0xffffu, f[0], f[1]);  pair(c.x >> 16, f[2], f[3]);
        pair(c.y & 0xffffu, f[4], f[5]);  pair(c.y >> 16, f[6], f[7]);
        pair(c.z & 0xffffu, f[8], f[9]);  pair(c.z >> 16, f[10], f[11]);
        pair(c.w & 0xffffu, f[12], f[13]); pair(c.w >> 16, f[14], f[15]);
    }
};

// ---- activation row: N consecutive elements of XT -> fp32 ------------------
template <typename XT, int N> struct XIo;
template <> struct XIo<float, 4> {
    __device__ static __forceinline__ void load(const float* p, float* f) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p));
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    __device__ static __forceinline__ void store(float* p, const float* f) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    }
};
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}
template <> struct XIo<__nv_bfloat16, 8> {
    __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* f) {
        const uint4 c = __ldg(reinterpret_cast<const uint4*>(p));
        f[0] = bf16_lo(c.x); f[1] = bf16_hi(c.x); f[2] = bf16_lo(c.y); f[3] = bf16_hi(c.y);
        f[4] = bf16_lo(c.z); f[5] = bf16_hi(c.z); f[6] = bf16_lo(c.w); f[7] = bf16_hi(c.w);
    }
    __device__ static __forceinline__ void store(__nv_bfloat16* p, const float* f) {
        *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]),
                                                  pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
    }
};
template <> struct XIo<__nv_bfloat16, 16> {
    __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* f) {
        XIo<__nv_bfloat16, 8>::load(p, f);
        XIo<__nv_bfloat16, 8>::load(p + 8, f + 8);
    }
    __device__ static __forceinline__ void store(__nv_bfloat16* p, const float* f) {
        XIo<__nv_bfloat16, 8>::store(p, f);
        XIo<__nv_bfloat16, 8>::store(p + 8, f + 8);
    }
};

// Dot product of 4 e4m3 values (one 32-bit word) with 4 f16 activations (two f16x2 words), accumulated in
// fp32 by mixed-precision FMAs: every product of two f16 values is exact in fp32, so the result is what the
// fp32 path computes, without widening the table values first.
__device__ __forceinline__ void dot4_e4m3_f16(uint32_t w, uint32_t x01, uint32_t x23, float& d0, float& d1) {
    asm("{\n\t"
        ".reg .b16 lo, hi;\n\t"
        ".reg .b32 h01, h23;\n\t"
        ".reg .f16 a0, a1, a2, a3, b0, b1, b2, b3;\n\t"
        "mov.b32 {lo, hi}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 h01, lo;\n\t"
        "cvt.rn.f16x2.e4m3x2 h23, hi;\n\t"
        "mov.b32 {a0, a1}, h01;\n\t"
        "mov.b32 {a2, a3}, h23;\n\t"
        "mov.b32 {b0, b1}, %3;\n\t"
        "mov.b32 {b2, b3}, %4;\n\t"
        "fma.rn.f32.f16 %0, a0, b0, %0;\n\t"
        "fma.rn.f32.f16 %1, a1, b1, %1;\n\t"
        "fma.rn.f32.f16 %0, a2, b2, %0;\n\t"
        "fma.rn.f32.f16 %1, a3, b3, %1;\n\t"
        "}"
        : "+f"(d0), "+f"(d1)
        : "r"(w), "r"(x01), "r"(x23));
}
// sum of the 8 products of two 16-byte chunks of bf16 values (a bf16 x bf16 product is exact in fp32)
__device__ __forceinline__ void dot8_bf16(const uint4& a, const uint32_t* b, float& d0, float& d1) {
    asm("{\n\t"
        ".reg .b16 a0, a1, b0, b1;\n\t"
        "mov.b32 {a0, a1}, %2;\n\tmov.b32 {b0, b1}, %6;\n\t"
        "fma.rn.f32.bf16 %0, a0, b0, %0;\n\tfma.rn.f32.bf16 %1, a1, b1, %1;\n\t"
        "mov.b32 {a0, a1}, %3;\n\tmov.b32 {b0, b1}, %7;\n\t"
        "fma.rn.f32.bf16 %0, a0, b0, %0;\n\tfma.rn.f32.bf16 %1, a1, b1, %1;\n\t"
        "mov.b32 {a0, a1}, %4;\n\tmov.b32 {b0, b1}, %8;\n\t"
        "fma.rn.f32.bf16 %0, a0, b0, %0;\n\tfma.rn.f32.bf16 %1, a1, b1, %1;\n\t"
        "mov.b32 {a0, a1}, %5;\n\tmov.b32 {b0, b1}, %9;\n\t"
        "fma.rn.f32.bf16 %0, a0, b0, %0;\n\tfma.rn.f32.bf16 %1, a1, b1, %1;\n\t"
        "}"
        : "+f"(d0), "+f"(d1)
        : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]));
}
__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

struct GatherParams {
    const void* x; const int32_t* ids; const float* weights;
    const char* down; const char* up; const float* down_scale; const float* up_scale;
    void* out; int64_t T; int HK; int64_t N; int D, Dout; int activation; int* status;
    int nch_u, nch_v;          // 16-byte chunks per down / up row
    const int32_t* counts;     // optional [T]: entries of token t that are in use (<= HK)
    float* out_f32;            // optional [T, Dout] fp32 output instead of `out`
    const void* residual;      // optional [T, Dout] in the activation dtype, added to the result
    int split;                 // the warps of a CTA share one token (few tokens: decode-shaped batches)
    int64_t block_tokens, block_stride;   // ids / weights / counts laid out in per-rank blocks (see GatherArgs)
    // tiered residency (TIER instances only): row_map[id] >= 0 -> the row is slot row_map[id] of the HBM-resident
    // cache_down / cache_up; < 0 -> it is read from `down` / `up`, which then point at host memory the GPU can address
    const int32_t* row_map; const char* cache_down; const char* cache_up;
};

template <typename XT, typename TT, int CH, bool W10, bool TIER>
__global__ void __launch_bounds__(WarpCfg<TT, CH, W10, TIER>::WARPS * 32, 1) gather_eval_kernel(const GatherParams p) {
    using RC = RingCfg<TT, CH, W10, TIER>;
    constexpr int WARPS = WarpCfg<TT, CH, W10, TIER>::WARPS;
    constexpr int STAGES = RC::STAGES;
    constexpr int SLOT = RC::SLOT;
    constexpr int EPC = Chunk<TT>::N;            // elements per 16-byte chunk
    constexpr bool SCALED = sizeof(TT) == 1;

    extern __shared__ __align__(128) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // layout: [WARPS][STAGES][SLOT] ring | [WARPS][STAGES] mbarriers | per-warp entry lists
    unsigned char* ring = smem + static_cast<size_t>(warp) * STAGES * SLOT;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(WARPS) * STAGES * SLOT) + warp * STAGES;
    unsigned char* lists = smem + static_cast<size_t>(WARPS) * STAGES * SLOT + WARPS * STAGES * 8;
    const int per_warp_list = p.HK * ((SCALED ? 16 : 8) + (TIER ? 4 : 0));
    int32_t* s_id = reinterpret_cast<int32_t*>(lists + static_cast<size_t>(warp) * per_warp_list);
    float* s_w = reinterpret_cast<float*>(s_id + p.HK);
    float* s_us = s_w + p.HK;       // only when SCALED
    float* s_vs = s_us + p.HK;
    int32_t* s_slot = reinterpret_cast<int32_t*>(s_w + (SCALED ? 3 : 1) * p.HK);   // only when TIER: cache slot or -1

    const uint32_t ring_a = smem_u32(ring);
    const uint32_t bars_a = smem_u32(bars);
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(bars_a + 8 * s, 1);
        mbar_fence_init();
    }
    __syncwarp();

    const uint32_t row_u = static_cast<uint32_t>(p.nch_u) * 16u, row_v = static_cast<uint32_t>(p.nch_v) * 16u;
    const XT* __restrict__ xg = static_cast<const XT*>(p.x);
    XT* __restrict__ og = static_cast<XT*>(p.out);

    int slot = 0;            // next ring slot to consume
    uint32_t parity = 0;     // its phase
    bool alive = true;

    // Two ways to spread the work.  Ordinarily every warp owns a token.  With few tokens (split) the WARPS warps
    // of a CTA share one: warp w takes the token's entries w, w + WARPS, ... and the partial sums meet in shared
    // memory at the end, added in warp order, so the result does not depend on timing.
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * WARPS;
    const int64_t t_first = p.split ? static_cast<int64_t>(blockIdx.x) : static_cast<int64_t>(blockIdx.x) * WARPS + warp;
    const int64_t t_step = p.split ? static_cast<int64_t>(gridDim.x) : nwarps;
    for (int64_t t = t_first; t < p.T && (alive || p.split); t += t_step) {
        // ---- token prologue: selections into shared memory, x into registers
        __syncwarp();
        // where this token's entries start: plain [T, HK] arrays, or the blocks an expert-parallel rank received
        const int64_t tb = p.block_tokens ? t / p.block_tokens : 0;
        const int64_t list0 = p.block_tokens ? tb * p.block_stride + (t - tb * p.block_tokens) * p.HK : t * p.HK;
        const int64_t cnt_at = p.block_tokens ? tb * p.block_stride + (t - tb * p.block_tokens) : t;
        const int hk_token = p.counts ? min(max(p.counts[cnt_at], 0), p.HK) : p.HK;
        // entries of this warp: all of the token's, or every WARPS-th one starting at `warp`
        const int e_first = p.split ? warp : 0, e_step = p.split ? WARPS : 1;
        const int hk = p.split ? (hk_token > warp ? (hk_token - warp + WARPS - 1) / WARPS : 0) : hk_token;
        const int total_rows = 2 * hk;
        for (int e = lane; e < hk; e += 32) {
            int32_t id = p.ids[list0 + e_first + e * e_step];
            float w = p.weights[list0 + e_first + e * e_step];
            if (static_cast<uint32_t>(id) >= static_cast<uint64_t>(p.N)) {
                atomicMax(p.status, STATUS_BOUNDS);
                id = 0; w = 0.f;
            }
            s_id[e] = id; s_w[e] = w;
            if (SCALED) { s_us[e] = __ldg(p.down_scale + id); s_vs[e] = __ldg(p.up_scale + id); }
            if constexpr (TIER) s_slot[e] = __ldg(p.row_map + id);
        }
        // The activation row stays in registers for the whole token: fp32, or (rows longer than 64
        // elements per lane, bf16 activations) as packed bf16 pairs widened at each use.
        // bf16 tables with bf16 activations: the activations stay packed and the down-row dot product runs on
        // mixed-precision FMAs (no widening of either operand)
        constexpr bool BFDOT = sizeof(TT) == 2 && sizeof(XT) == 2;
        constexpr bool PACKX = (CH * EPC > 64) || (WarpCfg<TT, CH, W10, TIER>::MANY && sizeof(XT) == 2) || BFDOT;
        // FP8 rows: the activations are kept as f16 pairs, scaled by a power of two so
        // that the row's largest magnitude lies in [1, 2) (a bf16 value then converts exactly unless it is more
        // than 2^14 times smaller than the largest), and the down-row dot product runs on mixed-precision FMAs.
        constexpr bool F16X = sizeof(TT) == 1 && sizeof(XT) == 2;
        static_assert(!PACKX || sizeof(XT) == 2, "long rows need bf16 activations");
        float xr[PACKX ? 1 : CH * EPC];
        uint32_t xp[PACKX ? CH * EPC / 2 : 1];
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int c = lane + 32 * i;
            if constexpr (PACKX) {
#pragma unroll
                for (int e = 0; e < EPC / 2; e += 4) {
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (c < p.nch_u) v = __ldg(reinterpret_cast<const uint4*>(xg + t * p.D + c * EPC + 2 * e));
                    xp[i * EPC / 2 + e] = v.x; xp[i * EPC / 2 + e + 1] = v.y;
                    xp[i * EPC / 2 + e + 2] = v.z; xp[i * EPC / 2 + e + 3] = v.w;
                }
            } else {
                if (c < p.nch_u) XIo<XT, EPC>::load(xg + t * p.D + c * EPC, xr + i * EPC);
                else {
#pragma unroll
                    for (int e = 0; e < EPC; ++e) xr[i * EPC + e] = 0.f;
                }
            }
        }
        float x_unscale = 1.0f;
        if constexpr (F16X) {
            float mx = 0.f;
#pragma unroll
            for (int i = 0; i < CH * EPC / 2; ++i) mx = fmaxf(mx, fmaxf(fabsf(bf16_lo(xp[i])), fabsf(bf16_hi(xp[i]))));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL_MASK, mx, o));
            const int ex = (__float_as_int(mx) >> 23) & 0xff;                 // biased exponent of the largest magnitude
            const bool usable = ex > 0 && ex < 254;                            // zero row, or inf/nan: leave the scale at 1
            const float sc = usable ? __int_as_float((254 - ex) << 23) : 1.0f; // 2^-(ex-127)
            x_unscale = usable ? __int_as_float(ex << 23) : 1.0f;              // 2^(ex-127)
#pragma unroll
            for (int i = 0; i < CH * EPC / 2; ++i) xp[i] = pack_f16(bf16_lo(xp[i]) * sc, bf16_hi(xp[i]) * sc);
        }
        auto xval = [&](int idx) -> float {
            if constexpr (PACKX) return (idx & 1) ? bf16_hi(xp[idx >> 1]) : bf16_lo(xp[idx >> 1]);
            else return xr[idx];
        };
        float acc[CH * EPC];
#pragma unroll
        for (int i = 0; i < CH * EPC; ++i) acc[i] = 0.f;
        __syncwarp();

        auto issue = [&](int r, int s) {      // lane 0 only: row r of this token into slot s
            const int id = s_id[r >> 1];
            const bool is_v = r & 1;
            const char* src = is_v ? p.up + static_cast<int64_t>(id) * row_v
                                   : p.down + static_cast<int64_t>(id) * row_u;
            const uint32_t bytes = is_v ? row_v : row_u;
            if constexpr (TIER) {
                const int cs = s_slot[r >> 1];
                if (cs < 0) {                 // host-resident row: nothing is staged, the consumer reads it in place;
                    mbar_arrive(bars_a + 8 * s);   // the slot's phase completes at once so the ring keeps its order
                    return;
                }
                src = is_v ? p.cache_up + static_cast<int64_t>(cs) * row_v : p.cache_down + static_cast<int64_t>(cs) * row_u;
            }
            fence_proxy_async();
            mbar_expect_tx(bars_a + 8 * s, bytes);
            bulk_g2s(ring_a + s * SLOT, src, bytes, bars_a + 8 * s);
        };
        if (lane == 0 && alive) {
            int s = slot;
            for (int r = 0; r < STAGES && r < total_rows; ++r) {
                issue(r, s);
                if (++s == STAGES) s = 0;
            }
        }

        for (int e = 0; e < hk && alive; ++e) {
            // ---- down row: dot with x
            if (!mbar_wait(bars_a + 8 * slot, parity, p.status)) { alive = false; }
            alive = __all_sync(FULL_MASK, alive);
            if (!alive) break;
            float d0 = 0.f, d1 = 0.f;
            {
                const unsigned char* rb = ring + slot * SLOT;
                if constexpr (TIER) {         // a row that is not cached is read where it lives (host memory the GPU addresses)
                    if (s_slot[e] < 0) rb = reinterpret_cast<const unsigned char*>(p.down) + static_cast<int64_t>(s_id[e]) * row_u;
                }
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const int c = lane + 32 * i;
                    if (c < p.nch_u) {
                        const uint4 raw = *reinterpret_cast<const uint4*>(rb + c * 16);
                        if constexpr (F16X) {
                            const uint32_t* xw = xp + i * EPC / 2;          // 8 f16x2 words for this chunk's 16 elements
                            dot4_e4m3_f16(raw.x, xw[0], xw[1], d0, d1);
                            dot4_e4m3_f16(raw.y, xw[2], xw[3], d0, d1);
                            dot4_e4m3_f16(raw.z, xw[4], xw[5], d0, d1);
                            dot4_e4m3_f16(raw.w, xw[6], xw[7], d0, d1);
                        } else if constexpr (BFDOT) {
                            dot8_bf16(raw, xp + i * EPC / 2, d0, d1);
                        } else {
                            float f[EPC];
                            Chunk<TT>::decode(raw, f);
#pragma unroll
                            for (int q = 0; q < EPC; q += 2) {
                                d0 = fmaf(f[q], xval(i * EPC + q), d0);
                                d1 = fmaf(f[q + 1], xval(i * EPC + q + 1), d1);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && 2 * e + STAGES < total_rows) issue(2 * e + STAGES, slot);
            if (++slot == STAGES) { slot = 0; parity ^= 1; }
            float dot = warp_sum(d0 + d1);
            if constexpr (F16X) dot *= x_unscale;
            if (SCALED) dot *= s_us[e];
            float g = p.activation == PEER_ACT_GELU ? gelu_erf(dot) : fmaxf(dot, 0.f);
            g *= s_w[e];
            if (SCALED) g *= s_vs[e];

            // ---- up row: accumulate
            if (!mbar_wait(bars_a + 8 * slot, parity, p.status)) { alive = false; }
            alive = __all_sync(FULL_MASK, alive);
            if (!alive) break;
            {
                const unsigned char* rb = ring + slot * SLOT;
                if constexpr (TIER) {
                    if (s_slot[e] < 0) rb = reinterpret_cast<const unsigned char*>(p.up) + static_cast<int64_t>(s_id[e]) * row_v;
                }
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const int c = lane + 32 * i;
                    if (c < p.nch_v) {
                        const uint4 raw = *reinterpret_cast<const uint4*>(rb + c * 16);
                        float f[EPC];
                        Chunk<TT>::decode(raw, f);
#pragma unroll
                        for (int q = 0; q < EPC; ++q) acc[i * EPC + q] = fmaf(g, f[q], acc[i * EPC + q]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && 2 * e + 1 + STAGES < total_rows) issue(2 * e + 1 + STAGES, slot);
            if (++slot == STAGES) { slot = 0; parity ^= 1; }
        }
        if (p.split) {
            // every warp of the CTA comes here, also one whose wait ran out (its sums are dropped with the status
            // word set): the partial sums go to shared memory - the rings are idle now - and are added in warp order
            __syncthreads();
            float* part = reinterpret_cast<float*>(smem);                 // [WARPS][Dout]
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const int c = lane + 32 * i;
                if (c < p.nch_v) {
#pragma unroll
                    for (int q = 0; q < EPC; q += 4)
                        *reinterpret_cast<float4*>(part + static_cast<size_t>(warp) * p.Dout + c * EPC + q) =
                            make_float4(acc[i * EPC + q], acc[i * EPC + q + 1], acc[i * EPC + q + 2], acc[i * EPC + q + 3]);
                }
            }
            __syncthreads();
            for (int col = threadIdx.x; col < p.Dout; col += WARPS * 32) {
                float sum = 0.f;
                for (int w = 0; w < WARPS; ++w) sum += part[static_cast<size_t>(w) * p.Dout + col];
                if (p.out_f32) p.out_f32[t * p.Dout + col] = sum;
                else {
                    if (p.residual) sum += to_f32<XT>(static_cast<const XT*>(p.residual)[t * p.Dout + col]);
                    og[t * p.Dout + col] = from_f32<XT>(sum);
                }
            }
            __syncthreads();                                              // before the rings are filled again
            continue;
        }
        if (!alive) break;

#pragma unroll
        for (int i = 0; i < CH; ++i) {
            const int c = lane + 32 * i;
            if (c < p.nch_v) {
                if (p.out_f32) {
#pragma unroll
                    for (int q = 0; q < EPC; q += 4)
                        *reinterpret_cast<float4*>(p.out_f32 + t * p.Dout + c * EPC + q) =
                            make_float4(acc[i * EPC + q], acc[i * EPC + q + 1], acc[i * EPC + q + 2], acc[i * EPC + q + 3]);
                } else {
                    if (p.residual) {
                        if constexpr (EPC * sizeof(XT) >= 16) {     // the table chunk covers whole 16-byte pieces of the row
                            float rsd[EPC];
                            XIo<XT, EPC>::load(static_cast<const XT*>(p.residual) + t * p.Dout + c * EPC, rsd);
#pragma unroll
                            for (int q = 0; q < EPC; ++q) acc[i * EPC + q] += rsd[q];
                        }
                    }
                    XIo<XT, EPC>::store(og + t * p.Dout + c * EPC, acc + i * EPC);
                }
            }
        }
    }
}

template <typename XT, typename TT, int CH, bool W10, bool TIER>
size_t smem_bytes(int HK) {
    using RC = RingCfg<TT, CH, W10, TIER>;
    constexpr int WARPS = WarpCfg<TT, CH, W10, TIER>::WARPS;
    return static_cast<size_t>(WARPS) * RC::STAGES * RC::SLOT + WARPS * RC::STAGES * 8 +
           static_cast<size_t>(WARPS) * HK * ((sizeof(TT) == 1 ? 16 : 8) + (TIER ? 4 : 0));
}

template <typename XT, typename TT, int CH, bool W10, bool TIER = false>
cudaError_t launch_w(const GatherArgs& a, const GatherParams& p, cudaStream_t s) {
    const size_t smem = smem_bytes<XT, TT, CH, W10, TIER>(a.HK);
    if (smem > MAX_SMEM) return cudaErrorInvalidValue;
    // Per instantiation and device; the attribute is sticky per function.  Setting it twice is harmless, so
    // two host threads (two handles) that meet here need only see a consistent flag: an atomic, no lock.
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaError_t de = cudaGetDevice(&dev);
    if (de != cudaSuccess) return de;
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(gather_eval_kernel<XT, TT, CH, W10, TIER>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    constexpr int WARPS = WarpCfg<TT, CH, W10, TIER>::WARPS;
    int64_t ctas = (a.T + WARPS - 1) / WARPS;
    if (ctas > a.sm_count) ctas = a.sm_count;
    GatherParams q = p;
    // few tokens (a decode-shaped batch): one token per CTA, its entries dealt to the warps, so that all SMs
    // stream rows instead of T / WARPS of them; the partial sums need WARPS * Dout floats of the ring space
    // (only for the partial evaluation of a row shard: the ordinary layer keeps one warp per token at every batch
    // size, so that a token's result never depends on how many tokens came with it)
    q.split = a.counts != nullptr && a.T <= a.sm_count &&
              static_cast<size_t>(WARPS) * a.Dout * sizeof(float) <= static_cast<size_t>(WARPS) * RingCfg<TT, CH, W10, TIER>::STAGES * RingCfg<TT, CH, W10, TIER>::SLOT;
    if (q.split) ctas = a.T;
    gather_eval_kernel<XT, TT, CH, W10, TIER><<<static_cast<unsigned>(ctas), WARPS * 32, smem, s>>>(q);
    return cudaGetLastError();
}

template <typename XT, typename TT, int CH>
cudaError_t launch_t(const GatherArgs& a, const GatherParams& p, cudaStream_t s) {
    if constexpr (sizeof(TT) <= 2) {          // tiered residency: 16-bit and FP8 tables
        if (a.row_map) return launch_w<XT, TT, CH, false, true>(a, p, s);
    } else {
        if (a.row_map) return cudaErrorInvalidValue;
    }
    if constexpr (sizeof(TT) == 2 && CH == 8) {
        if (a.rows_l2_resident) return launch_w<XT, TT, CH, true>(a, p, s);
    }
    return launch_w<XT, TT, CH, false>(a, p, s);
}

template <typename XT, typename TT>
cudaError_t launch_ch(const GatherArgs& a, const GatherParams& p, int max_ch, cudaStream_t s) {
    const int need = (max_ch + 31) / 32;     // chunks per lane
    // elements per lane: 64 with fp32 activations in registers, 128 with packed bf16 activations
    constexpr int EPC = Chunk<TT>::N;
    constexpr int EPL_LIMIT = sizeof(XT) == 2 ? 128 : 64;
    if (need * EPC > EPL_LIMIT && need > 1) return cudaErrorInvalidValue;
    if (need <= 1) return launch_t<XT, TT, 1>(a, p, s);
    if (need <= 2) return launch_t<XT, TT, 2>(a, p, s);
    if (need <= 4) return launch_t<XT, TT, 4>(a, p, s);
    if constexpr (8 * EPC <= EPL_LIMIT) { if (need <= 8) return launch_t<XT, TT, 8>(a, p, s); }
    if constexpr (16 * EPC <= EPL_LIMIT) { if (need <= 16) return launch_t<XT, TT, 16>(a, p, s); }
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_gather_eval(const GatherArgs& a, cudaStream_t s) {
    if (a.T == 0) return cudaSuccess;
    const int tb = a.table_dtype == PEER_DTYPE_F32 ? 4 : (a.table_dtype == PEER_DTYPE_BF16 ? 2 : 1);
    GatherParams p;
    p.x = a.x; p.ids = a.ids; p.weights = a.weights;
    p.down = static_cast<const char*>(a.down); p.up = static_cast<const char*>(a.up);
    p.down_scale = a.down_scale; p.up_scale = a.up_scale; p.out = a.out; p.T = a.T; p.HK = a.HK;
    p.N = a.N; p.D = a.D; p.Dout = a.Dout; p.activation = a.activation; p.status = a.status;
    p.nch_u = a.D * tb / 16; p.nch_v = a.Dout * tb / 16;
    p.counts = a.counts; p.out_f32 = a.out_f32; p.residual = a.residual; p.split = 0;
    p.block_tokens = a.block_tokens; p.block_stride = a.block_stride;
    p.row_map = a.row_map; p.cache_down = static_cast<const char*>(a.cache_down); p.cache_up = static_cast<const char*>(a.cache_up);
    const int max_ch = p.nch_u > p.nch_v ? p.nch_u : p.nch_v;
    if (a.act_dtype == PEER_DTYPE_F32 && a.table_dtype == PEER_DTYPE_F32)
        return launch_ch<float, float>(a, p, max_ch, s);
    if (a.act_dtype == PEER_DTYPE_BF16 && a.table_dtype == PEER_DTYPE_BF16)
        return launch_ch<__nv_bfloat16, __nv_bfloat16>(a, p, max_ch, s);
    if (a.act_dtype == PEER_DTYPE_BF16 && a.table_dtype == PEER_DTYPE_E4M3)
        return launch_ch<__nv_bfloat16, __nv_fp8_e4m3>(a, p, max_ch, s);
    return cudaErrorInvalidValue;
}

}  // namespace peer
