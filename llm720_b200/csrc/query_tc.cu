// Query stage on the tensor cores (bf16 layers): q = x W^T + b on tcgen05 with
// the accumulator in TMEM, then, straight out of TMEM, the LayerNorm over the
// head's query dimension and the per-half L2 normalisation.
//
// Follows llm/models/experts.py:302-308 (projection, LayerNorm shared by all
// heads) and :156-159 (F.normalize of each query half).
//
// One CTA tile = 128 tokens x one head (N = query_dim <= 256), K walked in
// 64-column TMA boxes through a 4-stage mbarrier ring.  Warp 0 issues the TMA
// loads, warp 1 the MMAs, warps 2-9 run the epilogue: a thread owns one TMEM
// lane (= one token row) and one half of the head's columns (= one query
// half), the two threads of a row exchange their LayerNorm partial sums through
// shared memory; two accumulators alternate so the epilogue of a tile overlaps
// the MMAs of the next.  The grid is persistent.
//
// Output: the normalised query halves split into three bf16 terms
// (hi + mid + lo = the fp32 value to 2^-27), the form the select kernel feeds
// to the tensor cores, and optionally the fp32 values.
#include "kernels.h"
#include "tc_common.cuh"

namespace peer {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int MAXQ = 256;
constexpr int A_BYTES = BM * BK * 2;        // 16 KB
constexpr int B_BYTES = MAXQ * BK * 2;      // 32 KB
constexpr int THREADS = 320;
constexpr int EPI_THREADS = 256;
constexpr float LN_EPS = 1e-5f;
constexpr float NORM_EPS = 1e-12f;
constexpr uint32_t TMEM_COLS = 512;

struct SmemLayout {
    static constexpr size_t a_off = 0;
    static constexpr size_t b_off = a_off + static_cast<size_t>(STAGES) * A_BYTES;
    static constexpr size_t par_off = b_off + static_cast<size_t>(STAGES) * B_BYTES;   // bias[2][256], gamma[256], beta[256]
    static constexpr size_t red_off = par_off + 4 * MAXQ * sizeof(float);             // LayerNorm partial sums [2][2][128]
    static constexpr size_t bar_off = red_off + 4 * BM * sizeof(float);
    static constexpr size_t total = bar_off + 16 * sizeof(uint64_t) + 16 + 1024;   // + slack to align the base to 1024
};

__device__ __forceinline__ uint32_t pack2_bf16(__nv_bfloat16 a, __nv_bfloat16 b) {
    return static_cast<uint32_t>(__bfloat16_as_ushort(a)) | (static_cast<uint32_t>(__bfloat16_as_ushort(b)) << 16);
}

__global__ void __launch_bounds__(THREADS, 1)
query_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ ln_w,
                const __nv_bfloat16* __restrict__ ln_b, float* __restrict__ q_ln_out,
                float* __restrict__ q_hat_out, __nv_bfloat16* __restrict__ split_out, int64_t split_stride,
                int64_t Ttok, int D, int H, int Q, int layer_norm, int norm_query, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzled tiles need 1024-byte alignment
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* s_bias = reinterpret_cast<float*>(smem + SmemLayout::par_off);       // [2][MAXQ]
    float* s_gamma = s_bias + 2 * MAXQ;
    float* s_beta = s_gamma + MAXQ;
    float* s_red = reinterpret_cast<float*>(smem + SmemLayout::red_off);        // [sum | centred squares][column half][row]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SmemLayout::bar_off);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    const uint32_t sA = smem_u32(smem + SmemLayout::a_off), sB = smem_u32(smem + SmemLayout::b_off);
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto accf_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
    auto acce_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accf_bar(a), 1); mbar_init(acce_bar(a), EPI_THREADS); }
        mbar_fence_init();
        tc::tma_prefetch_desc(&map_x);
        tc::tma_prefetch_desc(&map_w);
    }
    for (int c = tid; c < MAXQ; c += THREADS) {
        s_gamma[c] = (c < Q && ln_w) ? __bfloat162float(ln_w[c]) : 1.f;
        s_beta[c] = (c < Q && ln_b) ? __bfloat162float(ln_b[c]) : 0.f;
    }
    if (warp == 0) {
        __syncwarp();
        tc::tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t m_tiles = (Ttok + BM - 1) / BM;
    const int64_t n_tiles = m_tiles * H;
    const int num_kb = (D + BK - 1) / BK;
    const uint32_t idesc = tc::idesc_bf16_f32(BM, Q);
    const uint32_t stage_bytes = A_BYTES + static_cast<uint32_t>(Q) * BK * 2;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int m_blk = static_cast<int>(tile / H), h = static_cast<int>(tile % H);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_hint(empty_bar(stage), phase ^ 1, status)) { ok = false; break; }
                    mbar_expect_tx(full_bar(stage), stage_bytes);
                    tc::tma_load_2d(sA + stage * A_BYTES, &map_x, kb * BK, m_blk * BM, full_bar(stage));
                    tc::tma_load_2d(sB + stage * B_BYTES, &map_w, kb * BK, h * Q, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
            for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait_hint(acce_bar(acc), acc_phase ^ 1, status)) { ok = false; break; }
                tc::fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * MAXQ;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_hint(full_bar(stage), phase, status)) { ok = false; break; }
                    tc::fence_after_sync();
                    const uint64_t ad = tc::smem_desc_sw128(sA + stage * A_BYTES);
                    const uint64_t bd = tc::smem_desc_sw128(sB + stage * B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        tc::umma_bf16(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0);
                    tc::umma_commit(empty_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc::umma_commit(accf_bar(acc));
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else {
        // ---------------- epilogue: one thread per (token row, query half) ----------------
        const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
        const int colhalf = (warp - 2) >> 2;          // which half of the head's columns
        const int row = quarter * 32 + lane;
        const int et = tid - 64;                      // 0..255
        const int nb = Q / 32;
        const int b_lo = colhalf * (nb / 2), b_hi = b_lo + nb / 2;
        const int half = Q / 2;
        const float invQ = 1.0f / static_cast<float>(Q);
        int acc = 0; uint32_t acc_phase = 0; bool ok = true;
        for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            const int m_blk = static_cast<int>(tile / H), h = static_cast<int>(tile % H);
            float* sb = s_bias + acc * MAXQ;
            for (int c = et; c < Q; c += EPI_THREADS) sb[c] = bias ? __bfloat162float(bias[h * Q + c]) : 0.f;
            if (ok && !mbar_wait_hint(accf_bar(acc), acc_phase, status)) ok = false;
            {   // one barrier publishes the bias and makes the decision the same in every epilogue thread
                int all_ok;
                asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.s32 q, %1, 0;\n\tbar.red.and.pred p, 1, 256, q;\n\t"
                             "selp.s32 %0, 1, 0, p;\n\t}" : "=r"(all_ok) : "r"(static_cast<int>(ok)) : "memory");
                ok = all_ok != 0;
            }
            if (!ok) continue;
            tc::fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc) * MAXQ;
            uint32_t r[32];
            float mean = 0.f, rstd = 1.f;
            if (layer_norm) {
                float s = 0.f;
                for (int b = b_lo; b < b_hi; ++b) {
                    tc::tmem_ld32(taddr + b * 32, r);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) s += __uint_as_float(r[j]) + sb[b * 32 + j];
                }
                s_red[colhalf * BM + row] = s;
                asm volatile("bar.sync 1, 256;" ::: "memory");
                mean = (s_red[row] + s_red[BM + row]) * invQ;
                float ss = 0.f;
                for (int b = b_lo; b < b_hi; ++b) {
                    tc::tmem_ld32(taddr + b * 32, r);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float d = __uint_as_float(r[j]) + sb[b * 32 + j] - mean;
                        ss = fmaf(d, d, ss);
                    }
                }
                s_red[2 * BM + colhalf * BM + row] = ss;
                asm volatile("bar.sync 1, 256;" ::: "memory");
                rstd = 1.0f / sqrtf((s_red[2 * BM + row] + s_red[3 * BM + row]) * invQ + LN_EPS);
            }
            float n0 = 1.f, n1 = 1.f;
            const int64_t grow = static_cast<int64_t>(m_blk) * BM + row;
            const int64_t obase = (grow * H + h) * Q;
            {
                float s0 = 0.f, s1 = 0.f;
                for (int b = b_lo; b < b_hi; ++b) {
                    tc::tmem_ld32(taddr + b * 32, r);
                    tc::tmem_ld_wait();
                    float y[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int c = b * 32 + j;
                        float v = __uint_as_float(r[j]) + sb[c];
                        if (layer_norm) v = (v - mean) * rstd * s_gamma[c] + s_beta[c];
                        y[j] = v;
                    }
                    float p = 0.f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) p = fmaf(y[j], y[j], p);
                    if (b * 32 < half) s0 += p; else s1 += p;
                    if (q_ln_out && grow < Ttok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4*>(q_ln_out + obase + b * 32 + j) = make_float4(y[j], y[j + 1], y[j + 2], y[j + 3]);
                    }
                }
                if (norm_query) { n0 = fmaxf(sqrtf(s0), NORM_EPS); n1 = fmaxf(sqrtf(s1), NORM_EPS); }
            }
            if (q_hat_out || split_out) {
                // one reciprocal per query half instead of a division per element (the quotient may differ from
                // v / n in the last bit; scores move by about 1e-7, far inside the 1e-6 near-tie rule)
                const float inv0 = 1.0f / n0, inv1 = 1.0f / n1;
                for (int b = b_lo; b < b_hi; ++b) {
                    tc::tmem_ld32(taddr + b * 32, r);
                    tc::tmem_ld_wait();
                    const float inv_nn = (b * 32 < half) ? inv0 : inv1;
                    float y[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int c = b * 32 + j;
                        float v = __uint_as_float(r[j]) + sb[c];
                        if (layer_norm) v = (v - mean) * rstd * s_gamma[c] + s_beta[c];
                        y[j] = norm_query ? v * inv_nn : v;
                    }
                    if (grow < Ttok) {
                        if (q_hat_out) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(q_hat_out + obase + b * 32 + j) = make_float4(y[j], y[j + 1], y[j + 2], y[j + 3]);
                        }
                        if (split_out) {
                            // hi + mid + lo: three bf16 terms carrying 24 bits of the fp32 value
                            uint32_t w[3][16];
#pragma unroll
                            for (int j = 0; j < 32; j += 2) {
                                __nv_bfloat16 t[3][2];
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    float rem = y[j + e];
                                    t[0][e] = __float2bfloat16_rn(rem); rem -= __bfloat162float(t[0][e]);
                                    t[1][e] = __float2bfloat16_rn(rem); rem -= __bfloat162float(t[1][e]);
                                    t[2][e] = __float2bfloat16_rn(rem);
                                }
#pragma unroll
                                for (int q = 0; q < 3; ++q) w[q][j / 2] = pack2_bf16(t[q][0], t[q][1]);
                            }
#pragma unroll
                            for (int q = 0; q < 3; ++q) {
                                uint4* dst = reinterpret_cast<uint4*>(split_out + q * split_stride + obase + b * 32);
#pragma unroll
                                for (int v4 = 0; v4 < 4; ++v4)
                                    dst[v4] = make_uint4(w[q][4 * v4], w[q][4 * v4 + 1], w[q][4 * v4 + 2], w[q][4 * v4 + 3]);
                            }
                        }
                    }
                }
            }
            tc::fence_before_sync();
            mbar_arrive(acce_bar(acc));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace

bool query_tc_supported(const QueryArgs& a) {
    return a.act_dtype == PEER_DTYPE_BF16 && a.Q % 64 == 0 && a.Q >= 64 && a.Q <= MAXQ && a.D % 8 == 0;
}

cudaError_t query_tc_setup() {
    return cudaFuncSetAttribute(query_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(SmemLayout::total));
}

cudaError_t launch_query_tc(const QueryArgs& a, __nv_bfloat16* split_out, int64_t split_stride, int* status,
                            int sm_count, cudaStream_t s) {
    if (a.T == 0) return cudaSuccess;
    CUtensorMap mx, mw;
    if (!make_tensor_map_bf16(&mx, a.x, static_cast<uint64_t>(a.T), static_cast<uint64_t>(a.D),
                              static_cast<uint64_t>(a.D), BM) ||
        !make_tensor_map_bf16(&mw, a.w, static_cast<uint64_t>(a.H) * a.Q, static_cast<uint64_t>(a.D),
                              static_cast<uint64_t>(a.D), static_cast<uint32_t>(a.Q)))
        return cudaErrorInvalidValue;
    const int64_t n_tiles = ((a.T + BM - 1) / BM) * a.H;
    const unsigned grid = static_cast<unsigned>(n_tiles < sm_count ? n_tiles : sm_count);
    query_tc_kernel<<<grid, THREADS, SmemLayout::total, s>>>(
        mx, mw, static_cast<const __nv_bfloat16*>(a.b), static_cast<const __nv_bfloat16*>(a.ln_w),
        static_cast<const __nv_bfloat16*>(a.ln_b), a.q_ln_out, a.q_hat_out, split_out, split_stride, a.T, a.D,
        a.H, a.Q, a.layer_norm, a.norm_query, status);
    return cudaGetLastError();
}

}  // namespace peer
