// Product-key selection on the tensor cores (bf16 layers): the two sub-key
// score contractions run as tcgen05 MMAs with fp32 accumulators in TMEM, and
// the per-half top-k, the candidate sums, the final top-k, the softmax and
// the flat expert ids are computed straight out of TMEM.  No score reaches HBM.
//
// Follows llm/models/experts.py:153-163 (scores), :168-192 (per-half top-k'),
// :203-259 (candidate sums, flat ids, final top-k) and :327 (softmax).
//
// Exactness.  The reference's fp32 scores are reproduced to fp32 rounding
// level, not approximated: the normalised query half is fed as three bf16
// terms (hi + mid + lo carry 24 bits of the fp32 value), the sub-keys of a
// bf16 layer are exactly representable, every bf16 x bf16 product is exact in
// fp32, and the three partial contractions accumulate in the same fp32 TMEM
// accumulator.  The key's 1/||k|| is applied per column afterwards.
//
// Work split in one CTA (128 (token, head) rows per tile, persistent grid):
//   warp 0      TMA producer: the query tile of a half (3 terms), then the
//               key chunks (128 keys) through a ring;
//   warp 1      MMA issuer: 128x128 accumulators, four in flight in TMEM;
//   warps 4-7   scan group 0, warps 8-11 scan group 1 (warps 2-3 idle): thread = TMEM lane =
//               one row; the groups take alternate chunks.  A thread filters
//               its row's scores against its current 16th-best value, queues
//               the survivors in shared memory and, when a queue runs full,
//               the warp inserts the queued (score, key) pairs into
//               register-resident sorted lists; this keeps the expensive
//               insertion off the per-element path.
// Ordering among exactly equal scores: smaller sub-key index first (per
// half), smaller candidate position first (final), as in select_simt.cu.
#include <float.h>

#include "kernels.h"
#include "tc_common.cuh"

namespace peer {

namespace {

constexpr int BM = 128;            // rows per tile
constexpr int NC = 128;            // keys per chunk (UMMA N)
constexpr int BOX_BYTES = 128 * 64 * 2;   // one TMA box: 128 rows x 64 bf16
constexpr int MAX_KA = 2;          // 64-column boxes per half (half width 64 or 128)
constexpr int A_BYTES = 3 * MAX_KA * BOX_BYTES;     // 96 KB
constexpr int B_STAGE_BYTES = MAX_KA * BOX_BYTES;   // 32 KB
constexpr int B_STAGES = 2;
constexpr int N_ACC = 4;
constexpr int QC = 32;             // queue entries per row and scan group
constexpr int LK = 16;             // list length kept per half
constexpr int THREADS = 384;       // warps 0-3: TMA, MMA, two idle; warps 4-7 and 8-11: the scan groups
constexpr int CTRL_REGS = 40, SCAN_REGS = 232;   // 128*40 + 256*232 = 384*168 registers
constexpr uint32_t TMEM_COLS = 512;

struct Smem {
    static constexpr size_t a_off = 0;
    static constexpr size_t b_off = a_off + A_BYTES;
    static constexpr size_t q_off = b_off + static_cast<size_t>(B_STAGES) * B_STAGE_BYTES;   // [2][QC][128] x 8 B
    static constexpr size_t tau_off = q_off + 2 * QC * BM * 8;                                 // [2][128] floats
    static constexpr size_t bar_off = tau_off + 2 * BM * sizeof(float);
    static constexpr size_t total = bar_off + 16 * sizeof(uint64_t) + 16 + 1008;
};

struct SelTcParams {
    const float* invn0; const float* invn1;   // 1/||key|| per sub-key (or 1)
    int64_t rows;                             // T * H
    int64_t term_rows;                        // row distance between the hi/mid/lo query arrays
    int Q, n0, n1, kp0, kp1, k, mult0, mult1;
    int32_t* ids32; float* weights; int64_t* ids64; float* raw_scores;
    int* status;
};

// Sorted-list insertion, written as a pure function of the OLD list (new arrays, then copy):
// an in-place form of the same logic with a precomputed bool array was observed to be
// miscompiled by nvcc 12.9 for sm_100a (the first inserted element appeared twice).
// Values move through min/max; the indices follow the same predicates.
// strict: an equal score stays behind the entries already present.
__device__ __forceinline__ void insert_pair(float (&v)[LK], int (&c)[LK], float x, int col) {
    int nc[LK];
#pragma unroll
    for (int i = 0; i < LK; ++i) {
        const bool pi = x > v[i];
        const bool pm = (i == 0) ? false : (x > v[i == 0 ? 0 : i - 1]);
        nc[i] = pi ? (pm ? c[i == 0 ? 0 : i - 1] : col) : c[i];
    }
#pragma unroll
    for (int i = LK - 1; i >= 1; --i) v[i] = fmaxf(v[i], fminf(v[i - 1], x));
    v[0] = fmaxf(v[0], x);
#pragma unroll
    for (int i = 0; i < LK; ++i) c[i] = nc[i];
}
// full order: score descending, then index ascending
__device__ __forceinline__ void insert_pair_ordered(float (&v)[LK], int (&c)[LK], float x, int col) {
    int nc[LK];
#pragma unroll
    for (int i = 0; i < LK; ++i) {
        const int j = i == 0 ? 0 : i - 1;
        const bool pi = (x > v[i]) || (x == v[i] && col < c[i]);
        const bool pm = (i == 0) ? false : ((x > v[j]) || (x == v[j] && col < c[j]));
        nc[i] = pi ? (pm ? c[j] : col) : c[i];
    }
#pragma unroll
    for (int i = LK - 1; i >= 1; --i) v[i] = fmaxf(v[i], fminf(v[i - 1], x));
    v[0] = fmaxf(v[0], x);
#pragma unroll
    for (int i = 0; i < LK; ++i) c[i] = nc[i];
}

__global__ void __launch_bounds__(THREADS, 1)
select_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k0,
                 const __grid_constant__ CUtensorMap map_k1, const SelTcParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::bar_off);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    const uint32_t sA = smem_u32(smem + Smem::a_off), sB = smem_u32(smem + Smem::b_off);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t a_full = bar0, a_empty = bar0 + 8;
    auto b_full = [&](int s) { return bar0 + 8u * (2 + s); };
    auto b_empty = [&](int s) { return bar0 + 8u * (2 + B_STAGES + s); };
    auto acc_full = [&](int a) { return bar0 + 8u * (2 + 2 * B_STAGES + a); };
    auto acc_empty = [&](int a) { return bar0 + 8u * (2 + 2 * B_STAGES + N_ACC + a); };

    if (tid == 0) {
        mbar_init(a_full, 1); mbar_init(a_empty, 1);
        for (int s = 0; s < B_STAGES; ++s) { mbar_init(b_full(s), 1); mbar_init(b_empty(s), 1); }
        for (int a = 0; a < N_ACC; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), 128); }
        mbar_fence_init();
        tc::tma_prefetch_desc(&map_q); tc::tma_prefetch_desc(&map_k0); tc::tma_prefetch_desc(&map_k1);
    }
    float* tau_sh = reinterpret_cast<float*>(smem + Smem::tau_off);   // each group's current 16th-best score per row
    if (tid < 2 * BM) tau_sh[tid] = -INFINITY;
    if (warp == 0) {
        __syncwarp();
        tc::tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int hw = p.Q / 2;
    const int KA = hw / 64;                                   // 64-column boxes per half
    const int nch0 = (p.n0 + NC - 1) / NC, nch1 = (p.n1 + NC - 1) / NC;
    const int64_t n_tiles = (p.rows + BM - 1) / BM;
    const uint32_t a_bytes = 3u * KA * BOX_BYTES, b_bytes = static_cast<uint32_t>(KA) * BOX_BYTES;

    // The control warps need few registers; the rest of the launch allocation goes to the scan groups.
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(CTRL_REGS));
      if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t a_phase = 0; int stage = 0; uint32_t b_phase = 0; bool ok = true;
            for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                for (int hf = 0; hf < 2 && ok; ++hf) {
                    if (!mbar_wait(a_empty, a_phase ^ 1, p.status)) { ok = false; break; }
                    a_phase ^= 1;
                    mbar_expect_tx(a_full, a_bytes);
                    for (int t = 0; t < 3; ++t)
                        for (int ka = 0; ka < KA; ++ka)
                            tc::tma_load_2d(sA + (t * KA + ka) * BOX_BYTES, &map_q, hf * hw + ka * 64,
                                            static_cast<int>(t * p.term_rows + tile * BM), a_full);
                    const int nch = hf ? nch1 : nch0;
                    const CUtensorMap* mk = hf ? &map_k1 : &map_k0;
                    for (int c = 0; c < nch; ++c) {
                        if (!mbar_wait(b_empty(stage), b_phase ^ 1, p.status)) { ok = false; break; }
                        mbar_expect_tx(b_full(stage), b_bytes);
                        for (int ka = 0; ka < KA; ++ka)
                            tc::tma_load_2d(sB + stage * B_STAGE_BYTES + ka * BOX_BYTES, mk, ka * 64, c * NC, b_full(stage));
                        if (++stage == B_STAGES) { stage = 0; b_phase ^= 1; }
                    }
                }
            }
        }
      } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = tc::idesc_bf16_f32(BM, NC);
            uint32_t a_phase = 0; int stage = 0; uint32_t b_phase = 0; uint32_t g = 0; bool ok = true;
            for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                for (int hf = 0; hf < 2 && ok; ++hf) {
                    if (!mbar_wait(a_full, a_phase, p.status)) { ok = false; break; }
                    a_phase ^= 1;
                    const int nch = hf ? nch1 : nch0;
                    for (int c = 0; c < nch; ++c, ++g) {
                        const int acc = g & (N_ACC - 1);
                        if (!mbar_wait(acc_empty(acc), ((g / N_ACC) & 1) ^ 1, p.status)) { ok = false; break; }
                        if (!mbar_wait(b_full(stage), b_phase, p.status)) { ok = false; break; }
                        tc::fence_after_sync();
                        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * NC;
                        uint32_t first = 0;
                        for (int t = 0; t < 3; ++t)
                            for (int ka = 0; ka < KA; ++ka) {
                                const uint64_t ad = tc::smem_desc_sw128(sA + (t * KA + ka) * BOX_BYTES);
                                const uint64_t bd = tc::smem_desc_sw128(sB + stage * B_STAGE_BYTES + ka * BOX_BYTES);
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    tc::umma_bf16(d_tmem, ad + 2 * k, bd + 2 * k, idesc, first);
                                    first = 1;
                                }
                            }
                        tc::umma_commit(b_empty(stage));
                        tc::umma_commit(acc_full(acc));
                        if (++stage == B_STAGES) { stage = 0; b_phase ^= 1; }
                    }
                    if (ok) tc::umma_commit(a_empty);     // the query tile of this half is no longer read
                }
            }
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SCAN_REGS));
        // ---------------- scan groups ----------------
        const int wg = (warp - 4) >> 2;               // 0 or 1
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        uint2* queue = reinterpret_cast<uint2*>(smem + Smem::q_off) + static_cast<size_t>(wg) * QC * BM;   // [QC][128]
        uint2* other_queue = reinterpret_cast<uint2*>(smem + Smem::q_off) + static_cast<size_t>(wg ^ 1) * QC * BM;
        uint32_t g = 0;                                // global chunk counter (all chunks, both groups)
        bool ok = true;
        int64_t tile_iter = 0;
        for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tile_iter) {
            const bool merger = (tile_iter & 1) == wg;
            float hv[2][LK]; int hc[2][LK];           // merged per-half lists (merger group only)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int n = hf ? p.n1 : p.n0;
                const int nch = hf ? nch1 : nch0;
                const float* __restrict__ invn = hf ? p.invn1 : p.invn0;
                float v[LK]; int c[LK];
#pragma unroll
                for (int i = 0; i < LK; ++i) { v[i] = -INFINITY; c[i] = 0x7fffffff; }
                int cnt = 0;
                float tau = -INFINITY;
                // A score below the OTHER group's 16th-best cannot be among the row's 16 best either,
                // so the two groups share their thresholds through shared memory.
                volatile float* tau_mine = tau_sh + wg * BM + row;
                volatile float* tau_other = tau_sh + (wg ^ 1) * BM + row;
                auto drain = [&]() {
                    const int maxc = __reduce_max_sync(FULL_MASK, cnt);
                    for (int i = 0; i < maxc; ++i) {
                        float x = -INFINITY; int col = 0;
                        if (i < cnt) { const uint2 e = queue[i * BM + row]; x = __uint_as_float(e.x); col = static_cast<int>(e.y); }
                        if (!__any_sync(FULL_MASK, x > v[LK - 1])) continue;
                        insert_pair(v, c, x, col);
                    }
                    cnt = 0;
                    *tau_mine = v[LK - 1];
                    tau = fmaxf(v[LK - 1], *tau_other);
                };
                for (int ch = 0; ch < nch; ++ch, ++g) {
                    if ((g & 1u) != static_cast<uint32_t>(wg)) continue;
                    const int acc = g & (N_ACC - 1);
                    if (ok && !mbar_wait(acc_full(acc), (g / N_ACC) & 1, p.status)) ok = false;
                    if (!ok) continue;
                    tc::fence_after_sync();
                    tau = fmaxf(tau, *tau_other);
                    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc) * NC;
                    const int col0 = ch * NC;
#pragma unroll 1
                    for (int b = 0; b < NC / 32; ++b) {
                        uint32_t r[32];
                        tc::tmem_ld32(taddr + b * 32, r);
                        tc::tmem_ld_wait();
                        if (b == NC / 32 - 1) {        // accumulator fully read: hand it back to the MMA warp
                            tc::fence_before_sync();
                            mbar_arrive(acc_empty(acc));
                        }
                        const int cb = col0 + b * 32;
                        if (cb >= n) continue;
                        if (cb + 32 <= n) {
#pragma unroll
                            for (int j8 = 0; j8 < 32; j8 += 8) {
                                const float4 s0 = __ldg(reinterpret_cast<const float4*>(invn + cb + j8));
                                const float4 s1 = __ldg(reinterpret_cast<const float4*>(invn + cb + j8 + 4));
                                const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    // branch-free push: always store into the next free slot, keep it only if it passes
                                    const float x = __uint_as_float(r[j8 + e]) * sc[e];
                                    queue[cnt * BM + row] = make_uint2(__float_as_uint(x), static_cast<uint32_t>(cb + j8 + e));
                                    cnt += (x > tau) ? 1 : 0;
                                }
                                if (__any_sync(FULL_MASK, cnt > QC - 8)) drain();
                            }
                        } else {                       // ragged last batch of the table
#pragma unroll
                            for (int j8 = 0; j8 < 32; j8 += 8) {
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    const int col = cb + j8 + e;
                                    const float x = (col < n) ? __uint_as_float(r[j8 + e]) * __ldg(invn + col) : -INFINITY;
                                    queue[cnt * BM + row] = make_uint2(__float_as_uint(x), static_cast<uint32_t>(col));
                                    cnt += (x > tau) ? 1 : 0;
                                }
                                if (__any_sync(FULL_MASK, cnt > QC - 8)) drain();
                            }
                        }
                    }
                }
                drain();
                // ---- merge the two groups' lists of this half (both groups take part in both barriers)
                if (!merger) {
#pragma unroll
                    for (int i = 0; i < LK; ++i)
                        queue[i * BM + row] = make_uint2(__float_as_uint(v[i]), static_cast<uint32_t>(c[i]));
                }
                asm volatile("bar.sync 2, 256;" ::: "memory");
                *tau_mine = -INFINITY;                 // both groups are done scanning this half
                uint2 oth[LK];
                if (merger) {
#pragma unroll
                    for (int i = 0; i < LK; ++i) oth[i] = other_queue[i * BM + row];
                }
                asm volatile("bar.sync 3, 256;" ::: "memory");
                if (merger) {
#pragma unroll
                    for (int i = 0; i < LK; ++i)
                        insert_pair_ordered(v, c, __uint_as_float(oth[i].x), static_cast<int>(oth[i].y));
#pragma unroll
                    for (int i = 0; i < LK; ++i) { hv[hf][i] = v[i]; hc[hf][i] = c[i]; }
                }
            }
            if (!merger || !ok) continue;
            // ---- candidate sums, final top-k, softmax, ids (thread = row)
            const int64_t grow = tile * BM + row;
            float fv[LK]; int fid[LK];
#pragma unroll
            for (int i = 0; i < LK; ++i) { fv[i] = -INFINITY; fid[i] = 0; }
#pragma unroll
            for (int a = 0; a < LK; ++a) {
#pragma unroll
                for (int b = 0; b < LK / (a + 1); ++b) {
                    // only pairs with (a+1)(b+1) <= k can reach the top k: both lists are sorted
                    if ((a + 1) * (b + 1) <= p.k && a < p.kp0 && b < p.kp1)
                        insert_pair(fv, fid, hv[0][a] + hv[1][b], hc[0][a] * p.mult0 + hc[1][b] * p.mult1);
                }
            }
            if (grow < p.rows) {
                float e[LK], sum = 0.f;
#pragma unroll
                for (int i = 0; i < LK; ++i) { e[i] = (i < p.k) ? expf(fv[i] - fv[0]) : 0.f; sum += e[i]; }
                const float inv = 1.0f / sum;
                const int64_t o = grow * p.k;
#pragma unroll
                for (int i = 0; i < LK; ++i) {
                    if (i < p.k) {
                        if (p.ids32) p.ids32[o + i] = fid[i];
                        if (p.weights) p.weights[o + i] = e[i] * inv;
                        if (p.ids64) p.ids64[o + i] = fid[i];
                        if (p.raw_scores) p.raw_scores[o + i] = fv[i];
                    }
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

__global__ void key_inv_norm_kernel(const __nv_bfloat16* __restrict__ keys, int n, int width, int do_norm,
                                    float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (r >= n) return;
    float ss = 0.f;
    for (int c = lane; c < width; c += 32) {
        const float v = __bfloat162float(keys[static_cast<int64_t>(r) * width + c]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) out[r] = do_norm ? 1.0f / fmaxf(sqrtf(ss), 1e-12f) : 1.0f;
}

}  // namespace

bool select_tc_supported(int act_dtype, int Q, int n0, int n1, int k, int kp0, int kp1) {
    return act_dtype == PEER_DTYPE_BF16 && (Q == 128 || Q == 256) && k <= LK && kp0 <= LK && kp1 <= LK &&
           n0 % 4 == 0 && n1 % 4 == 0;
}

cudaError_t select_tc_setup() {
    return cudaFuncSetAttribute(select_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(Smem::total));
}

cudaError_t launch_key_inv_norms(const void* keys, int n, int width, int do_norm, float* out, cudaStream_t s) {
    const unsigned blocks = static_cast<unsigned>((static_cast<int64_t>(n) * 32 + 255) / 256);
    key_inv_norm_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(keys), n, width, do_norm, out);
    return cudaGetLastError();
}

cudaError_t launch_select_tc(const SelectTcArgs& a, cudaStream_t s) {
    if (a.rows == 0) return cudaSuccess;
    const int hw = a.Q / 2;
    CUtensorMap mq, mk0, mk1;
    if (!make_tensor_map_bf16(&mq, a.q_split, static_cast<uint64_t>(3 * a.term_rows), static_cast<uint64_t>(a.Q),
                              static_cast<uint64_t>(a.Q), BM) ||
        !make_tensor_map_bf16(&mk0, a.keys0, static_cast<uint64_t>(a.n0), static_cast<uint64_t>(hw),
                              static_cast<uint64_t>(hw), NC) ||
        !make_tensor_map_bf16(&mk1, a.keys1, static_cast<uint64_t>(a.n1), static_cast<uint64_t>(hw),
                              static_cast<uint64_t>(hw), NC))
        return cudaErrorInvalidValue;
    SelTcParams p;
    p.invn0 = a.invn0; p.invn1 = a.invn1; p.rows = a.rows; p.term_rows = a.term_rows; p.Q = a.Q;
    p.n0 = a.n0; p.n1 = a.n1; p.kp0 = a.kp0; p.kp1 = a.kp1; p.k = a.k; p.mult0 = a.mult0; p.mult1 = a.mult1;
    p.ids32 = a.ids32; p.weights = a.weights; p.ids64 = a.ids64; p.raw_scores = a.raw_scores; p.status = a.status;
    const int64_t n_tiles = (a.rows + BM - 1) / BM;
    const unsigned grid = static_cast<unsigned>(n_tiles < a.sm_count ? n_tiles : a.sm_count);
    select_tc_kernel<<<grid, THREADS, Smem::total, s>>>(mq, mk0, mk1, p);
    return cudaGetLastError();
}

}  // namespace peer
