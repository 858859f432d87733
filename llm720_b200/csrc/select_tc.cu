// Product-key selection on the tensor cores (bf16 layers): the two sub-key
// score contractions run as tcgen05 MMAs with fp32 accumulators in TMEM, and
// the per-half top-k, the candidate sums, the final top-k, the softmax and
// the flat expert ids are computed from TMEM by the scan warps.  No score
// reaches HBM.
//
// Follows llm/models/experts.py:153-163 (scores), :168-192 (per-half top-k'),
// :203-259 (candidate sums, flat ids, final top-k) and :327 (softmax).
//
// Exactness.  The reference's fp32 scores are reproduced to fp32 rounding
// level, not approximated: the normalised query half is fed as three bf16
// terms (hi + mid + lo carry the 24 bits of the fp32 value), the sub-keys of a
// bf16 layer are exactly representable, every bf16 x bf16 product is exact in
// fp32, and the three partial contractions accumulate in the same fp32 TMEM
// accumulator.  The key's 1/||k|| is applied afterwards.
//
// Layout of the work.  One CTA owns a tile of 128 (token, head) rows at a time
// (persistent grid).  The accumulator is KEY-major: M = 128 sub-keys (one chunk
// of the table), N = the 128 rows, so a TMEM lane is a key and a scan thread
// that reads 32 columns holds the scores of 32 rows for ITS key.
//
// Per tile and query half, two passes over the sub-key table (the tensor cores
// recompute the scores for the second pass; they are otherwise idle).  The
// first pass only has to produce a LOWER BOUND of each row's 16th best score,
// so with normalised queries it contracts two of the three bf16 terms of the
// query (hi + mid): two thirds of the MMAs.  Dropping lo changes a score by at
// most eps = 2^-16 ||k|| / max(||k||, 1e-12) (Cauchy-Schwarz with ||q|| = 1; hi and
// mid each leave a relative remainder of 2^-8 per element; key_prep_kernel
// takes the maximum over the table), and 16 distinct keys reach the 16th
// largest group maximum t of those scores, so the exact 16th best score is at
// least t - eps: that is the bound the exact second pass collects against.
// (One term and sub-keys rounded to bf16 after normalisation, a third of the
// MMAs and no scaling, was measured too: its eps of 6e-3 adds three candidates
// per row, enough list overflows to cost more than the MMAs saved.)
//   pass 0  every lane keeps, per row, the running maximum of its own keys
//           (one key per chunk); afterwards 4 adjacent lanes are combined with
//           two shuffles, which gives 32 group maxima per row in shared
//           memory; the 16th largest of them is a lower bound of the row's
//           16th best score (16 distinct scores reach it) and typically only
//           about 22 scores of a 1024-key table reach it;
//   pass 1  every lane compares its scores with the rows' bounds and notes
//           its own hits (score into a private shared-memory slot, row into a
//           bit mask) without votes or branches, then the lanes append their
//           hits to the rows' candidate lists (shared-memory atomicAdd for the
//           position); a list longer than CAP continues in a small pool shared
//           by 32 rows;
//   then    per row, a bitonic sort of the candidates by four adjacent lanes
//           (eight rows' networks side by side in a warp; a list that went on
//           into the pool takes a one-lane-per-candidate sort with the pool
//           entries inserted afterwards); the 16 best stay, in order.
// After both halves: the k best sums A[a] + B[b] of the two sorted lists, taken
// one at a time as the largest head of the 16 sequences "a fixed, b ascending"
// (four lanes per row hold four heads each; two shuffles per step), softmax,
// ids; eight rows per warp side by side.
// A row that loses a candidate (a lane with more than STAGE_CAP hits in one
// chunk, or a full pool: heavily clustered scores) is written to a list that
// the exact CUDA-core kernel reprocesses (select_simt.cu), so the result never
// depends on the bound heuristic.
//
// Warps: 0 = TMA producer, 1 = MMA issuer, 2-3 only take part in the set-up
// and the final barrier, 4-19 = 16 scan warps (scan warp s reads TMEM lanes
// 32*(s&3).. and columns 32*(s>>2)..).  The four warps with the same s>>2
// produce and consume everything that belongs to their 32 rows (group maxima,
// bounds, candidate lists, pool), so they synchronise among themselves only
// (one named barrier per group) and the four groups drift apart by up to the
// four accumulators in flight.
// Few rows (a decode-shaped batch, under a wave of 128-row tiles on a quarter of the SMs): tiles of 32 rows.  Four
// times as many SMs take part; a CTA then contracts with N = 32 and only the first set of four scan warps works,
// each lane on the same 32 rows per key as before, so a row's scores, bound and candidates - and with them the
// result - are what the 128-row tiles give.
// Ordering among exactly equal scores: smaller sub-key index first (per half),
// smaller candidate position first (final), as in select_simt.cu.
#include <float.h>
#include <limits.h>

#include "kernels.h"
#include "tc_common.cuh"

namespace peer {

namespace {

constexpr int BM = 128;            // rows per tile (MMA N)
constexpr int NC = 128;            // keys per chunk (MMA M)
constexpr int BOX_BYTES = 128 * 64 * 2;   // one TMA box: 128 rows x 64 bf16
constexpr int MAX_KA = 2;          // 64-column boxes per half (half width 64 or 128)
constexpr int Q_BYTES = 3 * MAX_KA * BOX_BYTES;     // 96 KB: query tile, three terms
constexpr int K_STAGE_BYTES = MAX_KA * BOX_BYTES;   // 32 KB: one key chunk
constexpr int K_STAGES = 2;
constexpr int N_ACC = 4;
constexpr int MAX_GROUPS = 32;     // key groups per row and half whose maxima bound the 16th best score
constexpr int CAP = 32;            // candidates per row and half
constexpr int LK = 16;             // list length per half (top_k and k' <= 16)
constexpr int SCAN_WARPS = 16;
constexpr int POOL = 64;           // candidates beyond CAP, per group of 32 rows (4 such pools per tile)
constexpr int LOST = 1 << 20;      // added to a row's count when one of its candidates could not be kept
constexpr int STAGE_CAP = 12;      // scores a lane can hold back per chunk before they go to the row lists: a sub-key that
                                   // is a hit in more than this many of a lane's 32 rows sends the surplus rows to the
                                   // exact kernel (with 12 a key in the top 16 of every fifth row still never does)
constexpr int GMAX_PITCH = 33;     // floats per key group in a row group's block of maxima (32 rows + 1: no bank conflicts)
constexpr int GROUP_BLOCK = STAGE_CAP * 128 > 32 * GMAX_PITCH ? STAGE_CAP * 128 : 32 * GMAX_PITCH;   // floats per row group
constexpr int CAND_PITCH = CAP + 1; // (score, sub-key) entries per row of the candidate lists: odd, so that the four-lanes-per-
                                   // row loads of eight rows spread over the banks
constexpr int THREADS = 128 + SCAN_WARPS * 32;
constexpr int CTRL_REGS = 24, SCAN_REGS = 112;     // 128*24 + 512*112 <= 640*96 registers at launch
constexpr uint32_t TMEM_COLS = 512;

struct Smem {
    static constexpr size_t q_off = 0;
    static constexpr size_t k_off = q_off + Q_BYTES;
    // group maxima, one block of GROUP_BLOCK floats per group of 32 rows (= per set of four scan warps):
    // [MAX_GROUPS][GMAX_PITCH].  The same block serves its four warps as staging slots in pass 1 ([STAGE_CAP][128]), when their own
    // group maxima are dead.  Blocks of different row groups never overlap: the four sets of warps run up to
    // N_ACC accumulators apart, so one may be in pass 1 while another still reads its group maxima.
    static constexpr size_t gmax_off = k_off + static_cast<size_t>(K_STAGES) * K_STAGE_BYTES;
    static constexpr size_t cand_off = gmax_off + 4 * GROUP_BLOCK * 4;                           // [128][CAND_PITCH] (key, col)
    static constexpr size_t cnt_off = cand_off + BM * CAND_PITCH * 8;                            // [128] int
    static constexpr size_t tau_off = cnt_off + BM * 4;                                          // [128] int
    static constexpr size_t pool_off = tau_off + BM * 4;                                         // [POOL] (row, score, sub-key, -)
    static constexpr size_t bar_off = pool_off + 4 * POOL * 16;
    static constexpr size_t total = bar_off + 16 * sizeof(uint64_t) + 32 + 1008;
};
static_assert(Smem::total <= 227 * 1024, "shared memory budget");
static_assert(STAGE_CAP * 128 <= GROUP_BLOCK && MAX_GROUPS * GMAX_PITCH <= GROUP_BLOCK, "a row group's staging slots reuse its own group maxima");

struct SelTcParams {
    const float* invn0; const float* invn1;   // 1/||key|| per sub-key (or 1)
    int64_t rows;                             // T * H
    int64_t term_rows;                        // row distance between the hi/mid/lo query arrays
    int Q, n0, n1, kp0, kp1, k, mult0, mult1;
    int32_t* ids32; float* weights; int64_t* ids64; float* raw_scores; int32_t* prod_ids;
    int* status;
    int32_t* overflow_rows; int* overflow_count;   // rows left to the exact kernel
    unsigned long long* stats;                     // optional [2]: pooled row-halves, rows left to the exact kernel
    int fast0;                                     // pass 0 contracts two query terms instead of three
    int bm;                                        // rows per tile: 128, or 32 for small batches (more CTAs, a quarter of the scan warps each)
    int vec_out;                                   // k == 16 and every output array 16-byte aligned: vector stores
    const float* eps0; const float* eps1;          // fast0: largest error of such a score, per table (device scalars)
};

// ---- bitonic networks over 32 elements held by FOUR ADJACENT LANES, eight per lane (element i = 8 * sub + e, sub =
// lane & 3).  A warp sorts the lists of eight rows at once, each in its own group of four lanes; two thirds of the
// compare-exchanges stay inside a lane, on registers, and only the strides 8 and 16 need a shuffle.  Result:
// descending in i.  Direction of a compare-exchange at merge size K for element i: the lower index keeps the larger
// value when (i & K) == 0 or K == 32.
__device__ __forceinline__ void cx_val(float& a, float& b, bool a_gets_max) {
    const float hi = fmaxf(a, b), lo = fminf(a, b);
    a = a_gets_max ? hi : lo;
    b = a_gets_max ? lo : hi;
}
// the same with a payload, ordered by (value descending, payload ascending): equal scores come out in the order of
// their sub-key indices whatever slots the candidates arrived in, so a row's result does not depend on timing
__device__ __forceinline__ void cx_pair(float& va, int& ca, float& vb, int& cb, bool a_gets_max) {
    const bool a_first = (va > vb) || (va == vb && ca < cb);
    const bool swap = a_first != a_gets_max;
    const float tv = swap ? vb : va;
    const int tc = swap ? cb : ca;
    vb = swap ? va : vb; cb = swap ? ca : cb;
    va = tv; ca = tc;
}
// strides 4, 2, 1 inside a lane
__device__ __forceinline__ void g4_in_lane_val(float (&v)[8], int from_stride, bool a_gets_max) {
#pragma unroll
    for (int j = 4; j > 0; j >>= 1) {
        if (j > from_stride) continue;
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if ((e & j) == 0) cx_val(v[e], v[e | j], a_gets_max);
    }
}
__device__ __forceinline__ void g4_in_lane_pair(float (&v)[8], int (&c)[8], int from_stride, bool a_gets_max) {
#pragma unroll
    for (int j = 4; j > 0; j >>= 1) {
        if (j > from_stride) continue;
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if ((e & j) == 0) cx_pair(v[e], c[e], v[e | j], c[e | j], a_gets_max);
    }
}
// merge sizes 2 and 4: the direction alternates inside a lane
__device__ __forceinline__ void g4_first_stages_val(float (&v)[8]) {
#pragma unroll
    for (int e = 0; e < 8; e += 2) cx_val(v[e], v[e + 1], (e & 2) == 0);                  // K = 2
#pragma unroll
    for (int e = 0; e < 8; ++e) if ((e & 2) == 0) cx_val(v[e], v[e | 2], (e & 4) == 0);     // K = 4, stride 2
#pragma unroll
    for (int e = 0; e < 8; e += 2) cx_val(v[e], v[e + 1], (e & 4) == 0);                  // K = 4, stride 1
}
__device__ __forceinline__ void g4_first_stages_pair(float (&v)[8], int (&c)[8]) {
#pragma unroll
    for (int e = 0; e < 8; e += 2) cx_pair(v[e], c[e], v[e + 1], c[e + 1], (e & 2) == 0);
#pragma unroll
    for (int e = 0; e < 8; ++e) if ((e & 2) == 0) cx_pair(v[e], c[e], v[e | 2], c[e | 2], (e & 4) == 0);
#pragma unroll
    for (int e = 0; e < 8; e += 2) cx_pair(v[e], c[e], v[e + 1], c[e + 1], (e & 4) == 0);
}
// stride 8 or 16: the partner element lives in the lane `lane_xor` away; keep the larger when keep_max
__device__ __forceinline__ void g4_cross_val(float (&v)[8], int lane_xor, bool keep_max) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float o = __shfl_xor_sync(FULL_MASK, v[e], lane_xor);
        v[e] = keep_max ? fmaxf(v[e], o) : fminf(v[e], o);
    }
}
__device__ __forceinline__ void g4_cross_pair(float (&v)[8], int (&c)[8], int lane_xor, bool keep_max) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float ov = __shfl_xor_sync(FULL_MASK, v[e], lane_xor);
        const int oc = __shfl_xor_sync(FULL_MASK, c[e], lane_xor);
        const bool mine_first = (v[e] > ov) || (v[e] == ov && c[e] < oc);
        const bool take = mine_first != keep_max;
        v[e] = take ? ov : v[e];
        c[e] = take ? oc : c[e];
    }
}
// the 16th largest of a row's 32 values: valid in the lanes with sub < 2
__device__ __forceinline__ float g4_sixteenth_largest(float (&v)[8], int sub) {
    const bool d8 = (sub & 1) == 0, d16 = (sub & 2) == 0;
    g4_first_stages_val(v);
    g4_in_lane_val(v, 4, d8);                                 // K = 8
    g4_cross_val(v, 1, d8 == d16);                            // K = 16, stride 8
    g4_in_lane_val(v, 4, d16);
    g4_cross_val(v, 2, true);                                 // K = 32, stride 16: the lower half now holds the 16 largest
    float m = v[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) m = fminf(m, v[e]);
    return fminf(m, __shfl_xor_sync(FULL_MASK, m, 1));
}
// full sort, descending in i = 8 * sub + e
__device__ __forceinline__ void g4_sort_pairs(float (&v)[8], int (&c)[8], int sub) {
    const bool d8 = (sub & 1) == 0, d16 = (sub & 2) == 0;
    g4_first_stages_pair(v, c);
    g4_in_lane_pair(v, c, 4, d8);                             // K = 8
    g4_cross_pair(v, c, 1, d8 == d16);                        // K = 16
    g4_in_lane_pair(v, c, 4, d16);
    g4_cross_pair(v, c, 2, d16);                              // K = 32
    g4_cross_pair(v, c, 1, d8);
    g4_in_lane_pair(v, c, 4, true);
}

__global__ void __launch_bounds__(THREADS, 1)
select_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k0,
                 const __grid_constant__ CUtensorMap map_k1, const SelTcParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* s_gmax = reinterpret_cast<float*>(smem + Smem::gmax_off); // [row group][key group][GMAX_PITCH]
    int2* s_cand = reinterpret_cast<int2*>(smem + Smem::cand_off);   // [row][CAP] (score key, sub-key index)
    int* s_cnt = reinterpret_cast<int*>(smem + Smem::cnt_off);
    float* s_tau = reinterpret_cast<float*>(smem + Smem::tau_off);
    int4* s_pool = reinterpret_cast<int4*>(smem + Smem::pool_off);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::bar_off);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    int* s_pool_cnt = reinterpret_cast<int*>(tmem_slot + 1);
    const uint32_t sQ = smem_u32(smem + Smem::q_off), sK = smem_u32(smem + Smem::k_off);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, q_empty = bar0 + 8;
    auto k_full = [&](int s) { return bar0 + 8u * (2 + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (2 + K_STAGES + s); };
    auto acc_full = [&](int a) { return bar0 + 8u * (2 + 2 * K_STAGES + a); };
    auto acc_empty = [&](int a) { return bar0 + 8u * (2 + 2 * K_STAGES + N_ACC + a); };
    const uint32_t q_box = static_cast<uint32_t>(p.bm) * 128u;          // bytes of one query box: bm rows x 64 bf16

    if (tid == 0) {
        mbar_init(q_full, 1); mbar_init(q_empty, 1);
        for (int s = 0; s < K_STAGES; ++s) { mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1); }
        for (int a = 0; a < N_ACC; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), p.bm * 4); }   // the scan threads of the tile's rows
        mbar_fence_init();
        tc::tma_prefetch_desc(&map_q); tc::tma_prefetch_desc(&map_k0); tc::tma_prefetch_desc(&map_k1);
    }
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
    const int64_t n_tiles = (p.rows + p.bm - 1) / p.bm;
    const uint32_t q_bytes = 3u * KA * q_box, k_bytes = static_cast<uint32_t>(KA) * BOX_BYTES;

    // The control warps need few registers; the rest of the launch allocation goes to the scan warps.
    if (warp < 4) {
      // (one value for the four control warps: the warps of a warpgroup must execute the same setmaxnreg)
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(CTRL_REGS));
      if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t q_phase = 0; int stage = 0; uint32_t k_phase = 0; bool ok = true;
            for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                for (int hf = 0; hf < 2 && ok; ++hf) {
                    if (!mbar_wait_hint(q_empty, q_phase ^ 1, p.status)) { ok = false; break; }
                    q_phase ^= 1;
                    mbar_expect_tx(q_full, q_bytes);
                    for (int t = 0; t < 3; ++t)
                        for (int ka = 0; ka < KA; ++ka)
                            tc::tma_load_2d(sQ + (t * KA + ka) * q_box, &map_q, hf * hw + ka * 64,
                                            static_cast<int>(t * p.term_rows + tile * p.bm), q_full);
                    const int nch = hf ? nch1 : nch0;
                    const CUtensorMap* mk = hf ? &map_k1 : &map_k0;
                    for (int c2 = 0; c2 < 2 * nch; ++c2) {          // two passes over the sub-keys
                        const int c = c2 < nch ? c2 : c2 - nch;
                        if (!mbar_wait_hint(k_empty(stage), k_phase ^ 1, p.status)) { ok = false; break; }
                        mbar_expect_tx(k_full(stage), k_bytes);
                        for (int ka = 0; ka < KA; ++ka)
                            tc::tma_load_2d(sK + stage * K_STAGE_BYTES + ka * BOX_BYTES, mk, ka * 64, c * NC, k_full(stage));
                        if (++stage == K_STAGES) { stage = 0; k_phase ^= 1; }
                    }
                }
            }
        }
      } else if (warp == 1) {
        // ---------------- MMA issuer: D[key, row] = sum over the three query terms of K . q^T ----------------
        if (lane == 0) {
            const uint32_t idesc = tc::idesc_bf16_f32(NC, p.bm);        // a narrow tile contracts its 32 rows only
            uint32_t q_phase = 0; int stage = 0; uint32_t k_phase = 0; uint32_t g = 0; bool ok = true;
            for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                for (int hf = 0; hf < 2 && ok; ++hf) {
                    if (!mbar_wait_hint(q_full, q_phase, p.status)) { ok = false; break; }
                    q_phase ^= 1;
                    const int nch = hf ? nch1 : nch0;
                    for (int c = 0; c < 2 * nch; ++c, ++g) {
                        const int acc = g & (N_ACC - 1);
                        if (!mbar_wait_hint(acc_empty(acc), ((g / N_ACC) & 1) ^ 1, p.status)) { ok = false; break; }
                        if (!mbar_wait_hint(k_full(stage), k_phase, p.status)) { ok = false; break; }
                        tc::fence_after_sync();
                        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * BM;
                        uint32_t first = 0;
                        const int terms = (c < nch && p.fast0) ? 2 : 3;     // pass 0 of the fast form: hi + mid
                        for (int t = 0; t < terms; ++t)
                            for (int ka = 0; ka < KA; ++ka) {
                                const uint64_t kd = tc::smem_desc_sw128(sK + stage * K_STAGE_BYTES + ka * BOX_BYTES);
                                const uint64_t qd = tc::smem_desc_sw128(sQ + (t * KA + ka) * q_box);
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    tc::umma_bf16(d_tmem, kd + 2 * k, qd + 2 * k, idesc, first);
                                    first = 1;
                                }
                            }
                        tc::umma_commit(k_empty(stage));
                        tc::umma_commit(acc_full(acc));
                        if (++stage == K_STAGES) { stage = 0; k_phase ^= 1; }
                    }
                    if (ok) tc::umma_commit(q_empty);     // the query tile of this half is no longer read
                }
            }
        }
      }
    } else {
        // ---------------- scan warps ----------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SCAN_REGS));
        const int s = warp - 4;                        // 0..15
        const int quarter = warp & 3;                  // TMEM lanes (keys) 32*quarter..
        const int cg = s >> 2;                         // TMEM columns (rows) 32*cg..
        const int half16 = lane & 16;                  // rows 4..7 of a warp keep their lists in lanes 16..31
        uint32_t g = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < n_tiles && cg * 32 < p.bm; tile += gridDim.x) {
            // sorted lists of my 8 rows, per half: rows 0-3 in lanes 0-15, rows 4-7 in lanes 16-31
            float hv[2][4]; int hc[2][4];
            unsigned overflow = 0;                     // bit rr: row 8s+rr overflowed its candidate list
#pragma unroll 1
            for (int hf = 0; hf < 2; ++hf) {
                const int n = hf ? p.n1 : p.n0;
                const int nch = hf ? nch1 : nch0;
                const float* __restrict__ invn = hf ? p.invn1 : p.invn0;
#pragma unroll 1
                for (int pass = 0; pass < 2; ++pass) {
                    // pass 0: bnd[j] = largest score of my keys (one per chunk) for row j;
                    // pass 1: bnd[j] = the bound of row j
                    float bnd[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) bnd[j] = pass ? s_tau[cg * 32 + j] : -INFINITY;
                    for (int ch = 0; ch < nch; ++ch, ++g) {
                        const int acc = g & (N_ACC - 1);
                        if (ok && !mbar_wait_hint(acc_full(acc), (g / N_ACC) & 1, p.status)) ok = false;
                        if (!ok) continue;
                        tc::fence_after_sync();
                        uint32_t r[32];
                        tc::tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc) * BM + cg * 32, r);
                        const int key = ch * NC + quarter * 32 + lane;       // this lane's sub-key
                        // keys past the end of the table get a NaN scale: their scores lose every comparison
                        const float sc = key < n ? __ldg(invn + key) : __int_as_float(0x7fc00000);
                        tc::tmem_ld_wait();
                        tc::fence_before_sync();
                        mbar_arrive(acc_empty(acc));                         // scores are in registers
                        if (pass == 0) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) bnd[j] = fmaxf(bnd[j], __uint_as_float(r[j]) * sc);
                        } else {
                            // Every lane notes its own hits (score into a private slot, row into a bit
                            // mask) without votes or branches, then the lanes append their hits to the
                            // rows' lists side by side.
                            float* slot = s_gmax + cg * GROUP_BLOCK + quarter * 32 + lane;   // this row group's block
                            constexpr uint32_t SLOT_STEP = 128 * 4;                      // bytes between a lane's slots
                            uint32_t addr = smem_u32(slot);
                            const uint32_t last = addr + (STAGE_CAP - 1) * SLOT_STEP;
                            unsigned myhits = 0;
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const float x = __uint_as_float(r[j]) * sc;
                                if (x >= bnd[j]) {                       // three predicated instructions, no branch
                                    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(x) : "memory");
                                    addr = min(addr + SLOT_STEP, last);
                                    myhits |= 1u << j;
                                }
                            }
                            const int nh = __popc(myhits);
                            int taken = 0;
                            while (myhits) {
                                {
                                    const int row = cg * 32 + __ffs(myhits) - 1;
                                    myhits &= myhits - 1;
                                    if (taken < STAGE_CAP - 1 || nh <= STAGE_CAP) {
                                        const float x = slot[taken * 128];
                                        const int pos = atomicAdd(&s_cnt[row], 1);
                                        if (pos < CAP) {
                                            s_cand[row * CAND_PITCH + pos] = make_int2(__float_as_int(x), key);
                                        } else {                             // a long list continues in the tile's pool
                                            const int pp = atomicAdd(s_pool_cnt + cg, 1);
                                            if (pp < POOL) s_pool[cg * POOL + pp] = make_int4(row, __float_as_int(x), key, 0);
                                            else atomicAdd(&s_cnt[row], LOST);
                                        }
                                    } else {
                                        atomicAdd(&s_cnt[row], LOST);        // slot lost: the row goes to the exact kernel
                                    }
                                    ++taken;
                                }
                            }
                            __syncwarp();
                        }
                    }
                    if (pass == 0) {
                        // group maxima: 4 adjacent lanes x all chunks = one group; 8 groups per warp, 32 per row.
                        // Each exchange halves what a lane keeps (the partner gets the other half), so the four
                        // lanes end with 8 rows' maxima each: 24 shuffles instead of 64.
                        const bool up1 = lane & 1, up2 = lane & 2;
                        float h1[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {                   // h1[i]: row i + 16 * up1
                            const float got = __shfl_xor_sync(FULL_MASK, up1 ? bnd[i] : bnd[i + 16], 1);
                            h1[i] = fmaxf(up1 ? bnd[i + 16] : bnd[i], got);
                        }
                        float* gm = s_gmax + cg * GROUP_BLOCK + (quarter * 8 + (lane >> 2)) * GMAX_PITCH + (up1 ? 16 : 0) + (up2 ? 8 : 0);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {                    // row i + 8 * up2 + 16 * up1
                            const float got = __shfl_xor_sync(FULL_MASK, up2 ? h1[i] : h1[i + 8], 2);
                            gm[i] = fmaxf(up2 ? h1[i + 8] : h1[i], got);
                        }
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(1 + cg) : "memory");      // the four warps that share these 32 rows
                    if (pass == 0) {
                        // bound of my 8 rows: the 16th largest of the row's 32 group maxima (16 distinct scores reach it).
                        // Four lanes per row: lane 4*rr + sub holds the maxima of key groups 8*sub .. 8*sub+7 of row rr.
                        const int rr = lane >> 2, sub = lane & 3;
                        float tv[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) tv[e] = s_gmax[cg * GROUP_BLOCK + (sub * 8 + e) * GMAX_PITCH + quarter * 8 + rr];
                        // fast form: the group maxima lack the lo term; the exact 16th best score is at least t - eps
                        const float eps = p.fast0 ? __ldg(hf ? p.eps1 : p.eps0) : 0.f;
                        const float t = g4_sixteenth_largest(tv, sub) - eps;
                        if (sub == 0) { s_tau[s * 8 + rr] = t; s_cnt[s * 8 + rr] = 0; }
                        if ((s & 3) == 0 && lane == 0) s_pool_cnt[cg] = 0;
                        asm volatile("bar.sync %0, 128;" ::"r"(1 + cg) : "memory");      // the four warps that share these 32 rows
                    }
                }
                // the 16 best candidates of my 8 rows, in order (score descending, sub-key ascending)
                bool sorted_fast = false;
                {
                    // Common case, no list of these rows went on into the pool: four lanes per row sort the row's (at most
                    // 32) candidates on registers; the sorted best 16 go back to the row's own list memory and are read
                    // from there in the layout the final combine uses (rows 0-3 in lanes 0-15, rows 4-7 in lanes 16-31).
                    const int rr = lane >> 2, sub = lane & 3;
                    const int row = s * 8 + rr;
                    const int cnt = s_cnt[row];
                    const bool lost = cnt >= LOST;
                    if (!__any_sync(FULL_MASK, !lost && cnt > CAP)) {
                        const unsigned lm = __ballot_sync(FULL_MASK, lost);
#pragma unroll
                        for (int q = 0; q < 8; ++q) overflow |= ((lm >> (4 * q)) & 1u) << q;
                        float v[8]; int c[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            v[e] = -INFINITY; c[e] = INT_MAX;
                            if (sub * 8 + e < min(cnt, CAP)) {
                                const int2 en = s_cand[row * CAND_PITCH + sub * 8 + e];
                                v[e] = __int_as_float(en.x); c[e] = en.y;
                            }
                        }
                        g4_sort_pairs(v, c, sub);
                        __syncwarp();                            // every lane of a row has read the list before it is rewritten
                        if (sub < 2) {
#pragma unroll
                            for (int e = 0; e < 8; ++e) s_cand[row * CAND_PITCH + sub * 8 + e] = make_int2(__float_as_int(v[e]), c[e]);
                        }
                        __syncwarp();
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int2 en = s_cand[(s * 8 + (half16 ? 4 : 0) + q) * CAND_PITCH + (lane & 15)];
                            if (hf == 0) { hv[0][q] = __int_as_float(en.x); hc[0][q] = en.y; }
                            else { hv[1][q] = __int_as_float(en.x); hc[1][q] = en.y; }
                        }
                        sorted_fast = true;
                    }
                }
                // otherwise (a list of these rows continues in the pool: rare) one lane per candidate, four rows side by side
#pragma unroll 1
                for (int rb = 0; rb < 8 && !sorted_fast; rb += 4) {
                    float v[4]; int c[4];
                    unsigned pooled = 0;                     // bit q: the row's list continues in the pool
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int row = s * 8 + rb + q;
                        const int cnt = s_cnt[row];
                        if (cnt >= LOST) overflow |= 1u << (rb + q);
                        else if (cnt > CAP) {
                            pooled |= 1u << q;
                            if (p.stats && lane == 0 && tile * p.bm + row < p.rows) atomicAdd(p.stats, 1ULL);
                        }
                        v[q] = -INFINITY; c[q] = INT_MAX;
                        if (lane < min(cnt, CAP)) { const int2 e = s_cand[row * CAND_PITCH + lane]; v[q] = __int_as_float(e.x); c[q] = e.y; }
                    }
#pragma unroll
                    for (int k = 2; k <= 32; k <<= 1)
#pragma unroll
                        for (int j = k >> 1; j > 0; j >>= 1) {
                            const bool keep_first = ((lane & j) == 0) == ((lane & k) == 0 || k == 32);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float ov = __shfl_xor_sync(FULL_MASK, v[q], j);
                                const int oc = __shfl_xor_sync(FULL_MASK, c[q], j);
                                const bool mine_first = (v[q] > ov) || (v[q] == ov && c[q] < oc);
                                const bool keep_mine = mine_first == keep_first;
                                v[q] = keep_mine ? v[q] : ov;
                                c[q] = keep_mine ? c[q] : oc;
                            }
                        }
                    if (pooled) {                            // rare: insert the pool's entries of these rows
                        const int np = min(s_pool_cnt[cg], POOL);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (!(pooled & (1u << q))) continue;
                            for (int e = 0; e < np; ++e) {
                                const int4 pe = s_pool[cg * POOL + e];
                                if (pe.x != s * 8 + rb + q) continue;
                                const float ex = __int_as_float(pe.y);
                                const bool before = (v[q] > ex) || (v[q] == ex && c[q] < pe.z);
                                const int at = __popc(__ballot_sync(FULL_MASK, before));
                                const float uv = __shfl_up_sync(FULL_MASK, v[q], 1);
                                const int uc = __shfl_up_sync(FULL_MASK, c[q], 1);
                                if (lane == at) { v[q] = ex; c[q] = pe.z; }
                                else if (lane > at) { v[q] = uv; c[q] = uc; }
                            }
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (rb) {                            // move lanes 0..15 to lanes 16..31
                            v[q] = __shfl_sync(FULL_MASK, v[q], lane & 15);
                            c[q] = __shfl_sync(FULL_MASK, c[q], lane & 15);
                        }
                        if ((rb != 0) == (half16 != 0)) {
                            if (hf == 0) { hv[0][q] = v[q]; hc[0][q] = c[q]; } else { hv[1][q] = v[q]; hc[1][q] = c[q]; }
                        }
                    }
                }
            }
            if (!ok) continue;
            // ---- the k best pair sums of each row, softmax, ids.  Both lists are sorted, so the sums A[a] + B[b] form one
            // sequence per a that descends in b, and the best sum not yet taken is always the head of a sequence.  Four
            // lanes per row (lane 4 * rr + sub keeps the heads of a = 4 * sub .. 4 * sub + 3), the warp's 8 rows at once:
            // k steps of "largest head of the row, advance that sequence".  Equal sums go to the smaller a * 16 + b.
            {
#pragma unroll
                for (int q = 0; q < 4; ++q) {                  // the lists go to row memory: B at slots 0..15, A at 16..31
                    int2* rowm = s_cand + (s * 8 + (half16 ? 4 : 0) + q) * CAND_PITCH;
                    rowm[lane & 15] = make_int2(__float_as_int(hv[1][q]), hc[1][q]);
                    rowm[16 + (lane & 15)] = make_int2(__float_as_int(hv[0][q]), hc[0][q]);
                }
                __syncwarp();
                const int rr = lane >> 2, sub = lane & 3;
                const int2* rowm = s_cand + (s * 8 + rr) * CAND_PITCH;
                const int64_t grow = tile * p.bm + s * 8 + rr;
                const bool lost_row = (overflow >> rr) & 1u;
                if (grow < p.rows && lost_row && sub == 0) {   // left to the exact kernel
                    p.overflow_rows[atomicAdd(p.overflow_count, 1)] = static_cast<int32_t>(grow);
                    if (p.stats) atomicAdd(p.stats + 1, 1ULL);
                }
                float av[4], head[4];
                int hpos[4];                                   // a * 16 + b of each head
                const float b_first = __int_as_float(rowm[0].x);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int a = sub * 4 + i;
                    av[i] = __int_as_float(rowm[16 + a].x);
                    hpos[i] = a * 16;
                    head[i] = a < p.kp0 ? av[i] + b_first : -INFINITY;
                }
                float ov[4]; int op[4];                        // results it = 4 * sub .. 4 * sub + 3 of the row
#pragma unroll
                for (int j = 0; j < 4; ++j) { ov[j] = -INFINITY; op[j] = 0; }
#pragma unroll
                for (int it = 0; it < LK; ++it) {
                    if (it < p.k) {                            // warp-uniform
                        float bv = head[0]; int bp = hpos[0];
#pragma unroll
                        for (int i = 1; i < 4; ++i) {          // a ascends with i: strict compare keeps the smaller a
                            const bool better = head[i] > bv;
                            bv = better ? head[i] : bv; bp = better ? hpos[i] : bp;
                        }
#pragma unroll
                        for (int m = 1; m <= 2; m <<= 1) {
                            const float xv = __shfl_xor_sync(FULL_MASK, bv, m);
                            const int xp = __shfl_xor_sync(FULL_MASK, bp, m);
                            const bool other = (xv > bv) || (xv == bv && xp < bp);
                            bv = other ? xv : bv; bp = other ? xp : bp;
                        }
                        if ((it >> 2) == sub) { ov[it & 3] = bv; op[it & 3] = bp; }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if ((bp >> 4) == sub * 4 + i) {    // my sequence was taken: its next element becomes the head
                                const int nb = (bp & 15) + 1;
                                if (nb < p.kp1) { hpos[i] = bp + 1; head[i] = av[i] + __int_as_float(rowm[nb].x); }
                                else head[i] = -INFINITY;
                            }
                        }
                    }
                }
                const float top = __shfl_sync(FULL_MASK, ov[0], lane & ~3);
                float e[4], sum = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) { e[j] = sub * 4 + j < p.k ? expf(ov[j] - top) : 0.f; sum += e[j]; }
                sum += __shfl_xor_sync(FULL_MASK, sum, 1);
                sum += __shfl_xor_sync(FULL_MASK, sum, 2);
                if (grow < p.rows && !lost_row) {
                    int i0[4], i1[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) { i0[j] = rowm[16 + (op[j] >> 4)].y; i1[j] = rowm[op[j] & 15].y; }
                    if (p.vec_out) {                           // k == 16, 16-byte aligned outputs: one store per array
                        const int64_t o = grow * LK + sub * 4;
                        const int4 id = make_int4(i0[0] * p.mult0 + i1[0] * p.mult1, i0[1] * p.mult0 + i1[1] * p.mult1,
                                                  i0[2] * p.mult0 + i1[2] * p.mult1, i0[3] * p.mult0 + i1[3] * p.mult1);
                        if (p.ids32) *reinterpret_cast<int4*>(p.ids32 + o) = id;
                        if (p.weights) *reinterpret_cast<float4*>(p.weights + o) = make_float4(e[0] / sum, e[1] / sum, e[2] / sum, e[3] / sum);
                        if (p.ids64) {
                            *reinterpret_cast<longlong2*>(p.ids64 + o) = make_longlong2(id.x, id.y);
                            *reinterpret_cast<longlong2*>(p.ids64 + o + 2) = make_longlong2(id.z, id.w);
                        }
                        if (p.raw_scores) *reinterpret_cast<float4*>(p.raw_scores + o) = make_float4(ov[0], ov[1], ov[2], ov[3]);
                        if (p.prod_ids) *reinterpret_cast<int4*>(p.prod_ids + o) = make_int4(i0[0] * p.n1 + i1[0], i0[1] * p.n1 + i1[1],
                                                                                             i0[2] * p.n1 + i1[2], i0[3] * p.n1 + i1[3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int it = sub * 4 + j;
                            if (it >= p.k) continue;
                            const int64_t o = grow * p.k + it;
                            const int id = i0[j] * p.mult0 + i1[j] * p.mult1;
                            if (p.ids32) p.ids32[o] = id;
                            if (p.weights) p.weights[o] = e[j] / sum;
                            if (p.ids64) p.ids64[o] = id;
                            if (p.raw_scores) p.raw_scores[o] = ov[j];
                            if (p.prod_ids) p.prod_ids[o] = i0[j] * p.n1 + i1[j];
                        }
                    }
                }
                __syncwarp();                                  // row memory is appended to again in the next tile
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

// What the selection needs of the two sub-key tables, in one launch (one warp per sub-key).  Per sub-key:
// invn[r] = 1 / max(||key||, 1e-12) (or 1), for the tensor-core kernel, which contracts with the keys as stored;
// khat[c][r] = key[c] / max(||key||, 1e-12) in fp32, transposed, for the exact kernel that redoes handed-over rows.
// Optionally also, as a running maximum per table, eps = 2^-16 * ||key|| * invn[r] * (1 + 2^-10) + 1e-6: how much a
// score can lose when the query's lo term is left out of the contraction (|lo . key| <= ||lo|| ||key||, ||lo|| <=
// 2^-16 for a unit query half; the last terms cover ||q|| = 1 up to rounding and the fp32 accumulation).
__global__ void key_prep_kernel(const __nv_bfloat16* __restrict__ keys0, const __nv_bfloat16* __restrict__ keys1,
                                int n0, int n1, int width, int do_norm, float* __restrict__ khat0,
                                float* __restrict__ khat1, float* __restrict__ invn0, float* __restrict__ invn1,
                                float* __restrict__ eps) {
    const int lane = threadIdx.x & 31;
    int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (r >= n0 + n1) return;
    const int table = r >= n0;
    if (table) r -= n0;
    const int n = table ? n1 : n0;
    const __nv_bfloat16* __restrict__ row = (table ? keys1 : keys0) + static_cast<int64_t>(r) * width;
    float* __restrict__ khat = table ? khat1 : khat0;
    float ss = 0.f;
    for (int c = lane; c < width; c += 32) {
        const float v = __bfloat162float(row[c]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float nrm = do_norm ? fmaxf(sqrtf(ss), 1e-12f) : 1.0f;
    for (int c = lane; c < width; c += 32) {
        const float v = __bfloat162float(row[c]);
        khat[static_cast<int64_t>(c) * n + r] = do_norm ? v / nrm : v;
    }
    const float inv = do_norm ? 1.0f / nrm : 1.0f;
    if (lane == 0) {
        (table ? invn1 : invn0)[r] = inv;
        if (eps) {
            const float e = 1.52587890625e-5f * sqrtf(ss) * inv * 1.0009765625f + 1e-6f;
            atomicMax(reinterpret_cast<int*>(eps + table), __float_as_int(e));  // positive floats order like their bit patterns
        }
    }
}

}  // namespace

bool select_tc_supported(int act_dtype, int Q, int n0, int n1, int k, int kp0, int kp1) {
    // lists of at most 16 per half; at least one full chunk of keys per table
    return act_dtype == PEER_DTYPE_BF16 && (Q == 128 || Q == 256) && k <= LK && kp0 <= LK && kp1 <= LK &&
           n0 >= 128 && n1 >= 128;
}

cudaError_t select_tc_setup() {
    return cudaFuncSetAttribute(select_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(Smem::total));
}

cudaError_t launch_key_prep(const void* keys0, const void* keys1, int n0, int n1, int width, int do_norm, float* khat0,
                            float* khat1, float* invn0, float* invn1, float* eps, cudaStream_t s) {
    if (eps) {
        const cudaError_t e = cudaMemsetAsync(eps, 0, 2 * sizeof(float), s);
        if (e != cudaSuccess) return e;
    }
    const unsigned blocks = static_cast<unsigned>((static_cast<int64_t>(n0 + n1) * 32 + 255) / 256);
    key_prep_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(keys0), static_cast<const __nv_bfloat16*>(keys1),
                                           n0, n1, width, do_norm, khat0, khat1, invn0, invn1, eps);
    return cudaGetLastError();
}

cudaError_t launch_select_tc(const SelectTcArgs& a, cudaStream_t s) {
    if (a.rows == 0) return cudaSuccess;
    const int hw = a.Q / 2;
    CUtensorMap mq, mk0, mk1;
    const int fast0 = a.eps0 && a.eps1;
    // Few rows (a decode-shaped batch): tiles of 32 rows, so that four times as many SMs take part and a tile's
    // chain of chunk steps is shorter (one set of four scan warps, MMAs of N = 32, a deeper key ring).  Same
    // results: a row's scores, bound and candidates do not depend on which rows share its tile.
    const int bm = ((a.rows + BM - 1) / BM) * 4 <= a.sm_count ? 32 : BM;
    if (!make_tensor_map_bf16(&mq, a.q_split, static_cast<uint64_t>(3 * a.term_rows), static_cast<uint64_t>(a.Q),
                              static_cast<uint64_t>(a.Q), bm) ||
        !make_tensor_map_bf16(&mk0, a.keys0, static_cast<uint64_t>(a.n0), static_cast<uint64_t>(hw),
                              static_cast<uint64_t>(hw), NC) ||
        !make_tensor_map_bf16(&mk1, a.keys1, static_cast<uint64_t>(a.n1), static_cast<uint64_t>(hw),
                              static_cast<uint64_t>(hw), NC))
        return cudaErrorInvalidValue;
    SelTcParams p;
    p.invn0 = a.invn0; p.invn1 = a.invn1; p.rows = a.rows; p.term_rows = a.term_rows; p.Q = a.Q;
    p.n0 = a.n0; p.n1 = a.n1; p.kp0 = a.kp0; p.kp1 = a.kp1; p.k = a.k; p.mult0 = a.mult0; p.mult1 = a.mult1;
    p.ids32 = a.ids32; p.weights = a.weights; p.ids64 = a.ids64; p.raw_scores = a.raw_scores; p.prod_ids = a.prod_ids; p.status = a.status;
    p.overflow_rows = a.overflow_rows; p.overflow_count = a.overflow_count; p.stats = a.stats;
    p.fast0 = fast0; p.eps0 = a.eps0; p.eps1 = a.eps1;
    const uintptr_t out_bits = reinterpret_cast<uintptr_t>(a.ids32) | reinterpret_cast<uintptr_t>(a.weights) |
                               reinterpret_cast<uintptr_t>(a.ids64) | reinterpret_cast<uintptr_t>(a.raw_scores) |
                               reinterpret_cast<uintptr_t>(a.prod_ids);
    p.vec_out = a.k == LK && (out_bits & 15u) == 0;
    p.bm = bm;
    const int64_t n_tiles = (a.rows + p.bm - 1) / p.bm;
    const unsigned grid = static_cast<unsigned>(n_tiles < a.sm_count ? n_tiles : a.sm_count);
    select_tc_kernel<<<grid, THREADS, Smem::total, s>>>(mq, mk0, mk1, p);
    return cudaGetLastError();
}

}  // namespace peer
