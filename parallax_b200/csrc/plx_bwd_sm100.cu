// Parallax training backward on the Blackwell tensor cores (tcgen05.mma, TMEM
// accumulators, TMA-staged tiles): one kernel template, two modes.
//
//   DQR: CTA = 128 query rows of one (batch, q head); streams key tiles of 64.
//        S1 = Q K^T, S2 = R K^T, A = dO V^T  ->  gl, gu  ->  dQ += gl K, dR += gu K
//   DKV: CTA = 128 keys of one (batch, kv head); streams 64-row tiles of q, r, dO
//        (and their row statistics) of every q head of the group.
//        S1^T = K Q^T, S2^T = K R^T, A^T = V dO^T  ->  gl^T, gu^T, W^T
//        ->  dK += gl^T Q + gu^T R, dV += W^T dO
//
// Formulas (parallax/triton/parallax_train.py:561-573 and :765-792 of the reference):
//   w = 2^(S1*c2 - m), p = w / d1, delta = A - b, cs = bart - S2
//   gl = p (A - t + cs delta), gu = -p delta, W = p (1 + cs); dQ and the gl part of dK carry qk_scale.
// Evaluated as W = p (1 + bart - S2), gl = W delta + p (b - t) with 1/d1 folded into the exponent.
//
// Pipeline per CTA (352 threads):
//   warp 0      TMA producer (resident tiles once, streamed tiles through an NS-deep ring)
//   warp 1      TMEM allocation + the lane that issues the score products
//   warp 10     the lane that issues the output products
//   warps 2-9   element-wise: the thread pair (w, w + 4) shares TMEM lane quarter w % 4
//               and splits the 64 columns; it reads the three score tiles from TMEM,
//               releases them at once (so the next tile's scores are computed while it
//               works), writes gl / gu / W as 16-bit tiles into shared memory in the
//               128-byte-swizzled K-major layout, and the MMA lane consumes them as the
//               A operand of the output products.
//
// TMEM columns: acc0 [0,128) (dQ | dK), acc1 [128,256) (dR | dV), S1 [256,320), S2 [320,384), A [384,448),
// and at [448,512) the M-side tile that is the A operand of score products: k in DKV mode (S1^T, S2^T), dO in DQR mode (A).
#include <cuda.h>

#include <climits>
#include <cstdlib>

#include "plx_common.cuh"
#include "plx_launch.h"
#include "plx_sm100.cuh"

namespace plx {

using namespace sm100;

namespace {

constexpr int kModeDQR = 0, kModeDKV = 1;
constexpr int kBM = 128, kBN = 64;
constexpr uint32_t kResPanel = kBM * 128;      // one 64-channel panel of a resident tile: [128][128 B]
constexpr uint32_t kStrPanel = kBN * 128;      // one 64-channel panel of a streamed tile: [64][128 B]
constexpr uint32_t kGBytes = kBM * kBN * 2;    // 16 KB gl / gu / W tile: [128][128 B]
constexpr uint32_t kTmemCols = 512;

template <typename T>
struct Fmt;
template <>
struct Fmt<__nv_bfloat16> {
    static constexpr int kUmma = 1;
    static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
};
template <>
struct Fmt<__half> {
    static constexpr int kUmma = 0;
    static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
};

constexpr uint32_t kStatBytes = kBN * 16;      // four planes of 64 floats: -mL, -(1 + bart), b, (b - t) * scale
constexpr int kStatStages = 2;
constexpr int kStatWriters = 64;               // one thread per row of the streamed tile

// DQR keeps q, r, dO of its rows in shared memory.  DKV keeps only v there: its k tile is the A
// operand of two of the three score products and lives in tensor memory (64 columns), which frees
// the shared memory for a third stage of streamed tiles.
// D = head dim (64 or 128): tiles are D / 64 panels.
template <int D, int MODE, int NS>
struct Smem {
    static constexpr int kPanels = D / 64;
    static constexpr uint32_t kResBytes = kPanels * kResPanel;   // resident tile (128 rows)
    static constexpr uint32_t kStrBytes = kPanels * kStrPanel;   // streamed tile (64 rows)
    static constexpr int kNRes = MODE == kModeDQR ? 2 : 1;   // DQR: q, r (its dO tile is in tensor memory); DKV: v
    static constexpr int kNStr = MODE == kModeDQR ? 2 : 3;
    static constexpr int kNG = MODE == kModeDQR ? 2 : 3;
    static constexpr uint32_t kRes = 0;
    static constexpr uint32_t kStr = kNRes * kResBytes;
    static constexpr uint32_t kStage = kNStr * kStrBytes;
    static constexpr uint32_t kG = kStr + NS * kStage;
    static constexpr uint32_t kStats = kG + kNG * kGBytes;
    static constexpr uint32_t kBars = kStats + (MODE == kModeDKV ? kStatStages * kStatBytes : 0);
    static constexpr int kXFull = 0, kNFull = 1, kNEmpty = 1 + NS, kSFull = 1 + 2 * NS, kSFree = kSFull + 1,
                         kGFull = kSFull + 2, kGFree = kSFull + 3, kAccDone = kSFull + 4, kKReady = kSFull + 5,
                         kStatFull = kSFull + 6, kNumBars = kStatFull + kStatStages;
    static constexpr uint32_t kTmemSlot = kBars + 8 * kNumBars;
    static constexpr uint32_t kLoc = kTmemSlot + 16;
    static constexpr uint32_t kBytes = kLoc + 16;   // the dynamic shared memory must start 1024-byte aligned
    static constexpr uint32_t kStageTx = kStage;
};

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

template <typename T, int D, int MODE, int NS>
__global__ void __launch_bounds__(352, 1)
bwd_sm100_kernel(const TrainArgs a, int n_tok, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_r, const __grid_constant__ CUtensorMap tm_go,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, int *err) {
    using L = Smem<D, MODE, NS>;
    constexpr bool DQR = MODE == kModeDQR;
    constexpr uint32_t kResBytes = L::kResBytes, kStrBytes = L::kStrBytes;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    int *s_loc = reinterpret_cast<int *>(smem_raw + L::kLoc);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        Seq s;
        int tis = 0;
        bool ok = locate_tile(a, DQR ? gridDim.x - 1 - blockIdx.x : blockIdx.x, kBM, s, tis);
        if (*reinterpret_cast<volatile int *>(err) != 0) ok = false;
        if ((smem_u32(smem_raw) & 1023u) != 0) {   // the swizzled tiles need a 1024-byte aligned base
            atomicCAS(err, 0, (12 << 8) | kErrWaitTimeout);
            ok = false;
        }
        s_loc[0] = ok ? s.bos : -1;
        s_loc[1] = s.nq;
        s_loc[2] = s.nk;
        s_loc[3] = tis;
    }
    __syncthreads();
    if (s_loc[0] < 0) return;
    const int bos = s_loc[0], nq = s_loc[1], nk = s_loc[2], m0 = s_loc[3] * kBM;  // first row (DQR) / key (DKV)
    if (m0 >= (DQR ? nq : nk)) return;
    const int heads_y = DQR ? a.heads_q : a.heads_kv;
    const int b = blockIdx.y / heads_y, hy = blockIdx.y % heads_y;
    const int hk = DQR ? hy / a.n_rep : hy;
    const int off = nk - nq;

    // streamed range
    int t_lo, n_t;  // first streamed tile, tiles per q head
    if (DQR) {
        // keys [lo_col, hi_col) are visible to some row of the tile (a sliding window drops whole key tiles)
        const int hi_col = min(nk, m0 + kBM + off);
        const int lo_col = a.window < 0 ? 0 : max(0, m0 + off - a.window + 1);
        t_lo = lo_col / kBN;
        n_t = hi_col > lo_col ? (hi_col + kBN - 1) / kBN - t_lo : 0;
    } else {
        // rows [i_lo, i_hi) see some key of the tile: key m is seen by rows m - off .. m - off + window - 1
        const int i_lo = max(0, m0 - off);
        const int i_hi = a.window < 0 ? nq : min(nq, m0 + kBM - 1 - off + a.window);
        t_lo = i_lo / kBN;
        n_t = i_hi > i_lo ? (i_hi + kBN - 1) / kBN - t_lo : 0;
    }
    const int n_iter = DQR ? n_t : n_t * a.n_rep;

    const uint32_t base = smem_u32(smem_raw);
    auto res = [&](int i) -> uint32_t { return base + L::kRes + i * kResBytes; };
    auto str = [&](int s, int i) -> uint32_t { return base + L::kStr + s * L::kStage + i * kStrBytes; };
    auto gt = [&](int i) -> uint32_t { return base + L::kG + i * kGBytes; };
    auto bar = [&](int i) -> uint32_t { return base + L::kBars + 8u * i; };
    const uint32_t tmem_slot = base + L::kTmemSlot;

    if (threadIdx.x == 0) {
        for (int i = 0; i < L::kNumBars; ++i) {
            const bool all_ew = i == L::kSFree || i == L::kGFull || i == L::kKReady;   // arrivals from all 256 element-wise threads
            const bool stat = i >= L::kStatFull && i < L::kStatFull + kStatStages;
            mbar_init(bar(i), all_ew ? 256 : stat ? kStatWriters : 1);
        }
        fence_barrier_init();
    }
    // streamed tile `it` -> stage it % NS (DQR: k, v of key tile it; DKV: q, r, dO of a 64-row tile of one q head)
    auto issue_tile = [&](int it) {
        const int s = it % NS;
        mbar_expect_tx(bar(L::kNFull + s), L::kStageTx);
        if (DQR) {
            const int row0 = bos + (t_lo + it) * kBN;
            const CUtensorMap *maps[2] = {&tm_k, &tm_v};
            for (int i = 0; i < 2; ++i)
                for (int pn = 0; pn < L::kPanels; ++pn)
                    tma_load_4d(str(s, i) + pn * kStrPanel, maps[i], bar(L::kNFull + s), 64 * pn, row0, hk, b);
        } else {
            const int hq = hk * a.n_rep + it / n_t;
            const int row0 = bos + (t_lo + it % n_t) * kBN;
            const CUtensorMap *maps[3] = {&tm_q, &tm_r, &tm_go};
            for (int i = 0; i < 3; ++i)
                for (int pn = 0; pn < L::kPanels; ++pn)
                    tma_load_4d(str(s, i) + pn * kStrPanel, maps[i], bar(L::kNFull + s), 64 * pn, row0, hq, b);
        }
    };
    if (threadIdx.x == 0 && n_iter > 0) {
        // start the first copies right away: their latency overlaps the TMEM allocation and the CTA-wide sync
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_r);
        prefetch_tensormap(&tm_go);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        mbar_expect_tx(bar(L::kXFull), L::kNRes * kResBytes);
        if (DQR) {
            const CUtensorMap *maps[2] = {&tm_q, &tm_r};
            for (int i = 0; i < 2; ++i)
                for (int pn = 0; pn < L::kPanels; ++pn)
                    tma_load_4d(res(i) + pn * kResPanel, maps[i], bar(L::kXFull), 64 * pn, bos + m0, hy, b);
        } else {
            for (int pn = 0; pn < L::kPanels; ++pn)
                tma_load_4d(res(0) + pn * kResPanel, &tm_v, bar(L::kXFull), 64 * pn, bos + m0, hk, b);
        }
        for (int it = 0; it < min(n_iter, NS); ++it) issue_tile(it);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(tmem_base) : "r"(tmem_slot));
    const uint32_t tAcc0 = tmem_base, tAcc1 = tmem_base + 128, tS = tmem_base + 256;  // S1, S2, A at tS + 0 / 64 / 128
    const uint32_t tK = tmem_base + 448;                                              // DKV: the k tile as an A operand

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // the resident tiles and the first NS streamed tiles were started before the CTA-wide sync
        if (lane == 0 && n_iter > 0) {
            int issued = min(n_iter, NS);
            bool ok = true;
            for (int it = 0; it < n_iter; ++it) {
                if (it >= NS) {
                    ok = mbar_wait(bar(L::kNEmpty + it % NS), ((it / NS) & 1) ^ 1, err, 1);
                    if (!ok) break;
                    issue_tile(it);
                    issued = it + 1;
                }
            }
            if (!ok) {
                for (int it = max(0, issued - NS); it < issued; ++it) mbar_wait_quiet(bar(L::kNFull + it % NS), (it / NS) & 1);
                mbar_wait_quiet(bar(L::kXFull), 0);
            }
        }
    } else if (warp == 1 || warp == 10) {
        // ------------------------------------------------------------------ MMA issuers
        // Two threads in two warps issue the MMAs (warp 1: the score products, warp 10: the output
        // products): one thread's instruction stream, not the tensor pipe, is what bounds a single issuer.
        // The whole warp runs the loop (so that its values stay warp-uniform); one elected lane issues.
        if (n_iter > 0) {
            // A single thread issues every MMA, so this path is kept to a few instructions per MMA:
            // descriptor low words are "base + immediate", high words and flags are compile-time constants.
            constexpr uint32_t idesc_s = umma_idesc(Fmt<T>::kUmma, 0, 0, kBM, kBN);
            constexpr uint32_t idesc_o = umma_idesc(Fmt<T>::kUmma, 0, 1, kBM, D);
            constexpr uint32_t hi = umma_desc_hi(1024);
            // DQR: q, r, dO.  DKV: only v (index 0) is in shared memory, k is in TMEM.
            const uint32_t res_lo0 = umma_desc_lo(res(0), 16), res_lo1 = umma_desc_lo(res(DQR ? 1 : 0), 16),
                           res_lo2 = umma_desc_lo(res(0), 16);   // DKV: v; DQR takes dO from tensor memory instead
            const uint32_t g_lo0 = umma_desc_lo(gt(0), 16), g_lo1 = umma_desc_lo(gt(1), 16), g_lo2 = umma_desc_lo(gt(DQR ? 1 : 2), 16);
            const uint32_t strk_lo0 = umma_desc_lo(str(0, 0), 16);          // streamed tiles as K-major B (scores)
            const uint32_t strm_lo0 = umma_desc_lo(str(0, 0), kStrPanel);   // streamed tiles as MN-major B (outputs)
            // scores: S1, S2, A into tS + 0 / 64 / 128
            auto issue_scores = [&](int s) {
                const uint32_t b0 = strk_lo0 + s * (L::kStage >> 4);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t aoff = ((ks >> 2) * kResPanel + (ks & 3) * 32) >> 4;
                    const uint32_t boff = ((ks >> 2) * kStrPanel + (ks & 3) * 32) >> 4;
                    // DQR: (Q, K) (R, K) (dO, V);  DKV: (K, Q) (K, R) (V, dO)
                    const uint32_t a1 = res_lo0 + aoff, a2 = (DQR ? res_lo1 : res_lo0) + aoff, a3 = res_lo2 + aoff;
                    const uint32_t b1 = b0 + boff, b2 = b0 + (DQR ? 0 : (kStrBytes >> 4)) + boff,
                                   b3 = b0 + ((DQR ? 1 : 2) * (kStrBytes >> 4)) + boff;
                    if (DQR) {
                        if (ks == 0) {
                            umma_ss_lean<false>(tS, a1, hi, b1, hi, idesc_s);
                            umma_ss_lean<false>(tS + 64, a2, hi, b2, hi, idesc_s);
                            umma_ts_lean<false>(tS + 128, tK + ks * 8, b3, hi, idesc_s);   // dO from tensor memory
                        } else {
                            umma_ss_lean<true>(tS, a1, hi, b1, hi, idesc_s);
                            umma_ss_lean<true>(tS + 64, a2, hi, b2, hi, idesc_s);
                            umma_ts_lean<true>(tS + 128, tK + ks * 8, b3, hi, idesc_s);
                        }
                    } else {   // k from tensor memory: 16 channels = 8 columns per step
                        if (ks == 0) {
                            umma_ts_lean<false>(tS, tK + ks * 8, b1, hi, idesc_s);
                            umma_ts_lean<false>(tS + 64, tK + ks * 8, b2, hi, idesc_s);
                            umma_ss_lean<false>(tS + 128, a3, hi, b3, hi, idesc_s);
                        } else {
                            umma_ts_lean<true>(tS, tK + ks * 8, b1, hi, idesc_s);
                            umma_ts_lean<true>(tS + 64, tK + ks * 8, b2, hi, idesc_s);
                            umma_ss_lean<true>(tS + 128, a3, hi, b3, hi, idesc_s);
                        }
                    }
                }
                umma_commit(bar(L::kSFull));
            };
            // outputs: A = G tile (K-major, 64 wide), B = streamed tile as MN-major [64 rows][128 channels]
            //   DQR: acc0 += G0 K, acc1 += G1 K;   DKV: acc0 += G0 Q + G1 R, acc1 += G2 dO
            auto issue_out = [&](int s, bool first) {
                const uint32_t b0 = strm_lo0 + s * (L::kStage >> 4);
                const uint32_t bq = b0, br = b0 + (DQR ? 0 : (kStrBytes >> 4)), bg = b0 + 2 * (kStrBytes >> 4);
                if (first) {
                    umma_ss_lean<false>(tAcc0, g_lo0, hi, bq, hi, idesc_o);
                    umma_ss_lean<false>(tAcc1, DQR ? g_lo1 : g_lo2, hi, DQR ? br : bg, hi, idesc_o);
                } else {
                    umma_ss_lean<true>(tAcc0, g_lo0, hi, bq, hi, idesc_o);
                    umma_ss_lean<true>(tAcc1, DQR ? g_lo1 : g_lo2, hi, DQR ? br : bg, hi, idesc_o);
                }
                if (!DQR) umma_ss_lean<true>(tAcc0, g_lo1, hi, br, hi, idesc_o);
#pragma unroll
                for (int kk = 1; kk < kBN / 16; ++kk) {
                    const uint32_t ao = kk * (32 >> 4), bo = kk * (2048 >> 4);
                    umma_ss_lean<true>(tAcc0, g_lo0 + ao, hi, bq + bo, hi, idesc_o);
                    umma_ss_lean<true>(tAcc1, (DQR ? g_lo1 : g_lo2) + ao, hi, (DQR ? br : bg) + bo, hi, idesc_o);
                    if (!DQR) umma_ss_lean<true>(tAcc0, g_lo1 + ao, hi, br + bo, hi, idesc_o);
                }
            };
            if (warp == 1) {
                bool ok = mbar_wait(bar(L::kXFull), 0, err, 4) && mbar_wait(bar(L::kKReady), 0, err, 14);
                ok = __all_sync(0xffffffffu, ok);
                int s = 0;
                uint32_t ph = 0;
                for (int it = 0; it < n_iter && ok; ++it) {
                    ok = mbar_wait(bar(L::kNFull + s), ph, err, 6);
                    // the score columns are free once the element-wise warps have read tile it - 1
                    if (ok && it > 0) ok = mbar_wait(bar(L::kSFree), (it - 1) & 1, err, 7);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one_sync()) issue_scores(s);
                    __syncwarp();
                    if (++s == NS) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            } else {
                bool ok = true;
                int s = 0;
                for (int it = 0; it < n_iter && ok; ++it) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kGFull), it & 1, err, 8));
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one_sync()) {
                        issue_out(s, it == 0);
                        umma_commit(bar(L::kGFree));
                        umma_commit(bar(L::kNEmpty + s));
                    }
                    __syncwarp();
                    if (++s == NS) s = 0;
                }
                if (ok && elect_one_sync()) umma_commit(bar(L::kAccDone));
            }
        }
    } else {
        // ------------------------------------------------------------------ element-wise + epilogue
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int ml = quarter * 32 + lane;                 // lane of the M tile: query row (DQR) / key (DKV)
        const int mg = m0 + ml;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const int col0 = half * 32;
        bool ok = true;

        // With mL = m + log2(d1), c1 = 1 + bart, ct = b - t:
        //   p = 2^(S1*c2 - mL), un = S2 - c1, dn = b - A   =>   W = -p un, gu = p dn, gl = (p un) dn + p ct
        // DQR: the constants of this thread's row
        float r_ml = INFINITY, r_c1 = 0.f, r_ct = 0.f, r_b = 0.f;
        if (DQR && mg < nq) {
            const float4 hi4 = *reinterpret_cast<const float4 *>(
                a.cst + ((static_cast<int64_t>(b) * a.heads_q + hy) * n_tok + bos + mg) * 4);   // b, mL, 1 + bart, (b - t) * scale
            r_b = hi4.x;
            r_ml = hi4.y;
            r_c1 = hi4.z;
            r_ct = hi4.w / a.scale;
        }
        const float2 c2v = make_float2(a.c2, a.c2);
        {
            // The tile of the M side that is the A operand of score products and fits the 64 spare TMEM
            // columns -- DKV: k (S1^T, S2^T), DQR: dO (A) -- goes there instead of shared memory, where MMA
            // operand reads are the scarce resource: this thread's half (D / 2 channels) of row mg, two
            // 16-bit channels per column.
            uint32_t kw[D / 4];
            const T *krow = DQR ? static_cast<const T *>(a.go) + b * a.q_sb + hy * a.q_sh + static_cast<int64_t>(bos + mg) * a.q_st + half * (D / 2)
                                : static_cast<const T *>(a.k) + b * a.kv_sb + hk * a.kv_sh + static_cast<int64_t>(bos + mg) * a.kv_st + half * (D / 2);
#pragma unroll
            for (int i = 0; i < D / 16; ++i) {
                uint4 x = make_uint4(0u, 0u, 0u, 0u);
                if (mg < (DQR ? nq : nk)) x = *reinterpret_cast<const uint4 *>(krow + 8 * i);
                kw[4 * i] = x.x; kw[4 * i + 1] = x.y; kw[4 * i + 2] = x.z; kw[4 * i + 3] = x.w;
            }
            if constexpr (D == 128) tmem_st32(tK + lane_base + half * 32, kw);
            else tmem_st16(tK + lane_base + half * 16, kw);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(L::kKReady));
        }

        // DKV: the per-row statistics of a streamed tile are per-COLUMN constants here.  The first 64
        // element-wise threads fetch one row each ({b, mL, 1 + bart, (b - t) * scale}, 16 bytes) a tile
        // ahead and lay them out in shared memory as four planes of 64 floats (with mL and 1 + bart
        // negated), so that every thread reads the constants of adjacent columns as aligned pairs for
        // the packed two-wide arithmetic.  Two buffers: tile it uses buffer it & 1.
        const int wid = static_cast<int>(threadIdx.x) - 64;
        const bool stat_writer = !DQR && wid < kStatWriters;
        auto stat_fetch = [&](int it) -> float4 {
            if (it >= n_iter) return make_float4(0.f, 0.f, 0.f, 0.f);
            const int hq = hk * a.n_rep + it / n_t;
            const int row0 = bos + (t_lo + it % n_t) * kBN;
            return __ldg(reinterpret_cast<const float4 *>(a.cst + ((static_cast<int64_t>(b) * a.heads_q + hq) * n_tok + row0 + wid) * 4));
        };
        auto stat_publish = [&](int it, const float4 &v) {
            float *dst = reinterpret_cast<float *>(smem_raw + L::kStats + (it % kStatStages) * kStatBytes);
            dst[wid] = -v.y;
            dst[kBN + wid] = -v.z;
            dst[2 * kBN + wid] = v.x;
            dst[3 * kBN + wid] = v.w;
            mbar_arrive(bar(L::kStatFull + it % kStatStages));
        };
        float4 stat_next = make_float4(0.f, 0.f, 0.f, 0.f);
        if (stat_writer && n_iter > 0) {
            stat_publish(0, stat_fetch(0));
            stat_next = stat_fetch(1);
        }

        for (int it = 0; it < n_iter; ++it) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kSFull), it & 1, err, 9));
            if (!ok) break;
            tc_fence_after();
            uint32_t x1[32], x2[32], x3[32];
            tmem_ld32(tS + lane_base + col0, x1);
            tmem_ld32(tS + 64 + lane_base + col0, x2);
            tmem_ld32(tS + 128 + lane_base + col0, x3);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(bar(L::kSFree));

            const int tile0 = (t_lo + (DQR ? it : it % n_t)) * kBN;   // first streamed index of the tile
            const int n0 = tile0 + col0;                              // ... of this thread's columns
            // DQR: columns are keys n0 + c, visible iff n0 + c <= lim_hi.   DKV: columns are rows, visible iff lim_lo <= n0 + c <= lim_hi
            const int win = a.window;
            const int lim_lo = DQR ? (win < 0 ? INT_MIN : mg + off - win + 1) : max(mg - off, 0);
            const int lim_hi = DQR ? (mg < nq ? min(mg + off, nk - 1) : -1)
                                   : (mg < nk ? (win < 0 ? nq - 1 : min(nq - 1, mg - off + win - 1)) : -1);
            // tile-uniform: every element of the tile is visible
            const bool full = DQR ? (tile0 + kBN - 1 <= m0 + off && tile0 + kBN <= nk && m0 + kBM <= nq &&
                                     (win < 0 || tile0 >= m0 + kBM + off - win))
                                  : (tile0 >= m0 + kBM - 1 - off && tile0 + kBN <= nq && m0 + kBM <= nk &&
                                     (win < 0 || tile0 + kBN - 1 <= m0 - off + win - 1));
            const int ss = it % kStatStages;
            const float *stats = reinterpret_cast<const float *>(smem_raw + L::kStats + ss * kStatBytes);
            if (!DQR) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kStatFull + ss), (it / kStatStages) & 1, err, 15));
                if (!ok) break;
            }
            uint32_t g0[16], g1[16], g2[16];
            // one pair of adjacent columns: constants nml = -mL, nc1 = -(1 + bart), bb = b, ct = b - t (DKV: times scale)
            auto pair = [&](int c, const float2 &nml, const float2 &nc1, const float2 &bb, const float2 &ct) {
                const float2 s1 = make_float2(__uint_as_float(x1[c]), __uint_as_float(x1[c + 1]));
                const float2 s2 = make_float2(__uint_as_float(x2[c]), __uint_as_float(x2[c + 1]));
                const float2 av = make_float2(__uint_as_float(x3[c]), __uint_as_float(x3[c + 1]));
                const float2 arg = __ffma2_rn(s1, c2v, nml);
                const float2 p = make_float2(fast_exp2(arg.x), fast_exp2(arg.y));
                const float2 un = __fadd2_rn(s2, nc1);
                const float2 dn = __ffma2_rn(av, make_float2(-1.f, -1.f), bb);
                const float2 pc = __fmul2_rn(p, ct);
                const float2 wn = __fmul2_rn(p, un);                      // -W
                float2 gu = __fmul2_rn(p, dn);
                // DKV carries qk_scale on gl: (wn dn) * scale + p ct scale
                float2 gl = __ffma2_rn(wn, DQR ? dn : __fmul2_rn(dn, make_float2(a.scale, a.scale)), pc);
                float2 gw = make_float2(-wn.x, -wn.y);
                if (!full) {
                    const bool v0 = n0 + c >= lim_lo && n0 + c <= lim_hi, v1 = n0 + c + 1 >= lim_lo && n0 + c + 1 <= lim_hi;
                    gl = make_float2(v0 ? gl.x : 0.f, v1 ? gl.y : 0.f);
                    gu = make_float2(v0 ? gu.x : 0.f, v1 ? gu.y : 0.f);
                    gw = make_float2(v0 ? gw.x : 0.f, v1 ? gw.y : 0.f);
                }
                g0[c >> 1] = Elem<T>::pack(gl.x, gl.y);
                g1[c >> 1] = Elem<T>::pack(gu.x, gu.y);
                if (!DQR) g2[c >> 1] = Elem<T>::pack(gw.x, gw.y);
            };
            if (DQR) {
                const float2 nml = make_float2(-r_ml, -r_ml), nc1 = make_float2(-r_c1, -r_c1), bb = make_float2(r_b, r_b),
                             ct = make_float2(r_ct, r_ct);
#pragma unroll
                for (int c = 0; c < 32; c += 2) pair(c, nml, nc1, bb, ct);
            } else {
                const float *pl = stats + col0;
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    const float4 nml = *reinterpret_cast<const float4 *>(pl + c);
                    const float4 nc1 = *reinterpret_cast<const float4 *>(pl + kBN + c);
                    const float4 bb = *reinterpret_cast<const float4 *>(pl + 2 * kBN + c);
                    const float4 ct = *reinterpret_cast<const float4 *>(pl + 3 * kBN + c);
                    pair(c, make_float2(nml.x, nml.y), make_float2(nc1.x, nc1.y), make_float2(bb.x, bb.y), make_float2(ct.x, ct.y));
                    pair(c + 2, make_float2(nml.z, nml.w), make_float2(nc1.z, nc1.w), make_float2(bb.z, bb.w), make_float2(ct.z, ct.w));
                }
            }
            if (it > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kGFree), (it - 1) & 1, err, 10));
                if (!ok) break;
            }
            // Every thread has handed over tile it - 1 (the output products that just completed needed all
            // of its G rows), so nobody reads the statistics buffer of tile it - 1 any more: refill it.
            if (stat_writer && it + 1 < n_iter) {
                stat_publish(it + 1, stat_next);
                stat_next = stat_fetch(it + 2);
            }
            // row ml of each G tile: 128 bytes, 16-byte chunk i stored at position i ^ (ml & 7)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t o = static_cast<uint32_t>(ml) * 128u + static_cast<uint32_t>(((half * 4 + i) ^ (ml & 7)) * 16);
                st_shared_v4(gt(0) + o, g0[4 * i], g0[4 * i + 1], g0[4 * i + 2], g0[4 * i + 3]);
                st_shared_v4(gt(1) + o, g1[4 * i], g1[4 * i + 1], g1[4 * i + 2], g1[4 * i + 3]);
                if (!DQR) st_shared_v4(gt(2) + o, g2[4 * i], g2[4 * i + 1], g2[4 * i + 2], g2[4 * i + 3]);
            }
            fence_proxy_async();
            mbar_arrive(bar(L::kGFull));
        }

        // epilogue: warps 2-5 write acc0 (dQ | dK), warps 6-9 write acc1 (dR | dV)
        if (ok && n_iter > 0) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kAccDone), 0, err, 11));
            tc_fence_after();
        }
        if (ok) {
            // The accumulators are read in the fragment arrangement (a row is spread over the four lanes
            // of a quad); a 4 x 4 word transpose inside the quad gives every thread 16 contiguous bytes,
            // so a warp store covers 64 contiguous bytes of 8 rows.
            const float mul = (DQR && half == 0) ? a.scale : 1.f;
            const int limit = DQR ? nq : nk;
            const int g = lane >> 2, t = lane & 3;
            const uint32_t acc = half == 0 ? tAcc0 : tAcc1;
            T *dst0;
            int64_t row_stride;
            if (DQR) {
                dst0 = static_cast<T *>(half == 0 ? a.dq : a.dr) + b * a.q_sb + hy * a.q_sh;
                row_stride = a.q_st;
            } else {
                dst0 = static_cast<T *>(half == 0 ? a.dk : a.dv) + b * a.kv_sb + hy * a.kv_sh;
                row_stride = a.kv_st;
            }
#pragma unroll 1
            for (int rh = 0; rh < 2; ++rh) {
                const int rl = quarter * 32 + rh * 16 + g;     // local rows of this thread: rl and rl + 8
#pragma unroll
                for (int cc = 0; cc < D / 64; ++cc) {
                    uint32_t x[32];
                    if (n_iter > 0) {
                        tmem_ld_16x256b_x8(acc + (static_cast<uint32_t>(quarter * 32 + rh * 16) << 16) + 64 * cc, x);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) x[i] = 0u;
                    }
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                        for (int grp = 0; grp < 2; ++grp) {
                            uint32_t w[4];
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk) {
                                const int i = 4 * (4 * grp + kk) + 2 * hh;
                                w[kk] = Elem<T>::pack(__uint_as_float(x[i]) * mul, __uint_as_float(x[i + 1]) * mul);
                            }
                            quad_transpose(w, t);
                            const int row = m0 + rl + 8 * hh;
                            if (row < limit)
                                *reinterpret_cast<uint4 *>(dst0 + static_cast<int64_t>(bos + row) * row_stride + 64 * cc + 32 * grp + 8 * t) =
                                    make_uint4(w[0], w[1], w[2], w[3]);
                        }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------- //
// host side
// ------------------------------------------------------------------------- //
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                              const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

bool make_map(CUtensorMap *map, CUtensorMapDataType dt, const void *ptr, int head_dim, int tokens, int heads, int batch,
              int64_t st, int64_t sh, int64_t sb, int rows) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(heads),
                                static_cast<cuuint64_t>(batch)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(st) * 2, static_cast<cuuint64_t>(sh) * 2,
                                   static_cast<cuuint64_t>(sb) * 2};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(rows), 1, 1};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    return fn(map, dt, 4, const_cast<void *>(ptr), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int D, int MODE>
int launch_mode(const TrainArgs &a, int n_tok, int *err, cudaStream_t stream) {
    constexpr int NS = (D == 128 && MODE == kModeDKV) ? 3 : 4;   // dk/dv at D = 128: as many stages as the 227 KB of shared memory allow
    using L = Smem<D, MODE, NS>;
    constexpr bool DQR = MODE == kModeDQR;
    const int q_rows = DQR ? kBM : kBN, kv_rows = DQR ? kBN : kBM;
    CUtensorMap tq, tr, tg, tk, tv;
    const CUtensorMapDataType dt = Fmt<T>::kTma;
    if (!make_map(&tq, dt, a.q, D, a.len_q, a.heads_q, a.batch, a.q_st, a.q_sh, a.q_sb, q_rows) ||
        !make_map(&tr, dt, a.r, D, a.len_q, a.heads_q, a.batch, a.q_st, a.q_sh, a.q_sb, q_rows) ||
        !make_map(&tg, dt, a.go, D, a.len_q, a.heads_q, a.batch, a.q_st, a.q_sh, a.q_sb, q_rows) ||
        !make_map(&tk, dt, a.k, D, a.len_k, a.heads_kv, a.batch, a.kv_st, a.kv_sh, a.kv_sb, kv_rows) ||
        !make_map(&tv, dt, a.v, D, a.len_k, a.heads_kv, a.batch, a.kv_st, a.kv_sh, a.kv_sb, kv_rows))
        return PLX_ERR_LAUNCH;
    auto kern = bwd_sm100_kernel<T, D, MODE, NS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(L::kBytes)) != cudaSuccess)
        return PLX_ERR_LAUNCH;
    const int len = DQR ? a.len_q : a.len_k;
    const int tiles = a.cu ? (len + kBM - 1) / kBM + a.n_seqs : (len + kBM - 1) / kBM;
    dim3 grid(tiles, a.batch * (DQR ? a.heads_q : a.heads_kv));
    kern<<<grid, 352, L::kBytes, stream>>>(a, n_tok, tq, tr, tg, tk, tv, err);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? PLX_OK : PLX_ERR_LAUNCH;
}

}  // namespace

bool train_bwd_sm100_supported(const TrainArgs &a, int head_dim) {
    if ((head_dim != 64 && head_dim != 128) || a.window == 0 || !(a.c2 > 0.f)) return false;
    const char *env = std::getenv("PLX_BWD_KERNEL");
    if (env && env[0] == 'm') return false;  // "mma": force the warp-level kernels
    return encode_fn() != nullptr;
}

int launch_train_bwd_sm100(const TrainArgs &a, int dtype, int head_dim, int stage, cudaStream_t stream) {
    int *err = sm100_error_ptr();
    if (!err) return PLX_ERR_LAUNCH;
    const int n_tok = a.len_q;
    const bool dqr = stage == PLX_BWD_DQR;
    if (dtype == PLX_BF16) {
        if (head_dim == 64)
            return dqr ? launch_mode<__nv_bfloat16, 64, kModeDQR>(a, n_tok, err, stream)
                       : launch_mode<__nv_bfloat16, 64, kModeDKV>(a, n_tok, err, stream);
        return dqr ? launch_mode<__nv_bfloat16, 128, kModeDQR>(a, n_tok, err, stream)
                   : launch_mode<__nv_bfloat16, 128, kModeDKV>(a, n_tok, err, stream);
    }
    if (dtype == PLX_FP16) {
        if (head_dim == 64)
            return dqr ? launch_mode<__half, 64, kModeDQR>(a, n_tok, err, stream)
                       : launch_mode<__half, 64, kModeDKV>(a, n_tok, err, stream);
        return dqr ? launch_mode<__half, 128, kModeDQR>(a, n_tok, err, stream)
                   : launch_mode<__half, 128, kModeDKV>(a, n_tok, err, stream);
    }
    return PLX_ERR_UNSUPPORTED;
}

}  // namespace plx
