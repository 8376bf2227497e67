// Parallax training backward on the Blackwell tensor cores (tcgen05.mma, TMEM
// accumulators, TMA-staged tiles): one kernel template, two modes.
//
//   DQR: CTA = 128 query rows of one (batch, q head); streams key tiles of 64.
//        S1 = Q K^T, S2 = R K^T, A = dO V^T  ->  gl, gu  ->  dQ += gl K, dR += gu K
//   DKV: CTA = 128 keys of one (batch, kv head); streams 64-row tiles of q, r, dO
//        (and their row statistics) of every q head of the group.
//        S1^T = K Q^T, S2^T = K R^T, A^T = V dO^T  ->  gl^T, gu^T, W^T
//        ->  dK += gl^T Q + gu^T R, dV += W^T dO   (the tile holds -W^T, the accumulator -dV until it is written)
//
// Formulas (parallax/triton/parallax_train.py:561-573 and :765-792 of the reference):
//   w = 2^(S1*c2 - m), p = w / d1, delta = A - b, cs = bart - S2
//   gl = p (A - t + cs delta), gu = -p delta, W = p (1 + cs); dQ and the gl part of dK carry qk_scale.
// Evaluated as W = p (1 + bart - S2), gl = W delta + p (b - t) with 1/d1 folded into the exponent.
//
// The kernel is persistent: at most one CTA per SM, each walking its share of the work items.
// Pipeline per CTA (12 warps):
//   warp 0      TMA producer (resident tiles once per item, streamed tiles through an NS-deep ring)
//   warp 1      TMEM allocation + the lane that issues the score products
//   warp 2      the lane that issues the output products          (warp 3 idles)
//   warps 4-11  element-wise: warp 4 + w works on TMEM lane quarter w % 4 (128 rows of the M tile, one
//               per thread) and column group w / 4 (32 of the 64 streamed columns; with sixteen such
//               warps, a build option, 16).  A thread reads its columns of the three score tiles from
//               TMEM, releases them at once (so the next tile's scores are computed while it works),
//               writes gl / gu / -W as 16-bit values into shared memory in the 128-byte-swizzled K-major
//               layout, and the MMA lane consumes them as the A operand of the output products.
//               The arithmetic of a tile is ONE basic block (tiles that need a mask run a second copy
//               of the loop): measured with every MMA removed, the element-wise chain (TMEM load ->
//               arithmetic -> shared-memory store -> hand-over), not the tensor pipe, sets the pace,
//               and the independent column pairs of a thread must be free to interleave.
//
// TMEM columns: acc0 [0,128) (dQ | dK), acc1 [128,256) (dR | dV), S1 [256,320), S2 [320,384), A [384,448),
// and at [448,512) the M-side tile that is the A operand of score products: k in DKV mode (S1^T, S2^T), dO in DQR mode (A).
#include <cuda.h>

#include <climits>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "plx_common.cuh"
#include "plx_launch.h"
#include "plx_sm100.cuh"
#include "plx_tma_host.h"

namespace plx {

using namespace sm100;

namespace {

constexpr int kModeDQR = 0, kModeDKV = 1;
#ifndef PLX_BWD_EW_WARPS
#define PLX_BWD_EW_WARPS 8    // element-wise warps per CTA (8 or 16)
#endif
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
    // per streamed tile: NFull / NEmpty (ring), SFull / SFree (score columns), GFull / GFree (G tiles), StatFull;
    // per work item: XFull / XEmpty (resident tiles), KReady (M-side tile in tensor memory), AccDone / AccFree
    static constexpr int kXFull = 0, kXEmpty = 1, kNFull = 2, kNEmpty = 2 + NS, kSFull = 2 + 2 * NS, kSFree = kSFull + 1,
                         kGFull = kSFull + 2, kGFree = kSFull + 3, kAccDone = kSFull + 4, kAccFree = kSFull + 5,
                         kKReady = kSFull + 6, kStatFull = kSFull + 7, kNumBars = kStatFull + kStatStages;
    static constexpr uint32_t kTmemSlot = kBars + 8 * kNumBars;
    static constexpr uint32_t kAbort = kTmemSlot + 8;
    static constexpr uint32_t kBytes = kTmemSlot + 16;   // the dynamic shared memory must start 1024-byte aligned
    static constexpr uint32_t kStageTx = kStage;
};

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// One unit of work: 128 query rows of one (batch, q head) (DQR) or 128 keys of one (batch, kv head) (DKV),
// and the range of 64-wide tiles of the other side that it streams.
struct Item {
    int bos, nq, nk, m0, b, hy, hk, off, t_lo, n_t, n_iter;   // streamed tiles t_lo .. t_lo + n_t - 1, per q head
    bool valid;
};

// Work item `idx` of the launch.  Items are (batch, head)-major, so that CTAs running at the same time
// share their streamed tiles in L2; inside a (batch, head) the 128-wide tiles alternate last, first,
// last - 1, second, ...: under the causal mask any two neighbours add up to the same work.
template <bool DQR>
__device__ __forceinline__ Item get_item(const TrainArgs &a, int idx, int n_mt) {
    Item it;
    const int bh = idx / n_mt, k = idx % n_mt;
    const int tile_id = (k & 1) ? (k >> 1) : n_mt - 1 - (k >> 1);
    Seq s;
    int tis = 0;
    it.valid = locate_tile(a, tile_id, kBM, s, tis);
    it.bos = s.bos;
    it.nq = s.nq;
    it.nk = s.nk;
    it.m0 = tis * kBM;
    if (it.valid && it.m0 >= (DQR ? it.nq : it.nk)) it.valid = false;
    const int heads_y = DQR ? a.heads_q : a.heads_kv;
    it.b = bh / heads_y;
    it.hy = bh % heads_y;
    it.hk = DQR ? it.hy / a.n_rep : it.hy;
    it.off = it.nk - it.nq;
    int n_t = 0;
    if (DQR) {
        // keys [lo_col, hi_col) are visible to some row of the tile (a sliding window drops whole key tiles)
        const int hi_col = min(it.nk, it.m0 + kBM + it.off);
        const int lo_col = a.window < 0 ? 0 : max(0, it.m0 + it.off - a.window + 1);
        it.t_lo = lo_col / kBN;
        n_t = hi_col > lo_col ? (hi_col + kBN - 1) / kBN - it.t_lo : 0;
    } else {
        // rows [i_lo, i_hi) see some key of the tile: key m is seen by rows m - off .. m - off + window - 1
        const int i_lo = max(0, it.m0 - it.off);
        const int i_hi = a.window < 0 ? it.nq : min(it.nq, it.m0 + kBM - 1 - it.off + a.window);
        it.t_lo = i_lo / kBN;
        n_t = i_hi > i_lo ? (i_hi + kBN - 1) / kBN - it.t_lo : 0;
    }
    it.n_t = it.valid ? n_t : 0;
    it.n_iter = DQR ? it.n_t : it.n_t * a.n_rep;
    return it;
}

// n-th item of this CTA: CTAs take chunks of 2^chunk_shift neighbouring items, round robin.
__device__ __forceinline__ int item_index(int n, int chunk_shift) {
    return ((blockIdx.x + gridDim.x * (n >> chunk_shift)) << chunk_shift) + (n & ((1 << chunk_shift) - 1));
}

// Persistent kernel: gridDim.x CTAs (at most one per SM) walk the item list.  The streamed-tile pipeline
// (TMA ring -> score products -> element-wise -> G tiles -> output products) runs as ONE sequence of
// tiles across items; what an item adds is its resident tiles, its M-side tile in tensor memory and its
// accumulators, and the hand-overs for those are arranged so that the loads, the tensor-memory tile and
// the first score products of the next item are under way while the element-wise warps write out the
// accumulators of the current one.  TMEM allocation, barrier set-up and launch latency are paid once.
template <typename T, int D, int MODE, int NS, int EW>
__global__ void __launch_bounds__((4 + EW) * 32, 1)
bwd_sm100_kernel(const TrainArgs a, int n_tok, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_r, const __grid_constant__ CUtensorMap tm_go,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const ErrSink sink,
                 int n_mt, int n_items, int chunk_shift) {
    using L = Smem<D, MODE, NS>;
    constexpr bool DQR = MODE == kModeDQR;
    constexpr uint32_t kResBytes = L::kResBytes, kStrBytes = L::kStrBytes;
    constexpr int CG = EW / 4;        // element-wise warps per TMEM lane quarter = column groups of a streamed tile
    constexpr int CPT = kBN / CG;     // columns of a streamed tile per element-wise thread
    constexpr int kEwThreads = EW * 32;
    static_assert(EW == 8 || EW == 16, "two or four element-wise warps per lane quarter");
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t base = smem_u32(smem_raw);
    auto res = [&](int i) -> uint32_t { return base + L::kRes + i * kResBytes; };
    auto str = [&](int s, int i) -> uint32_t { return base + L::kStr + s * L::kStage + i * kStrBytes; };
    auto gt = [&](int i) -> uint32_t { return base + L::kG + i * kGBytes; };
    auto bar = [&](int i) -> uint32_t { return base + L::kBars + 8u * i; };
    const uint32_t tmem_slot = base + L::kTmemSlot;
    const WaitCtx err{sink, base + L::kAbort};

    if (threadIdx.x == 0) {
        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(err.abort_flag), "r"(0u) : "memory");
        for (int i = 0; i < L::kNumBars; ++i) {
            // arrivals from all element-wise threads
            const bool all_ew = i == L::kSFree || i == L::kGFull || i == L::kKReady || i == L::kAccFree;
            const bool stat = i >= L::kStatFull && i < L::kStatFull + kStatStages;
            mbar_init(bar(i), all_ew ? kEwThreads : stat ? kStatWriters : 1);
        }
        fence_barrier_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_r);
        prefetch_tensormap(&tm_go);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        if ((base & 1023u) != 0) cta_abort(err, (12 << 8) | kErrWaitTimeout);   // the swizzled tiles need a 1024-byte aligned base
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
    const uint32_t tK = tmem_base + 448;                                              // the M-side tile as an A operand
    const bool misaligned = cta_aborted(err);

    if (misaligned) {
        // nothing was started: fall through to the common exit
    } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int g = 0, n = 0, s = 0;      // streamed tiles and items so far, ring stage of tile g
            uint32_t ph = 0;              // phase of the ring
            bool ok = true;
            int x_issued = 0;             // resident-tile loads started
            for (int i = 0; ok; ++i) {
                const int idx = item_index(i, chunk_shift);
                if (idx >= n_items) break;
                const Item it = get_item<DQR>(a, idx, n_mt);
                if (it.n_iter == 0) continue;
                // the resident tiles of the previous item are free once its last score product has completed
                if (n > 0) {
                    ok = mbar_wait(bar(L::kXEmpty), (n - 1) & 1, err, 1);
                    if (!ok) break;
                }
                mbar_expect_tx(bar(L::kXFull), L::kNRes * kResBytes);
                ++x_issued;
                if (DQR) {
                    const CUtensorMap *maps[2] = {&tm_q, &tm_r};
                    for (int j = 0; j < 2; ++j)
                        for (int pn = 0; pn < L::kPanels; ++pn)
                            tma_load_4d(res(j) + pn * kResPanel, maps[j], bar(L::kXFull), 64 * pn, it.bos + it.m0, it.hy, it.b);
                } else {
                    for (int pn = 0; pn < L::kPanels; ++pn)
                        tma_load_4d(res(0) + pn * kResPanel, &tm_v, bar(L::kXFull), 64 * pn, it.bos + it.m0, it.hk, it.b);
                }
                // streamed tile t of the item -> stage s (DQR: k, v of key tile t; DKV: q, r, dO of a 64-row tile of one q head)
                int hq = it.hk * a.n_rep, tt = 0;
                for (int t = 0; t < it.n_iter; ++t, ++g) {
                    if (g >= NS) {
                        ok = mbar_wait(bar(L::kNEmpty + s), ph ^ 1, err, 2);
                        if (!ok) break;
                    }
                    mbar_expect_tx(bar(L::kNFull + s), L::kStageTx);
                    const int row0 = it.bos + (it.t_lo + tt) * kBN;
                    if (DQR) {
                        const CUtensorMap *maps[2] = {&tm_k, &tm_v};
                        for (int j = 0; j < 2; ++j)
                            for (int pn = 0; pn < L::kPanels; ++pn)
                                tma_load_4d(str(s, j) + pn * kStrPanel, maps[j], bar(L::kNFull + s), 64 * pn, row0, it.hk, it.b);
                    } else {
                        const CUtensorMap *maps[3] = {&tm_q, &tm_r, &tm_go};
                        for (int j = 0; j < 3; ++j)
                            for (int pn = 0; pn < L::kPanels; ++pn)
                                tma_load_4d(str(s, j) + pn * kStrPanel, maps[j], bar(L::kNFull + s), 64 * pn, row0, hq, it.b);
                    }
                    if (++tt == it.n_t) {
                        tt = 0;
                        ++hq;
                    }
                    if (++s == NS) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                ++n;
            }
            if (!ok) {
                // unwinding: let the copies already in flight land before the CTA (and its shared memory) goes away
                for (int j = 0; j < min(g, NS); ++j) {
                    if (--s < 0) {
                        s = NS - 1;
                        ph ^= 1;
                    }
                    mbar_wait_quiet(bar(L::kNFull + s), ph);
                }
                if (x_issued > 0) mbar_wait_quiet(bar(L::kXFull), (x_issued - 1) & 1);
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------------------------------------------ MMA issuers
        // Two threads in two warps issue the MMAs (warp 1: the score products, warp 2: the output
        // products): one thread's instruction stream, not the tensor pipe, is what bounds a single issuer.
        // The whole warp runs the loop (so that its values stay warp-uniform); one elected lane issues.
        // This path is kept to a few instructions per MMA: descriptor low words are "base + immediate",
        // high words and flags are compile-time constants.
        constexpr uint32_t idesc_s = umma_idesc(Fmt<T>::kUmma, 0, 0, kBM, kBN);
        constexpr uint32_t idesc_o = umma_idesc(Fmt<T>::kUmma, 0, 1, kBM, D);
        constexpr uint32_t hi = umma_desc_hi(1024);
        // DQR: q, r (dO comes from tensor memory).  DKV: only v (index 0) is in shared memory, k is in TMEM.
        const uint32_t res_lo0 = umma_desc_lo(res(0), 16), res_lo1 = umma_desc_lo(res(DQR ? 1 : 0), 16);
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
                const uint32_t a1 = res_lo0 + aoff, a2 = res_lo1 + aoff;
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
                        umma_ss_lean<false>(tS + 128, a1, hi, b3, hi, idesc_s);
                    } else {
                        umma_ts_lean<true>(tS, tK + ks * 8, b1, hi, idesc_s);
                        umma_ts_lean<true>(tS + 64, tK + ks * 8, b2, hi, idesc_s);
                        umma_ss_lean<true>(tS + 128, a1, hi, b3, hi, idesc_s);
                    }
                }
            }
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
        int g = 0, n = 0, s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int i = 0; ok; ++i) {
            const int idx = item_index(i, chunk_shift);
            if (idx >= n_items) break;
            const Item it = get_item<DQR>(a, idx, n_mt);
            if (it.n_iter == 0) continue;
            if (warp == 1) {
                ok = mbar_wait(bar(L::kXFull), n & 1, err, 4) && mbar_wait(bar(L::kKReady), n & 1, err, 14);
                ok = __all_sync(0xffffffffu, ok);
                for (int t = 0; t < it.n_iter && ok; ++t, ++g) {
                    ok = mbar_wait(bar(L::kNFull + s), ph, err, 6);
                    // the score columns are free once the element-wise warps have read the previous tile
                    if (ok && g > 0) ok = mbar_wait(bar(L::kSFree), (g - 1) & 1, err, 7);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one_sync()) {
                        issue_scores(s);
                        umma_commit(bar(L::kSFull));
                        if (t == it.n_iter - 1) umma_commit(bar(L::kXEmpty));   // resident tiles and the TMEM tile may be replaced
                    }
                    __syncwarp();
                    if (++s == NS) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            } else {
                for (int t = 0; t < it.n_iter && ok; ++t, ++g) {
                    ok = mbar_wait(bar(L::kGFull), g & 1, err, 8);
                    // the first product of an item overwrites the accumulators: the previous item's epilogue must have read them
                    if (ok && t == 0 && n > 0) ok = mbar_wait(bar(L::kAccFree), (n - 1) & 1, err, 13);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one_sync()) {
                        issue_out(s, t == 0);
                        umma_commit(bar(L::kGFree));
                        umma_commit(bar(L::kNEmpty + s));
                        if (t == it.n_iter - 1) umma_commit(bar(L::kAccDone));
                    }
                    __syncwarp();
                    if (++s == NS) s = 0;
                }
            }
            ++n;
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ element-wise + epilogue
        // warp 4 + w: TMEM lane quarter w % 4 (a warp may only touch the lanes of its own quarter), column
        // group cg = w / 4 of the streamed tile (CPT columns), and for the accumulators one of the two
        const int quarter = warp & 3, cg = (warp - 4) >> 2;
        const int ml = quarter * 32 + lane;                 // lane of the M tile: query row (DQR) / key (DKV)
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const int col0 = cg * CPT;
        const int acc_sel = cg / (CG / 2), part = cg % (CG / 2);   // accumulator (0: dQ | dK, 1: dR | dV) and this warp's share of it
        const float2 c2v = make_float2(a.c2, a.c2), scale2 = make_float2(a.scale, a.scale);
        const int wid = static_cast<int>(threadIdx.x) - 128;
        const bool stat_writer = !DQR && wid < kStatWriters;
        bool ok = true;
        int g = 0, n = 0, i_next = 0;

        // With mL = m + log2(d1), c1 = 1 + bart, ct = b - t:
        //   p = 2^(S1*c2 - mL), un = S2 - c1, dn = b - A   =>   W = -p un, gu = p dn, gl = (p un) dn + p ct
        // DQR: the constants of this thread's row
        float r_ml = INFINITY, r_c1 = 0.f, r_ct = 0.f, r_b = 0.f;
        float4 stat_next = make_float4(0.f, 0.f, 0.f, 0.f);

        // DKV: the per-row statistics of a streamed tile are per-COLUMN constants here.  The first 64
        // element-wise threads fetch one row each ({b, mL, 1 + bart, (b - t) * scale}, 16 bytes) a tile
        // ahead and lay them out in shared memory as four planes of 64 floats (with mL and 1 + bart
        // negated, the latter also times scale), so that every thread reads the constants of adjacent
        // columns as aligned pairs for the packed two-wide arithmetic.  Two buffers: tile g of the CTA
        // uses buffer g & 1.
        auto stat_fetch = [&](const Item &it, int t) -> float4 {
            if (t >= it.n_iter) return make_float4(0.f, 0.f, 0.f, 0.f);
            const int hq = it.hk * a.n_rep + t / it.n_t;
            const int row0 = it.bos + (it.t_lo + t % it.n_t) * kBN;
            return __ldg(reinterpret_cast<const float4 *>(a.cst + ((static_cast<int64_t>(it.b) * a.heads_q + hq) * n_tok + row0 + wid) * 4));
        };
        auto stat_publish = [&](int gg, const float4 &v) {
            float *dst = reinterpret_cast<float *>(smem_raw + L::kStats + (gg % kStatStages) * kStatBytes);
            dst[wid] = -v.y;
            dst[kBN + wid] = -v.z * a.scale;
            dst[2 * kBN + wid] = v.x;
            dst[3 * kBN + wid] = v.w;
            mbar_arrive(bar(L::kStatFull + gg % kStatStages));
        };

        Item cur;
        // next item of this CTA that has tiles to stream; items without any (no visible key / no row
        // that sees the keys) get their zero outputs here
        auto next_item = [&]() -> bool {
            for (;;) {
                const int idx = item_index(i_next++, chunk_shift);
                if (idx >= n_items) return false;
                cur = get_item<DQR>(a, idx, n_mt);
                if (!cur.valid) continue;
                if (cur.n_iter > 0) return true;
                const int row = cur.m0 + ml;
                if (row < (DQR ? cur.nq : cur.nk)) {
                    constexpr int kCh = D / (CG / 2);          // channels of the row written by this thread
                    T *dst = DQR ? static_cast<T *>(acc_sel == 0 ? a.dq : a.dr) + cur.b * a.q_sb + cur.hy * a.q_sh + static_cast<int64_t>(cur.bos + row) * a.q_st
                                 : static_cast<T *>(acc_sel == 0 ? a.dk : a.dv) + cur.b * a.kv_sb + cur.hy * a.kv_sh + static_cast<int64_t>(cur.bos + row) * a.kv_st;
#pragma unroll
                    for (int c = 0; c < kCh / 8; ++c) *reinterpret_cast<uint4 *>(dst + part * kCh + 8 * c) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
        };
        // Start of an item (n-th with tiles of this CTA): the tile of the M side that is the A operand of
        // score products and fits the 64 spare TMEM columns -- DKV: k (S1^T, S2^T), DQR: dO (A) -- goes
        // there instead of shared memory, where MMA operand reads are the scarce resource: this thread's
        // share (D / CG channels) of row mg, two 16-bit channels per column.
        auto prologue = [&](int nn) -> bool {
            const int mg = cur.m0 + ml;
            uint32_t kw[D / (2 * CG)];
            const T *krow = DQR ? static_cast<const T *>(a.go) + cur.b * a.q_sb + cur.hy * a.q_sh + static_cast<int64_t>(cur.bos + mg) * a.q_st + cg * (D / CG)
                                : static_cast<const T *>(a.k) + cur.b * a.kv_sb + cur.hk * a.kv_sh + static_cast<int64_t>(cur.bos + mg) * a.kv_st + cg * (D / CG);
#pragma unroll
            for (int c = 0; c < D / (8 * CG); ++c) {
                uint4 x = make_uint4(0u, 0u, 0u, 0u);
                if (mg < (DQR ? cur.nq : cur.nk)) x = *reinterpret_cast<const uint4 *>(krow + 8 * c);
                kw[4 * c] = x.x; kw[4 * c + 1] = x.y; kw[4 * c + 2] = x.z; kw[4 * c + 3] = x.w;
            }
            if (DQR) {
                r_ml = INFINITY;
                r_c1 = r_ct = r_b = 0.f;
                if (mg < cur.nq) {
                    const float4 hi4 = *reinterpret_cast<const float4 *>(
                        a.cst + ((static_cast<int64_t>(cur.b) * a.heads_q + cur.hy) * n_tok + cur.bos + mg) * 4);   // b, mL, 1 + bart, (b - t) * scale
                    r_b = hi4.x;
                    r_ml = hi4.y;
                    r_c1 = hi4.z;
                    r_ct = hi4.w / a.scale;
                }
            }
            float4 st0 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (stat_writer) {
                st0 = stat_fetch(cur, 0);
                stat_next = stat_fetch(cur, 1);
            }
            // the previous item's score products (the readers of the TMEM tile) must have completed
            if (nn > 0 && !__all_sync(0xffffffffu, mbar_wait(bar(L::kXEmpty), (nn - 1) & 1, err, 16))) return false;
            tc_fence_after();
            tmem_st_cols(tK + lane_base + cg * (D / (2 * CG)), kw);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(L::kKReady));
            // Every thread has handed over the tile before this item's first one (g - 1) and, through the
            // G-buffer wait of that tile, seen tile g - 2 completed by all: the statistics buffer of tile g is free.
            if (stat_writer) stat_publish(g, st0);
            return true;
        };

        bool have = next_item();
        if (have) ok = prologue(0);
        while (have && ok) {
            const int m0 = cur.m0, nq = cur.nq, nk = cur.nk, off = cur.off, mg = m0 + ml;
            for (int it = 0; it < cur.n_iter; ++it, ++g) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kSFull), g & 1, err, 9));
                if (!ok) break;
                tc_fence_after();
                uint32_t x1[CPT], x2[CPT], x3[CPT];
                tmem_ld_cols(tS + lane_base + col0, x1);
                tmem_ld_cols(tS + 64 + lane_base + col0, x2);
                tmem_ld_cols(tS + 128 + lane_base + col0, x3);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(bar(L::kSFree));

                const int tile0 = (cur.t_lo + (DQR ? it : it % cur.n_t)) * kBN;   // first streamed index of the tile
                const int n0 = tile0 + col0;                                      // ... of this thread's columns
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
                const int ss = g % kStatStages;
                const float *stats = reinterpret_cast<const float *>(smem_raw + L::kStats + ss * kStatBytes);
                if (!DQR) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kStatFull + ss), (g / kStatStages) & 1, err, 15));
                    if (!ok) break;
                }
                uint32_t g0[CPT / 2], g1[CPT / 2], g2[CPT / 2];
                // One pair of adjacent columns: constants nml = -mL, nc1 = -(1 + bart), bb = b, ct = b - t (DKV:
                // times scale; DKV: nc1 times scale too).  The third tile carries -W * scale = p un scale (DKV
                // only): the dV accumulator is multiplied by -1 / scale when it is written out, which saves a
                // negation and a multiplication per element here.  `masked` is a compile-time tag:
                // tiles that are visible as a whole (all but the ones on the diagonal or at a window edge) run
                // the loop without any mask arithmetic AND as one basic block, so that the independent pairs
                // interleave; a branch per pair would keep them apart.
                auto pair = [&](auto masked, int c, const float2 &nml, const float2 &nc1, const float2 &bb, const float2 &ct) {
                    const float2 s1 = make_float2(__uint_as_float(x1[c]), __uint_as_float(x1[c + 1]));
                    const float2 s2 = make_float2(__uint_as_float(x2[c]), __uint_as_float(x2[c + 1]));
                    const float2 av = make_float2(__uint_as_float(x3[c]), __uint_as_float(x3[c + 1]));
                    const float2 arg = __ffma2_rn(s1, c2v, nml);
                    const float2 p = make_float2(fast_exp2(arg.x), fast_exp2(arg.y));
                    // DKV carries qk_scale on gl = (p un scale) dn + p ct scale: nc1 and ct come scaled from the
                    // statistics planes, so wn = -W scale there (1 / scale goes on dV when it is written out)
                    const float2 un = DQR ? __fadd2_rn(s2, nc1) : __ffma2_rn(s2, scale2, nc1);
                    const float2 dn = __ffma2_rn(av, make_float2(-1.f, -1.f), bb);
                    const float2 pc = __fmul2_rn(p, ct);
                    float2 wn = __fmul2_rn(p, un);                            // -W (DKV: times scale)
                    float2 gu = __fmul2_rn(p, dn);
                    float2 gl = __ffma2_rn(wn, dn, pc);
                    if (decltype(masked)::value) {
                        const bool v0 = n0 + c >= lim_lo && n0 + c <= lim_hi, v1 = n0 + c + 1 >= lim_lo && n0 + c + 1 <= lim_hi;
                        gl = make_float2(v0 ? gl.x : 0.f, v1 ? gl.y : 0.f);
                        gu = make_float2(v0 ? gu.x : 0.f, v1 ? gu.y : 0.f);
                        wn = make_float2(v0 ? wn.x : 0.f, v1 ? wn.y : 0.f);
                    }
                    g0[c >> 1] = Elem<T>::pack(gl.x, gl.y);
                    g1[c >> 1] = Elem<T>::pack(gu.x, gu.y);
                    if (!DQR) g2[c >> 1] = Elem<T>::pack(wn.x, wn.y);
                };
                auto tile_math = [&](auto masked) {
                    if (DQR) {
                        const float2 nml = make_float2(-r_ml, -r_ml), nc1 = make_float2(-r_c1, -r_c1), bb = make_float2(r_b, r_b),
                                     ct = make_float2(r_ct, r_ct);
#pragma unroll
                        for (int c = 0; c < CPT; c += 2) pair(masked, c, nml, nc1, bb, ct);
                    } else {
                        const float *pl = stats + col0;
#pragma unroll
                        for (int c = 0; c < CPT; c += 4) {
                            const float4 nml = *reinterpret_cast<const float4 *>(pl + c);
                            const float4 nc1 = *reinterpret_cast<const float4 *>(pl + kBN + c);
                            const float4 bb = *reinterpret_cast<const float4 *>(pl + 2 * kBN + c);
                            const float4 ct = *reinterpret_cast<const float4 *>(pl + 3 * kBN + c);
                            pair(masked, c, make_float2(nml.x, nml.y), make_float2(nc1.x, nc1.y), make_float2(bb.x, bb.y), make_float2(ct.x, ct.y));
                            pair(masked, c + 2, make_float2(nml.z, nml.w), make_float2(nc1.z, nc1.w), make_float2(bb.z, bb.w), make_float2(ct.z, ct.w));
                        }
                    }
                };
                if (full) tile_math(std::false_type{});
                else tile_math(std::true_type{});
                // the G tiles are free once the output products of the previous tile have completed
                if (g > 0) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kGFree), (g - 1) & 1, err, 10));
                    if (!ok) break;
                }
                // Every thread has handed over tile g - 1 (the output products that just completed needed all
                // of its G rows), so nobody reads the statistics buffer of tile g - 1 any more: refill it.
                if (stat_writer && it + 1 < cur.n_iter) {
                    stat_publish(g + 1, stat_next);
                    stat_next = stat_fetch(cur, it + 2);
                }
                // row ml of each G tile: 128 bytes, 16-byte chunk i stored at position i ^ (ml & 7)
#pragma unroll
                for (int c = 0; c < CPT / 8; ++c) {
                    const uint32_t o = static_cast<uint32_t>(ml) * 128u + static_cast<uint32_t>(((cg * (CPT / 8) + c) ^ (ml & 7)) * 16);
                    st_shared_v4(gt(0) + o, g0[4 * c], g0[4 * c + 1], g0[4 * c + 2], g0[4 * c + 3]);
                    st_shared_v4(gt(1) + o, g1[4 * c], g1[4 * c + 1], g1[4 * c + 2], g1[4 * c + 3]);
                    if (!DQR) st_shared_v4(gt(2) + o, g2[4 * c], g2[4 * c + 1], g2[4 * c + 2], g2[4 * c + 3]);
                }
                fence_proxy_async();
                mbar_arrive(bar(L::kGFull));
            }
            if (!ok) break;

            // ---- what the epilogue of this item needs, then the start of the next item: its TMEM tile and
            // first score products are under way while the accumulators of this one are written out
            // dQ carries qk_scale; the dV accumulator holds -dV * qk_scale (the W tile is stored as -W * qk_scale)
            const float mul = DQR ? (acc_sel == 0 ? a.scale : 1.f) : (acc_sel == 0 ? 1.f : -1.f / a.scale);
            const int rows_left = (DQR ? nq : nk) - m0;
            T *dst0;
            int64_t row_stride;
            if (DQR) {
                dst0 = static_cast<T *>(acc_sel == 0 ? a.dq : a.dr) + cur.b * a.q_sb + cur.hy * a.q_sh + static_cast<int64_t>(cur.bos + m0) * a.q_st;
                row_stride = a.q_st;
            } else {
                dst0 = static_cast<T *>(acc_sel == 0 ? a.dk : a.dv) + cur.b * a.kv_sb + cur.hy * a.kv_sh + static_cast<int64_t>(cur.bos + m0) * a.kv_st;
                row_stride = a.kv_st;
            }
            have = next_item();
            if (have) {
                ok = prologue(n + 1);
                if (!ok) break;
            }

            // epilogue: half of the element-wise warps write acc0 (dQ | dK), the other half acc1 (dR | dV); an
            // accumulator is 2 x D / 64 units of 16 rows x 64 columns per lane quarter, dealt out to the CG / 2
            // warps of the quarter.  The accumulators are read in the fragment arrangement (a row is spread
            // over the four lanes of a quad); a 4 x 4 word transpose inside the quad gives every thread 16
            // contiguous bytes, so a warp store covers 64 contiguous bytes of 8 rows.
            ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kAccDone), n & 1, err, 11));
            if (!ok) break;
            tc_fence_after();
            const int gq = lane >> 2, t = lane & 3;
            const uint32_t acc = acc_sel == 0 ? tAcc0 : tAcc1;
            constexpr int kUnits = 2 * (D / 64), kParts = CG / 2;
#pragma unroll 1
            for (int u = part; u < kUnits; u += kParts) {
                const int rh = u / (D / 64), cc = u % (D / 64);
                const int rl = quarter * 32 + rh * 16 + gq;     // local rows of this thread: rl and rl + 8
                uint32_t x[32];
                tmem_ld_16x256b_x8(acc + (static_cast<uint32_t>(quarter * 32 + rh * 16) << 16) + 64 * cc, x);
                tmem_wait_ld();
                if (u + kParts >= kUnits) {
                    // this thread's share of the accumulators is in registers: the next item may overwrite them
                    tc_fence_before();
                    mbar_arrive(bar(L::kAccFree));
                }
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                    for (int grp = 0; grp < 2; ++grp) {
                        uint32_t w[4];
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const int e = 4 * (4 * grp + kk) + 2 * hh;
                            w[kk] = Elem<T>::pack(__uint_as_float(x[e]) * mul, __uint_as_float(x[e + 1]) * mul);
                        }
                        quad_transpose(w, t);
                        const int row = rl + 8 * hh;
                        if (row < rows_left)
                            *reinterpret_cast<uint4 *>(dst0 + static_cast<int64_t>(row) * row_stride + 64 * cc + 32 * grp + 8 * t) =
                                make_uint4(w[0], w[1], w[2], w[3]);
                    }
            }
            ++n;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------- //
// host side
// ------------------------------------------------------------------------- //
template <typename T, int D, int MODE>
int launch_mode(const TrainArgs &a, int n_tok, const ErrSink &sink, cudaStream_t stream) {
    // Ring depth: as many stages as the 227 KB of shared memory allow at head_dim 128 (dk/dv 3, dq/dr 4); six at
    // head_dim 64 (measured against four: dq/dr 0.883 vs 0.919 ms, dk/dv 1.337 vs 1.352 ms; two stages cost 20 %).
    constexpr int NS = D == 64 ? 6 : (MODE == kModeDKV ? 3 : 4);
    using L = Smem<D, MODE, NS>;
    constexpr bool DQR = MODE == kModeDQR;
    const int q_rows = DQR ? kBM : kBN, kv_rows = DQR ? kBN : kBM;
    CUtensorMap tq, tr, tg, tk, tv;
    const CUtensorMapDataType dt = Fmt<T>::kTma;
    if (!tma::make_map(&tq, dt, a.q, D, a.len_q, a.heads_q, a.batch, a.q_st, a.q_sh, a.q_sb, q_rows) ||
        !tma::make_map(&tr, dt, a.r, D, a.len_q, a.heads_q, a.batch, a.q_st, a.q_sh, a.q_sb, q_rows) ||
        !tma::make_map(&tg, dt, a.go, D, a.len_q, a.heads_q, a.batch, a.q_st, a.q_sh, a.q_sb, q_rows) ||
        !tma::make_map(&tk, dt, a.k, D, a.len_k, a.heads_kv, a.batch, a.kv_st, a.kv_sh, a.kv_sb, kv_rows) ||
        !tma::make_map(&tv, dt, a.v, D, a.len_k, a.heads_kv, a.batch, a.kv_st, a.kv_sh, a.kv_sb, kv_rows))
        return PLX_ERR_LAUNCH;
    // Eight element-wise warps (32 of the 64 streamed columns per thread).  Sixteen were faster while the
    // tile arithmetic had a branch per column pair; as one basic block the longer per-thread chain
    // interleaves well enough, and eight measured 1.150 / 1.530 ms (dq/dr, dk/dv) against 1.176 / 1.588 with
    // sixteen at B=8, H=16, L=4096, head_dim 128 (head_dim 64: 0.923 / 1.353 against 0.926 / 1.50).
    constexpr int EW = PLX_BWD_EW_WARPS;
    auto kern = bwd_sm100_kernel<T, D, MODE, NS, EW>;
    static std::mutex attr_mu;
    static bool attr_done[tma::kMaxDevices] = {};
    if (!tma::opt_in_smem(kern, static_cast<int>(L::kBytes), attr_done, attr_mu)) return PLX_ERR_LAUNCH;
    const int len = DQR ? a.len_q : a.len_k;
    const int tiles = a.cu ? (len + kBM - 1) / kBM + a.n_seqs : (len + kBM - 1) / kBM;
    const int n_items = tiles * a.batch * (DQR ? a.heads_q : a.heads_kv), sms = tma::sm_count();
    if (sms <= 0) return PLX_ERR_LAUNCH;
    // with plenty of items a CTA takes them in neighbouring pairs (a heavy and a light tile)
    const int chunk_shift = n_items >= 2 * sms ? 1 : 0;
    const int units = (n_items + (1 << chunk_shift) - 1) >> chunk_shift;
    kern<<<units < sms ? units : sms, (4 + EW) * 32, L::kBytes, stream>>>(a, n_tok, tq, tr, tg, tk, tv, sink, tiles, n_items, chunk_shift);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? PLX_OK : PLX_ERR_LAUNCH;
}

}  // namespace

bool train_bwd_sm100_supported(const TrainArgs &a, int head_dim) {
    if ((head_dim != 64 && head_dim != 128) || a.window == 0 || !(a.c2 > 0.f)) return false;
    const char *env = std::getenv("PLX_BWD_KERNEL");
    if (env && env[0] == 'm') return false;  // "mma": force the warp-level kernels
    return tma::encode_fn() != nullptr;
}

int launch_train_bwd_sm100(const TrainArgs &a, int dtype, int head_dim, int stage, cudaStream_t stream) {
    const ErrorWords ew = sm100_error_words();
    if (!ew.word) return PLX_ERR_LAUNCH;
    const ErrSink err{ew.word, ew.mirror};
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
