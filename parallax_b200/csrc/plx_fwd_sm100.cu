// Parallax training forward on the Blackwell tensor cores: tcgen05.mma with the
// accumulators in tensor memory, q / r / k / v tiles staged by TMA, and a
// warp-specialised producer / MMA-issuer / softmax pipeline.  head_dim 64 or 128.
//
// Work item = one 128-row query tile of one (batch, q head); key tiles of 64.  The kernel is
// persistent: at most one CTA per SM, each walking its share of the item list, so the loads and
// first score products of an item run under the epilogue of the one before it.
//
//   warp 0      TMA producer: Q and R of each item, K_j and V_j through NS-deep rings
//   warp 1      allocates the 512 TMEM columns; one lane issues the score products
//                   S1_j = Q K_j^T, S2_j = R K_j^T        (A, B from shared memory)
//   warp 10     one lane issues the output products
//                   O1 += P1_j V_j,  O2 += P2_j V_j        (A = P from TMEM, B = V from shared memory)
//   warps 2-9   softmax: warps w and w + 4 share TMEM lane quarter w % 4 (16 rows each);
//               they read S1, S2 in the accumulator-fragment arrangement, keep the
//               running max / sums, write P1 = 2^(S1*c2 - m), P2 = P1*S2 as 16-bit pairs
//               into a P buffer, rescale O1 / O2 when the reference maximum has to
//               move, and write the outputs at the end (one thread per row).
//
// TMEM columns at head_dim 128: O1 [0,128)  O2 [128,256)  S1 [256,320)  S2 [320,384)  and two P
// buffers {P1 [.., +32), P2 [.., +32)} at 384 and 448.  The softmax warps copy S1 / S2 into registers and
// release the S columns at once, so S_{j+1} is computed while they work on tile j; P_j waits in
// its own buffer for the output products, which run under the softmax of tile j + 1.
// At head_dim 64 the accumulators take 128 columns and there are THREE score buffers (at 128, 256, 384),
// with P1 / P2 written in place over the first 32 columns of the tile's own S1 / S2: the score products
// of tile j + 1 do not wait for the softmax warps to pick up tile j, only for the output products of
// tile j - 2.  Measured with clock64 stamps at head_dim 128, the round trip scores -> TMEM load ->
// release -> issue -> scores sets the pace with one buffer (1700 clocks per tile, 950 of them the 16
// score MMAs queued behind the previous output products); two buffers with P in place, all that fits at
// head_dim 128, put softmax -> output products -> scores of tile j + 2 in series instead and measured
// slower (1.02 vs 0.985 ms).  At head_dim 64: one buffer 0.87 ms, two buffers and separate P buffers
// 0.92 ms (the scores run ahead and delay the output products in the tensor queue), two in place 0.77 ms,
// three in place 0.76 ms.
//
// The reference maximum m_ref only moves when a tile maximum exceeds it by more
// than 8 (in base-2 units): P stays below 2^8, the O rescale (a TMEM round trip)
// is skipped for almost every tile, and the saved statistics are converted to the
// true row maximum at the end, so results do not depend on when it moved.
//
// Math and saved statistics: parallax/triton/parallax_train.py:144-252 of the reference.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "plx_common.cuh"
#include "plx_launch.h"
#include "plx_sm100.cuh"
#include "plx_tma_host.h"

namespace plx {

using namespace sm100;

// first error recorded by a tcgen05 kernel of this library on the current device (0 = none)
static __device__ int g_sm100_error;

namespace {

constexpr int kBM = 128, kBN = 64;
constexpr uint32_t kQPanel = kBM * 128;       // bytes of one 64-channel panel of a q tile
constexpr uint32_t kKVPanel = kBN * 128;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.f;

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

// D = head dim (64 or 128): tiles are D / 64 panels of [rows][64 channels]
template <int D, int NS>
struct Smem {
    static constexpr int kPanels = D / 64;
    static constexpr uint32_t kQBytes = kPanels * kQPanel;     // one q or r tile
    static constexpr uint32_t kKVBytes = kPanels * kKVPanel;   // one k or v tile
    static constexpr uint32_t kQ = 0, kR = kQBytes, kK = 2 * kQBytes, kV = kK + NS * kKVBytes;
    static constexpr uint32_t kBars = kV + NS * kKVBytes;
    // barrier indices (8 bytes each)
    static constexpr int kQFull = 0, kQEmpty = 1, kOFree = 2, kKFull = 3, kKEmpty = kKFull + NS,
                         kVFull = kKEmpty + NS, kVEmpty = kVFull + NS, kSFull = kVEmpty + NS, kSFree = kSFull + 3,
                         kPFull = kSFree + 1, kPVDone = kPFull + 3, kNumBars = kPVDone + 3;
    static constexpr uint32_t kTmemSlot = kBars + 8 * kNumBars;
    static constexpr uint32_t kBytes = kTmemSlot + 16 + 1024;  // + slack to align the base to 1024
};

// One unit of work: a 128-row query tile of one (batch, q head).
struct Item {
    int bos, nq, nk, r0, b, h, hk, off, t_lo, n_tiles;   // key tiles t_lo .. t_lo + n_tiles - 1
    bool valid;
};

// Work item `idx` of the launch.  Items are ordered (batch, head)-major so that CTAs running at the
// same time share K / V in L2; inside a (batch, head) the row tiles alternate last, first, last - 1,
// second, ... so that under a causal mask any two neighbours add up to the same work.
__device__ __forceinline__ Item get_item(const TrainArgs &a, int idx, int n_rt) {
    Item it;
    const int bh = idx / n_rt, k = idx % n_rt;
    const int tile_id = (k & 1) ? (k >> 1) : n_rt - 1 - (k >> 1);
    Seq s;
    int tis = 0;
    it.valid = locate_tile(a, tile_id, kBM, s, tis);
    it.bos = s.bos;
    it.nq = s.nq;
    it.nk = s.nk;
    it.r0 = tis * kBM;
    if (it.valid && it.r0 >= it.nq) it.valid = false;
    it.b = bh / a.heads_q;
    it.h = bh % a.heads_q;
    it.hk = it.h / a.n_rep;
    it.off = it.nk - it.nq;
    // keys [lo_col, hi_col) are visible to some row of this tile (a sliding window drops whole key tiles)
    const int hi_col = min(it.nk, it.r0 + kBM + it.off);
    const int lo_col = a.window < 0 ? 0 : max(0, it.r0 + it.off - a.window + 1);
    it.t_lo = lo_col / kBN;
    it.n_tiles = (it.valid && hi_col > lo_col) ? (hi_col + kBN - 1) / kBN - it.t_lo : 0;
    return it;
}

// n-th item of this CTA: CTAs take chunks of 2^chunk_shift neighbouring items, round robin.
__device__ __forceinline__ int item_index(int n, int chunk_shift) {
    return ((blockIdx.x + gridDim.x * (n >> chunk_shift)) << chunk_shift) + (n & ((1 << chunk_shift) - 1));
}

// Persistent kernel: gridDim.x CTAs (at most one per SM) walk the item list, so the loads and first
// score products of the next item overlap the epilogue of the current one, and the TMEM allocation,
// barrier set-up and launch latency are paid once per SM.
template <typename T, int D, int NS>
__global__ void __launch_bounds__(352, 1)
fwd_sm100_kernel(const TrainArgs a, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_r,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const ErrSink sink, int n_rt,
                 int n_items, int chunk_shift) {
    using L = Smem<D, NS>;
    constexpr uint32_t kQBytes = L::kQBytes, kKVBytes = L::kKVBytes;
    extern __shared__ unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base + L::kQ, sR = base + L::kR, sK = base + L::kK, sV = base + L::kV;
    auto bar = [&](int i) -> uint32_t { return base + L::kBars + 8u * i; };
    const uint32_t tmem_slot = base + L::kTmemSlot;
    const WaitCtx err{sink, tmem_slot + 8};   // the CTA's abort flag sits beside the TMEM slot

    if (threadIdx.x == 0) {
        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(err.abort_flag), "r"(0u) : "memory");
        for (int i = 0; i < L::kNumBars; ++i) {
            const bool all_softmax =
                (i >= L::kPFull && i < L::kPFull + 3) || i == L::kOFree || i == L::kSFree;
            mbar_init(bar(i), all_softmax ? 256 : 1);   // arrivals from all 256 softmax threads, else one
        }
        fence_barrier_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_r);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
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
    const uint32_t tO1 = tmem_base, tO2 = tmem_base + D;
    // Score buffers {S1, S2}.  head_dim 128: one (the accumulators leave no room for more), and two P
    // buffers of their own.  head_dim 64: three, and P1 / P2 of a tile (16-bit pairs, 32 columns each) are
    // written IN PLACE over the first half of its S1 / S2 once the softmax warps hold the scores in
    // registers; the buffer is free for the scores of tile g + 3 when the output products of tile g have
    // completed.  Tile g uses buffer g % kSBufs (and P buffer g % kPBufs) for the (g / k..Bufs)-th time.
    constexpr bool kInPlace = D == 64;
    constexpr int kSBufs = kInPlace ? 3 : 1, kPBufs = kInPlace ? 3 : 2;
    auto tS1 = [&](int sb) -> uint32_t { return tmem_base + 2 * D + 128 * sb; };
    auto tS2 = [&](int sb) -> uint32_t { return tmem_base + 2 * D + 128 * sb + 64; };
    auto tP1 = [&](int pb) -> uint32_t { return kInPlace ? tS1(pb) : tmem_base + 384 + 64 * pb; };
    auto tP2 = [&](int pb) -> uint32_t { return kInPlace ? tS2(pb) : tmem_base + 384 + 64 * pb + 32; };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // lane 0: Q, R of every item and the K ring; lane 1: the V ring (a V stage is released a tile
        // later than its K stage, so one thread serving both would hold the K refills back)
        if (lane < 2) {
            const bool is_k = lane == 0;
            const CUtensorMap *map = is_k ? &tm_k : &tm_v;
            const uint32_t ring = is_k ? sK : sV;
            const int full0 = is_k ? L::kKFull : L::kVFull, empty0 = is_k ? L::kKEmpty : L::kVEmpty;
            int s = 0, n_issued = 0, n_items_done = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int n = 0; ok; ++n) {
                const int idx = item_index(n, chunk_shift);
                if (idx >= n_items) break;
                const Item it = get_item(a, idx, n_rt);
                if (it.n_tiles == 0) continue;
                if (is_k) {
                    // the q / r tiles of the previous item are free once its last score product has completed
                    ok = mbar_wait(bar(L::kQEmpty), (n_items_done & 1) ^ 1, err, 1);
                    if (!ok) break;
                    mbar_expect_tx(bar(L::kQFull), 2 * kQBytes);
#pragma unroll
                    for (int pn = 0; pn < L::kPanels; ++pn) {
                        tma_load_4d(sQ + pn * kQPanel, &tm_q, bar(L::kQFull), 64 * pn, it.bos + it.r0, it.h, it.b);
                        tma_load_4d(sR + pn * kQPanel, &tm_r, bar(L::kQFull), 64 * pn, it.bos + it.r0, it.h, it.b);
                    }
                }
                ++n_items_done;
                for (int j = 0; j < it.n_tiles; ++j) {
                    ok = mbar_wait(bar(empty0 + s), ph ^ 1, err, is_k ? 2 : 3);
                    if (!ok) break;
                    mbar_expect_tx(bar(full0 + s), kKVBytes);
#pragma unroll
                    for (int pn = 0; pn < L::kPanels; ++pn)
                        tma_load_4d(ring + s * kKVBytes + pn * kKVPanel, map, bar(full0 + s), 64 * pn, it.bos + (it.t_lo + j) * kBN,
                                    it.hk, it.b);
                    ++n_issued;
                    if (++s == NS) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
            if (!ok) {
                // unwinding: let the copies already in flight land before the CTA (and its shared memory) goes away
                for (int i = 0; i < min(n_issued, NS); ++i) {
                    if (--s < 0) {
                        s = NS - 1;
                        ph ^= 1;
                    }
                    mbar_wait_quiet(bar(full0 + s), ph);
                }
                if (is_k && n_items_done > 0) mbar_wait_quiet(bar(L::kQFull), (n_items_done - 1) & 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer 1: S1_j, S2_j
        // The MMAs are issued by two threads in two warps (this one: the score products; warp 10: the
        // output products), because one thread's instruction stream, not the tensor pipe, is what bounds
        // a single issuer.  Descriptor low words are "base + immediate", high words and flags constants.
        // The whole warp runs the loop (so that its values stay warp-uniform); one elected lane issues.
        {
            constexpr uint32_t idesc_s = umma_idesc(Fmt<T>::kUmma, 0, 0, kBM, kBN);
            constexpr uint32_t hi_k = umma_desc_hi(1024);                 // K-major tiles: 8-row groups 1024 B apart
            const uint32_t q_lo = umma_desc_lo(sQ, 16), r_lo = umma_desc_lo(sR, 16);
            const uint32_t k_lo0 = umma_desc_lo(sK, 16);
            bool ok = true;
            int s = 0, g = 0, n_items_done = 0;                           // K ring stage, key tiles and items so far
            uint32_t ph = 0;                                              // phase of the K ring
            for (int n = 0; ok; ++n) {
                const int idx = item_index(n, chunk_shift);
                if (idx >= n_items) break;
                const Item it = get_item(a, idx, n_rt);
                if (it.n_tiles == 0) continue;
                ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kQFull), n_items_done & 1, err, 4));
                ++n_items_done;
                for (int j = 0; j < it.n_tiles && ok; ++j, ++g) {
                    ok = mbar_wait(bar(L::kKFull + s), ph, err, 6);
                    const int sb = g % kSBufs;
                    if (kInPlace) {
                        // the buffer holds the P of tile g - 3 until its output products have completed
                        if (ok && g >= kSBufs) ok = mbar_wait(bar(L::kPVDone + sb), (g / kSBufs - 1) & 1, err, 5);
                    } else {
                        // the softmax warps must have copied the previous S1 / S2 into registers
                        if (ok && g >= 1) ok = mbar_wait(bar(L::kSFree), (g - 1) & 1, err, 5);
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t k_lo = k_lo0 + s * (kKVBytes >> 4);
                    const uint32_t d1 = tS1(sb), d2 = tS2(sb);
                    if (elect_one_sync()) {
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        const uint32_t qoff = ((ks >> 2) * kQPanel + (ks & 3) * 32) >> 4;
                        const uint32_t koff = ((ks >> 2) * kKVPanel + (ks & 3) * 32) >> 4;
                        if (ks == 0) {
                            umma_ss_lean<false>(d1, q_lo + qoff, hi_k, k_lo + koff, hi_k, idesc_s);
                            umma_ss_lean<false>(d2, r_lo + qoff, hi_k, k_lo + koff, hi_k, idesc_s);
                        } else {
                            umma_ss_lean<true>(d1, q_lo + qoff, hi_k, k_lo + koff, hi_k, idesc_s);
                            umma_ss_lean<true>(d2, r_lo + qoff, hi_k, k_lo + koff, hi_k, idesc_s);
                        }
                    }
                    umma_commit(bar(L::kKEmpty + s));
                    umma_commit(bar(L::kSFull + sb));
                    if (j == it.n_tiles - 1) umma_commit(bar(L::kQEmpty));   // q / r may be replaced
                    }
                    __syncwarp();
                    if (++s == NS) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 10) {
        // ------------------------------------------------------------------ MMA issuer 2: O1 += P1_j V_j, O2 += P2_j V_j
        {
            constexpr uint32_t idesc_pv = umma_idesc(Fmt<T>::kUmma, 0, 1, kBM, D);
            constexpr uint32_t hi_v = umma_desc_hi(1024);                 // V as MN-major B: 8-key groups 1024 B apart
            const uint32_t v_lo0 = umma_desc_lo(sV, kKVPanel);            // LBO = distance of the two 64-channel panels
            bool ok = true;
            int s = 0, g = 0, n_items_done = 0;
            uint32_t ph = 0;
            for (int n = 0; ok; ++n) {
                const int idx = item_index(n, chunk_shift);
                if (idx >= n_items) break;
                const Item it = get_item(a, idx, n_rt);
                if (it.n_tiles == 0) continue;
                for (int j = 0; j < it.n_tiles && ok; ++j, ++g) {
                    const int buf = g % kPBufs;
                    ok = mbar_wait(bar(L::kPFull + buf), (g / kPBufs) & 1, err, 7) && mbar_wait(bar(L::kVFull + s), ph, err, 8);
                    // the first product of an item overwrites O1 / O2: the previous item's epilogue must have read them
                    if (ok && j == 0 && n_items_done > 0) ok = mbar_wait(bar(L::kOFree), (n_items_done - 1) & 1, err, 13);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t v_lo = v_lo0 + s * (kKVBytes >> 4);
                    const uint32_t a1 = tP1(buf), a2 = tP2(buf);
                    // 16 keys per MMA: P columns advance by 8, V rows by 16 x 128 B
                    if (elect_one_sync()) {
                    if (j > 0) {
                        umma_ts_lean<true>(tO1, a1, v_lo, hi_v, idesc_pv);
                        umma_ts_lean<true>(tO2, a2, v_lo, hi_v, idesc_pv);
                    } else {
                        umma_ts_lean<false>(tO1, a1, v_lo, hi_v, idesc_pv);
                        umma_ts_lean<false>(tO2, a2, v_lo, hi_v, idesc_pv);
                    }
#pragma unroll
                    for (int kk = 1; kk < kBN / 16; ++kk) {
                        umma_ts_lean<true>(tO1, a1 + kk * 8, v_lo + kk * (2048 >> 4), hi_v, idesc_pv);
                        umma_ts_lean<true>(tO2, a2 + kk * 8, v_lo + kk * (2048 >> 4), hi_v, idesc_pv);
                    }
                    umma_commit(bar(L::kVEmpty + s));
                    umma_commit(bar(L::kPVDone + buf));
                    }
                    __syncwarp();
                    if (++s == NS) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                ++n_items_done;
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        // Eight warps.  Warps w and w + 4 share TMEM lane quarter w % 4: warp w owns its rows 0..15,
        // warp w + 4 its rows 16..31, each for all 64 columns of a key tile, in the accumulator-fragment
        // arrangement (a row is spread over the four lanes of a quad), so row maxima are quad shuffles
        // and the two warps of a scheduler partition hide each other's latencies.
        const int quarter = warp & 3, hf = (warp - 2) >> 2;
        const int g4 = lane >> 2, t = lane & 3;
        const int rl0 = quarter * 32 + hf * 16 + g4;       // local rows of this thread: rl0 and rl0 + 8
        const uint32_t frag_base = static_cast<uint32_t>(quarter * 32 + hf * 16) << 16;
        const float2 c2v = make_float2(a.c2, a.c2);
        bool ok = true;
        int g = 0, n_items_done = 0;                       // key tiles and items (with keys) so far

        for (int n = 0; ok; ++n) {
            const int idx = item_index(n, chunk_shift);
            if (idx >= n_items) break;
            const Item it = get_item(a, idx, n_rt);
            if (!it.valid) continue;
            if (it.n_tiles == 0) {
                // no key is visible to any row of the tile: outputs are zero (one thread per row and column half)
                const int row = it.r0 + quarter * 32 + lane;
                if (row < it.nq) {
                    const int64_t q_base = it.b * a.q_sb + it.h * a.q_sh + static_cast<int64_t>(it.bos + row) * a.q_st;
                    T *go = static_cast<T *>(a.o) + q_base + (D / 2) * hf;
                    T *gb = static_cast<T *>(a.barv) + q_base + (D / 2) * hf;
                    const int64_t si = it.b * a.st_sb + it.h * a.st_sh + static_cast<int64_t>(it.bos + row) * a.st_st;
                    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                    for (int i = 0; i < D / 16; ++i) {
                        *reinterpret_cast<uint4 *>(go + 8 * i) = z;
                        *reinterpret_cast<uint4 *>(gb + 8 * i) = z;
                    }
                    if (hf == 0) {
                        a.d1[si] = 0.f;
                        a.bart[si] = 0.f;
                        a.m[si] = -INFINITY;
                    }
                }
                continue;
            }

            const int r0 = it.r0, off = it.off, nk = it.nk;
            float m_ref[2] = {-INFINITY, -INFINITY}, m_true[2] = {-INFINITY, -INFINITY};
            float d1[2] = {0.f, 0.f}, d2[2] = {0.f, 0.f};  // this thread's share of the row sums
            // Rows that see only a few keys (the first 64 positions of a sequence) do not average out the
            // rounding of P: for them the output is normalised with the sums of the ROUNDED P1 / P2 that
            // multiply V, so that bart * barv - O2 / d1 = sum_j P2_j (barv - v_j) / d1 cancels as in exact
            // arithmetic (a row with a single key returns v exactly).  The saved statistics are always the
            // fp32 sums, which is what the backward recomputes.
            const bool exact_norm = (r0 + off < kBN) || (a.window >= 0 && a.window <= 2 * kBN);
            float d1r[2] = {0.f, 0.f}, d2r[2] = {0.f, 0.f};

            for (int j = 0; j < it.n_tiles; ++j, ++g) {
                const int buf = g % kPBufs;
                const int sb = g % kSBufs;
                ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kSFull + sb), (g / kSBufs) & 1, err, 9));
                if (!ok) break;
                tc_fence_after();
                uint32_t s1[32], s2[32];
                tmem_ld_16x256b_x8(tS1(sb) + frag_base, s1);
                tmem_ld_16x256b_x8(tS2(sb) + frag_base, s2);
                tmem_wait_ld();
                if (!kInPlace) {
                    tc_fence_before();
                    mbar_arrive(bar(L::kSFree));                 // the next score products may overwrite S1 / S2
                }

                const int c0 = (it.t_lo + j) * kBN;
                const bool need_mask = (c0 + kBN - 1 > r0 + off) || (c0 + kBN > nk) ||
                                       (a.window >= 0 && c0 < r0 + kBM + off - a.window);
                if (need_mask) {
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int pos = r0 + rl0 + 8 * hh + off;
                        const int last = min(pos, nk - 1);                        // last visible key of the row
                        const int first = a.window < 0 ? 0 : pos - a.window + 1;  // first visible key of the row
#pragma unroll
                        for (int k = 0; k < 8; ++k)
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int c = c0 + 8 * k + 2 * t + e;
                                if (c > last || c < first) s1[4 * k + 2 * hh + e] = 0xff800000u;  // -inf
                            }
                    }
                }
                float mx[2];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        m0 = fmaxf(m0, __uint_as_float(s1[4 * k + 2 * hh]));
                        m1 = fmaxf(m1, __uint_as_float(s1[4 * k + 2 * hh + 1]));
                    }
                    float m = fmaxf(m0, m1);
                    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                    mx[hh] = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                }
                bool grow[2];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const float m_tile = mx[hh] * a.c2;               // c2 > 0 (checked on the host)
                    m_true[hh] = fmaxf(m_true[hh], m_tile);
                    grow[hh] = m_tile > m_ref[hh] + kRescaleThreshold;
                }
                if (__any_sync(0xffffffffu, grow[0] || grow[1])) {
                    float alpha[2];
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const float m_new = grow[hh] ? m_true[hh] : m_ref[hh];
                        alpha[hh] = (m_ref[hh] == -INFINITY) ? 0.f : fast_exp2(m_ref[hh] - m_new);
                        m_ref[hh] = m_new;
                        d1[hh] *= alpha[hh];
                        d2[hh] *= alpha[hh];
                        d1r[hh] *= alpha[hh];
                        d2r[hh] *= alpha[hh];
                    }
                    if (j > 0) {
                        ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kPVDone + (g - 1) % kPBufs), ((g - 1) / kPBufs) & 1, err, 10));
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll 1
                        for (int c = 0; c < 2 * D; c += 64) {  // O1 then O2, 64 columns at a time
                            uint32_t o[32];
                            tmem_ld_16x256b_x8(tO1 + frag_base + c, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha[(i >> 1) & 1]);
                            tmem_st_16x256b_x8(tO1 + frag_base + c, o);
                        }
                        tmem_wait_st();
                    }
                }
                float2 negm[2], sum1[2], sum2[2];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const float nm = (m_ref[hh] == -INFINITY) ? 0.f : -m_ref[hh];
                    negm[hh] = make_float2(nm, nm);
                    sum1[hh] = sum2[hh] = make_float2(0.f, 0.f);
                }
#pragma unroll
                for (int k = 0; k < 8; ++k)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int i = 4 * k + 2 * hh;
                        const float2 arg =
                            __ffma2_rn(make_float2(__uint_as_float(s1[i]), __uint_as_float(s1[i + 1])), c2v, negm[hh]);
                        const float2 p = make_float2(fast_exp2(arg.x), fast_exp2(arg.y));
                        sum1[hh] = __fadd2_rn(sum1[hh], p);
                        s1[i] = __float_as_uint(p.x);
                        s1[i + 1] = __float_as_uint(p.y);
                    }
                uint32_t p1[16], p2[16];
#pragma unroll
                for (int k = 0; k < 8; ++k)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int i = 4 * k + 2 * hh;
                        const float2 p = make_float2(__uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
                        const float2 q = __fmul2_rn(p, make_float2(__uint_as_float(s2[i]), __uint_as_float(s2[i + 1])));
                        sum2[hh] = __fadd2_rn(sum2[hh], q);
                        p1[2 * k + hh] = Elem<T>::pack(p.x, p.y);
                        p2[2 * k + hh] = Elem<T>::pack(q.x, q.y);
                    }
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    d1[hh] += sum1[hh].x + sum1[hh].y;
                    d2[hh] += sum2[hh].x + sum2[hh].y;
                }
                if (exact_norm) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float2 x = Elem<T>::unpack(p1[i]), y = Elem<T>::unpack(p2[i]);
                        d1r[i & 1] += x.x + x.y;
                        d2r[i & 1] += y.x + y.y;
                    }
                }
                // P buffer `buf` is free once the output products of two tiles ago have completed (in place: it
                // is this tile's own score buffer, every thread of the warp has its scores in registers, and
                // no other warp touches these rows)
                if (!kInPlace && g >= 2) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kPVDone + buf), ((g - 2) >> 1) & 1, err, 12));
                    if (!ok) break;
                }
                // two 16-bit values per column
                tmem_st_16x128b_x8(tP1(buf) + frag_base, p1);
                tmem_st_16x128b_x8(tP2(buf) + frag_base, p2);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar(L::kPFull + buf));
            }
            if (!ok) break;

            // ---- epilogue of the item, still in the fragment arrangement: every thread of a quad gets the
            // scalars of the quad's two rows, and a 4 x 4 word transpose inside the quad turns the fragment
            // columns into 16 contiguous bytes per thread, so a warp store covers 64 contiguous bytes of 8 rows
            float inv[2], bart_o[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                float s1f = d1[hh], s2f = d2[hh], r1f = d1r[hh], r2f = d2r[hh];
#pragma unroll
                for (int sh = 1; sh <= 2; sh <<= 1) {
                    s1f += __shfl_xor_sync(0xffffffffu, s1f, sh);
                    s2f += __shfl_xor_sync(0xffffffffu, s2f, sh);
                    r1f += __shfl_xor_sync(0xffffffffu, r1f, sh);
                    r2f += __shfl_xor_sync(0xffffffffu, r2f, sh);
                }
                if (!exact_norm) {
                    r1f = s1f;
                    r2f = s2f;
                }
                inv[hh] = r1f > 0.f ? 1.f / r1f : 0.f;                           // normaliser of the output
                bart_o[hh] = r2f * inv[hh];                                      // bart used for the output
                const int row = r0 + rl0 + 8 * hh;
                if (t == 0 && row < it.nq) {
                    const int64_t si = it.b * a.st_sb + it.h * a.st_sh + static_cast<int64_t>(it.bos + row) * a.st_st;
                    // the sums are relative to m_ref; the saved pair is relative to the true row maximum
                    a.d1[si] = (m_true[hh] == -INFINITY) ? 0.f : s1f * fast_exp2(m_ref[hh] - m_true[hh]);
                    a.bart[si] = s1f > 0.f ? s2f / s1f : 0.f;
                    a.m[si] = m_true[hh];
                }
            }
            // the last output products of the item
            ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kPVDone + (g - 1) % kPBufs), ((g - 1) / kPBufs) & 1, err, 11));
            if (!ok) break;
            tc_fence_after();
            const int64_t q_base = it.b * a.q_sb + it.h * a.q_sh + static_cast<int64_t>(it.bos + r0 + rl0) * a.q_st + 8 * t;
            T *go = static_cast<T *>(a.o) + q_base;
            T *gb = static_cast<T *>(a.barv) + q_base;
#pragma unroll
            for (int cc = 0; cc < D / 64; ++cc) {
                uint32_t o1[32], o2[32];
                tmem_ld_16x256b_x8(tO1 + frag_base + 64 * cc, o1);
                tmem_ld_16x256b_x8(tO2 + frag_base + 64 * cc, o2);
                tmem_wait_ld();
                if (cc == D / 64 - 1) {
                    // O1 / O2 are in registers: the next item may overwrite them
                    tc_fence_before();
                    mbar_arrive(bar(L::kOFree));
                }
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                    for (int grp = 0; grp < 2; ++grp) {
                        uint32_t wo[4], wb[4];
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const int i = 4 * (4 * grp + kk) + 2 * hh;
                            const float b0 = __uint_as_float(o1[i]) * inv[hh], b1 = __uint_as_float(o1[i + 1]) * inv[hh];
                            const float x0 = b0 + bart_o[hh] * b0 - __uint_as_float(o2[i]) * inv[hh];
                            const float x1 = b1 + bart_o[hh] * b1 - __uint_as_float(o2[i + 1]) * inv[hh];
                            wo[kk] = Elem<T>::pack(x0, x1);
                            wb[kk] = Elem<T>::pack(b0, b1);
                        }
                        quad_transpose(wo, t);
                        quad_transpose(wb, t);
                        if (r0 + rl0 + 8 * hh < it.nq) {
                            const int64_t at = static_cast<int64_t>(8 * hh) * a.q_st + 64 * cc + 32 * grp;
                            *reinterpret_cast<uint4 *>(go + at) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
                            *reinterpret_cast<uint4 *>(gb + at) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
                        }
                    }
            }
            ++n_items_done;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------- //
// host side
// ------------------------------------------------------------------------- //
using tma::make_map;
using tma::sm_count;

// Error words of the current device: the device word is a symbol of this library, its mirror one int
// of a pinned, mapped host allocation made on first use (one slot per device).
ErrorWords error_words(int **host_view = nullptr) {
    static std::mutex mu;
    static int *word[tma::kMaxDevices] = {};
    static int *mirror[tma::kMaxDevices] = {};
    static int *host_block = nullptr;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= tma::kMaxDevices) return {nullptr, nullptr};
    std::lock_guard<std::mutex> lock(mu);
    if (!word[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_sm100_error) != cudaSuccess) {
            (void)cudaGetLastError();
            return {nullptr, nullptr};
        }
        if (!host_block) {
            void *h = nullptr;
            if (cudaHostAlloc(&h, tma::kMaxDevices * sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
                (void)cudaGetLastError();
                return {nullptr, nullptr};
            }
            memset(h, 0, tma::kMaxDevices * sizeof(int));
            host_block = static_cast<int *>(h);
        }
        void *d = nullptr;
        if (cudaHostGetDevicePointer(&d, host_block + dev, 0) != cudaSuccess) {
            (void)cudaGetLastError();
            return {nullptr, nullptr};
        }
        mirror[dev] = static_cast<int *>(d);
        word[dev] = static_cast<int *>(p);
    }
    if (host_view) *host_view = host_block + dev;
    return {word[dev], mirror[dev]};
}

// the host's own pointer to the mirror of the current device (null on failure)
int *mirror_host_view() {
    int *h = nullptr;
    const ErrorWords w = error_words(&h);
    return w.word ? h : nullptr;
}

template <typename T, int D>
int launch_t(const TrainArgs &a, cudaStream_t stream) {
    constexpr int NS = 4;
    using L = Smem<D, NS>;
    const ErrorWords ew = error_words();
    if (!ew.word) return PLX_ERR_LAUNCH;
    const ErrSink sink{ew.word, ew.mirror};
    CUtensorMap tq, tr, tk, tv;
    const CUtensorMapDataType dt = Fmt<T>::kTma;
    if (!make_map(&tq, dt, a.q, D, a.len_q, a.heads_q, a.batch, a.q_st, a.q_sh, a.q_sb, kBM) ||
        !make_map(&tr, dt, a.r, D, a.len_q, a.heads_q, a.batch, a.q_st, a.q_sh, a.q_sb, kBM) ||
        !make_map(&tk, dt, a.k, D, a.len_k, a.heads_kv, a.batch, a.kv_st, a.kv_sh, a.kv_sb, kBN) ||
        !make_map(&tv, dt, a.v, D, a.len_k, a.heads_kv, a.batch, a.kv_st, a.kv_sh, a.kv_sb, kBN))
        return PLX_ERR_LAUNCH;
    auto kern = fwd_sm100_kernel<T, D, NS>;
    static std::mutex attr_mu;
    static bool attr_done[tma::kMaxDevices] = {};
    if (!tma::opt_in_smem(kern, static_cast<int>(L::kBytes), attr_done, attr_mu)) return PLX_ERR_LAUNCH;
    const int tiles = a.cu ? (a.len_q + kBM - 1) / kBM + a.n_seqs : (a.len_q + kBM - 1) / kBM;
    const int n_items = tiles * a.batch * a.heads_q, sms = sm_count();
    if (sms <= 0) return PLX_ERR_LAUNCH;
    // with plenty of items a CTA takes them in neighbouring pairs (a heavy and a light row tile)
    const int chunk_shift = n_items >= 2 * sms ? 1 : 0;
    const int units = (n_items + (1 << chunk_shift) - 1) >> chunk_shift;
    kern<<<units < sms ? units : sms, 352, L::kBytes, stream>>>(a, tq, tr, tk, tv, sink, tiles, n_items, chunk_shift);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? PLX_OK : PLX_ERR_LAUNCH;
}

}  // namespace

bool train_fwd_sm100_supported(const TrainArgs &a, int head_dim) {
    if ((head_dim != 64 && head_dim != 128) || a.window == 0 || !(a.c2 > 0.f)) return false;
    // TMA needs 16-byte aligned strides; the ABI already guarantees multiples of 8 elements
    const char *env = std::getenv("PLX_FWD_KERNEL");
    if (env && env[0] == 'm') return false;  // "mma": force the warp-level kernels
    return tma::encode_fn() != nullptr;
}

int launch_train_fwd_sm100(const TrainArgs &a, int dtype, int head_dim, cudaStream_t stream) {
    if (dtype == PLX_BF16) return head_dim == 64 ? launch_t<__nv_bfloat16, 64>(a, stream) : launch_t<__nv_bfloat16, 128>(a, stream);
    if (dtype == PLX_FP16) return head_dim == 64 ? launch_t<__half, 64>(a, stream) : launch_t<__half, 128>(a, stream);
    return PLX_ERR_UNSUPPORTED;
}

ErrorWords sm100_error_words() { return error_words(); }

// Reads (and optionally clears) the error word of the current device.  Synchronises the device.
int sm100_error_word(int *value, bool clear) {
    const ErrorWords w = error_words();
    if (!w.word) return PLX_ERR_LAUNCH;
    if (cudaMemcpy(value, w.word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return PLX_ERR_LAUNCH;
    if (clear && *value != 0) {
        const int zero = 0;
        if (cudaMemcpy(w.word, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) return PLX_ERR_LAUNCH;
        *reinterpret_cast<volatile int *>(mirror_host_view()) = 0;
    }
    return PLX_OK;
}

// The host mirror of the error word: whatever error report has reached host memory so far.  No CUDA call
// that synchronises; `clear` acknowledges the report (the device word keeps the first error until
// sm100_error_word clears it).
int sm100_error_peek(int *value, bool clear) {
    int *m = mirror_host_view();
    if (!m) return PLX_ERR_LAUNCH;
    *value = *reinterpret_cast<volatile int *>(m);
    if (clear && *value != 0) *reinterpret_cast<volatile int *>(m) = 0;
    return PLX_OK;
}

}  // namespace plx
