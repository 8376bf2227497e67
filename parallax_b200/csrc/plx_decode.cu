// Parallax single-token decode: an HBM-bound split-KV sweep over the cache.
//
// (Grouped-query shapes run the tensor-core kernel further down; this is the kernel
// of the one-q-head-per-kv-head case.)
// One warp per (split, q head, batch row); a CTA groups the warps of adjacent q
// heads.  Inside a warp the key range is dealt out to independent "streams" of D/8
// lanes: every lane owns 8 of the D channels and fetches them with one 128-bit
// load per key, so a stream reads a whole K (or V) row per load instruction and a
// warp keeps 32/(D/8) * 8 rows of K and as many of V in flight (two register buffers).  Each stream runs
// its own online softmax (m, d1, d2, O1, O2); streams are merged by shuffles,
// splits by the last warp to arrive (wait-free: an atomic counter, no spinning).
//
// Math: parallax/triton/parallax_decode.py:43-97 (per-key update and final
// out = O1/d1 * (1 + d2/d1) - O2/d1); partial-state merge:
// parallax/cute/parallax_decode.py:1107-1136.
#include <atomic>
#include <mutex>
#include <type_traits>

#include "plx_common.cuh"
#include "plx_decode.h"
#include "plx_launch.h"
#include "plx_sm100.cuh"

namespace plx {

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4 &x, float (&f)[8]) {
    float2 a = Elem<T>::unpack(x.x), b = Elem<T>::unpack(x.y), c = Elem<T>::unpack(x.z), d = Elem<T>::unpack(x.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
    f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// Combine `n` partial records (record s at rec0 + s * stride floats; layout
// m, d1, d2, pad, O1[D], O2[D]) for channel `d`.  Returns the merged
// un-normalised state of that channel.
template <int D, bool VOLATILE_READ>
__device__ __forceinline__ void merge_records(const float *rec0, int n, int64_t stride, int d, float &m_out,
                                              float &d1, float &d2, float &o1, float &o2) {
    auto rd = [](const float *p) -> float { return VOLATILE_READ ? __ldcg(p) : *p; };
    float big = -INFINITY;
    for (int s = 0; s < n; ++s) big = fmaxf(big, rd(rec0 + s * stride));
    const float safe = big == -INFINITY ? 0.f : big;
    d1 = d2 = o1 = o2 = 0.f;
    for (int s = 0; s < n; ++s) {
        const float *rec = rec0 + s * stride;
        const float w = fast_exp2(rd(rec) - safe);
        d1 += w * rd(rec + 1);
        d2 += w * rd(rec + 2);
        o1 += w * rd(rec + 4 + d);
        o2 += w * rd(rec + 4 + D + d);
    }
    m_out = big;
}

// thread-block cluster: size and rank along x, the address of a shared-memory word of another CTA of the
// cluster, a store through it, and the cluster-wide barrier
__device__ __forceinline__ uint32_t cluster_size_x() {
    uint32_t v;
    asm volatile("mov.u32 %0, %%cluster_nctaid.x;\n" : "=r"(v));
    return v;
}
__device__ __forceinline__ uint32_t cluster_rank_x() {
    uint32_t v;
    asm volatile("mov.u32 %0, %%cluster_ctaid.x;\n" : "=r"(v));
    return v;
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
    uint32_t v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(v) : "r"(smem_addr), "r"(rank));
    return v;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float x) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(x) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// Paged cache: element offset of key kj of batch row b inside k / v (head and channel offsets not
// included).  Dense caches are addressed by strides directly at the call sites.
__device__ __forceinline__ int64_t paged_key_offset(const DecodeArgs &a, int b, int kj) {
    const int page = __ldg(a.page_table + static_cast<int64_t>(b) * a.pages_per_seq + (kj >> a.page_shift));
    return page * a.kv_sb + static_cast<int64_t>(kj & a.page_mask) * a.kv_st;
}

__device__ __forceinline__ float finalize(float d1, float d2, float o1, float o2) {
    const float inv = d1 > 0.f ? 1.f / d1 : 0.f;
    return o1 * inv * (1.f + d2 * inv) - o2 * inv;
}

template <typename T>
__device__ __forceinline__ void store_elem(void *out, int64_t idx, float x);
template <>
__device__ __forceinline__ void store_elem<__nv_bfloat16>(void *out, int64_t idx, float x) {
    static_cast<__nv_bfloat16 *>(out)[idx] = __float2bfloat16_rn(x);
}
template <>
__device__ __forceinline__ void store_elem<__half>(void *out, int64_t idx, float x) {
    static_cast<__half *>(out)[idx] = __float2half_rn(x);
}

// Merge of n <= 32 partial records (stride REC floats) by one warp.  On return every lane holds the
// maximum, the two sums, and the D / 32 channels lane * (D / 32) .. of O1 and O2, all relative to
// the common maximum.
template <int D>
__device__ __forceinline__ void warp_merge(const float *rec0, int n, int lane, float &big, float &D1, float &D2,
                                           float (&O1)[D / 32], float (&O2)[D / 32]) {
    constexpr int CH = D / 32, REC = 2 * D + 4;
    float4 h = make_float4(-INFINITY, 0.f, 0.f, 0.f);
    if (lane < n) h = __ldcg(reinterpret_cast<const float4 *>(rec0 + static_cast<int64_t>(lane) * REC));
    big = h.x;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, off));
    const float safe = big == -INFINITY ? 0.f : big;
    const float wl = fast_exp2(h.x - safe);   // weight of record `lane` (0 beyond n: m = -inf there)
    D1 = wl * h.y;
    D2 = wl * h.z;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        D1 += __shfl_xor_sync(0xffffffffu, D1, off);
        D2 += __shfl_xor_sync(0xffffffffu, D2, off);
    }
#pragma unroll
    for (int e = 0; e < CH; ++e) O1[e] = O2[e] = 0.f;
    const float *col = rec0 + 4 + lane * CH;
#pragma unroll
    for (int j0 = 0; j0 < 32; j0 += 8) {
        if (j0 >= n) break;
        float x[8][CH], y[8][CH], w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            w[j] = __shfl_sync(0xffffffffu, wl, j0 + j);
            const float *pr = col + static_cast<int64_t>(min(j0 + j, n - 1)) * REC;   // weight 0 past the end
            if (CH == 4) {
                const float4 u = __ldcg(reinterpret_cast<const float4 *>(pr)), v = __ldcg(reinterpret_cast<const float4 *>(pr + D));
                x[j][0] = u.x; x[j][1] = u.y; x[j][CH - 2] = u.z; x[j][CH - 1] = u.w;
                y[j][0] = v.x; y[j][1] = v.y; y[j][CH - 2] = v.z; y[j][CH - 1] = v.w;
            } else {
                const float2 u = __ldcg(reinterpret_cast<const float2 *>(pr)), v = __ldcg(reinterpret_cast<const float2 *>(pr + D));
                x[j][0] = u.x; x[j][1] = u.y;
                y[j][0] = v.x; y[j][1] = v.y;
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < CH; ++e) {
                O1[e] = fmaf(w[j], x[j][e], O1[e]);
                O2[e] = fmaf(w[j], y[j][e], O2[e]);
            }
    }
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}

// Inbox layout of the peer-memory exchange (see decode_exchange_merge_kernel below): record slots
// [2 parities][world][n_records], then as many 32-bit stamps, then [n_records] step counters.
struct InboxView {
    int world, n_records, rec;      // rec = floats per record
    __device__ __forceinline__ size_t rec_floats() const { return static_cast<size_t>(2) * world * n_records * rec; }
    __device__ __forceinline__ float *slot(float *inbox, uint32_t parity, int src, int64_t i) const {
        return inbox + ((static_cast<size_t>(parity) * world + src) * n_records + i) * rec;
    }
    __device__ __forceinline__ uint32_t *stamp(float *inbox, uint32_t parity, int src, int64_t i) const {
        return reinterpret_cast<uint32_t *>(inbox + rec_floats()) + (static_cast<size_t>(parity) * world + src) * n_records + i;
    }
    __device__ __forceinline__ uint32_t *epoch(float *inbox, int64_t i) const {
        return reinterpret_cast<uint32_t *>(inbox + rec_floats()) + static_cast<size_t>(2) * world * n_records + i;
    }
};

// Sweep and exchange in ONE kernel.  The warp that holds the merged state of (batch, head) `bh` -- every
// lane the maximum, the two sums and D / 32 channels of O1 and O2 -- pushes it as record bh into every
// rank's inbox (plain stores over NVLink, then a release-stamp per peer), waits, bounded, for the stamps
// of record bh from the other ranks, merges the `world` records and writes row bh of `out`.  The protocol
// is that of decode_exchange_merge_kernel, and the merge is the same per-channel arithmetic, so the
// result is bit-identical to partial sweep + that kernel.  The waiting warp keeps its CTA resident; it
// waits only for warps of OTHER GPUs, which wait for nothing of this GPU's launch.
template <typename T, int D>
__device__ __forceinline__ void exchange_merge_warp(const DecodeArgs &a, int64_t bh, int lane, float big, float D1, float D2,
                                                    const float (&O1)[D / 32], const float (&O2)[D / 32]) {
    constexpr int REC = 2 * D + 4, CH = D / 32;
    const ExchangeArgs &x = a.xch;
    const InboxView iv{x.world, x.n_records, REC};
    uint32_t epoch = 0;
    if (lane == 0) epoch = *iv.epoch(x.inbox[x.rank], bh);
    epoch = __shfl_sync(0xffffffffu, epoch, 0);
    const uint32_t parity = epoch & 1u, stamp = epoch + 1u;
    // (1) push this rank's record to every rank (own inbox included)
    for (int p = 0; p < x.world; ++p) {
        float *dst = iv.slot(x.inbox[p], parity, x.rank, bh);
        if (lane == 0) *reinterpret_cast<float4 *>(dst) = make_float4(big, D1, D2, 0.f);
#pragma unroll
        for (int e = 0; e < CH; ++e) {
            dst[4 + lane * CH + e] = O1[e];
            dst[4 + D + lane * CH + e] = O2[e];
        }
    }
    __threadfence_system();
    __syncwarp();
    if (lane < x.world && lane != x.rank) {
        uint32_t *f = iv.stamp(x.inbox[lane], parity, x.rank, bh);
        asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(f), "r"(stamp) : "memory");
    }
    // (2) wait for record bh of every other rank
    int bad = 0;
    if (lane < x.world && lane != x.rank) {
        const uint32_t *f = iv.stamp(x.inbox[x.rank], parity, lane, bh);
        const uint64_t t0 = global_timer_ns(), limit = static_cast<uint64_t>(x.wait_ms) * 1000000ull;
        uint32_t seen;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(f) : "memory");
            if (seen == stamp) break;
            if (global_timer_ns() - t0 > limit) {
                sm100::report_error(sm100::ErrSink{x.err_word, x.err_mirror}, ((40 + lane) << 8) | 1);   // source rank never delivered
                if (x.status) atomicOr(x.status, 1 << lane);
                bad = 1;
                break;
            }
        }
    }
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) *iv.epoch(x.inbox[x.rank], bh) = epoch + 1u;   // also after a time-out: the ranks stay in step
    // (3) merge and finalise this lane's channels (NaN when a record is missing)
    const float *rec0 = iv.slot(x.inbox[x.rank], parity, 0, bh);
#pragma unroll
    for (int e = 0; e < CH; ++e) {
        float M, S1, S2, A1, A2, y = __int_as_float(0x7fc00000);
        if (!bad) {
            merge_records<D, true>(rec0, x.world, static_cast<int64_t>(x.n_records) * REC, lane * CH + e, M, S1, S2, A1, A2);
            y = finalize(S1, S2, A1, A2);
        }
        store_elem<T>(a.out, bh * D + lane * CH + e, y);
    }
}

// One WARP per (split, q head, batch row); a CTA is HG warps working on HG adjacent q
// heads of the same key range, so that together they sweep contiguous memory (all heads
// of a key are adjacent in the cache layout) and, under grouped-query attention, the q
// heads of a group find the shared K / V rows in L1.  Warps never synchronise with each
// other: streams are merged by shuffles, splits by the last warp to arrive.
//
// SG ("split group") is the arrangement for launches with few (batch, head) pairs, which are bound by
// latency, not bandwidth: a CTA is the HG = 8 warps of eight ADJACENT SPLITS of one q head.  Every
// warp still sweeps its own keys, but the eight partial states meet in shared memory, so only one
// record per CTA goes through global memory, and the CTA that arrives last merges the (at most 32) CTA
// records with all 256 threads at once -- one round trip to L2 where a single merging warp needs one
// per eight records.  That allows splits of ~16 keys, whose loads are all in flight together.
template <typename T, int D, int HG, int U, bool GQA, bool SG>
__global__ void __launch_bounds__(HG * 32, U > 4 ? 1 : 512 / (HG * 32)) decode_kernel(const DecodeArgs a) {
    constexpr int LPK = D / 8;      // lanes per key row
    constexpr int NS = 32 / LPK;    // streams per warp
    constexpr int REC = 2 * D + 4;  // floats per partial record
    constexpr int CH = D / 32;      // channels per lane in the merge

    const int b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = SG ? blockIdx.x * HG + warp : blockIdx.x;
    const int hq = SG ? blockIdx.y : blockIdx.y * HG + warp;
    const int hk = hq / a.n_rep;
    const int sid = lane / LPK, sl = lane % LPK;

    // active key range of this batch row, then of this split (local key indices)
    int hi_g = a.total_len;
    if (a.seqused) hi_g = min(max(a.seqused[b], 1), a.total_len);
    int lo_g = a.cache_start ? max(a.cache_start[b], 0) : 0;
    if (a.window >= 0) lo_g = max(lo_g, hi_g - a.window);
    const int lo = min(max(lo_g - a.kv_offset, 0), a.cache_len);
    const int hi = min(max(hi_g - a.kv_offset, 0), a.cache_len);
    const int n = max(hi - lo, 0);
    int chunk = (n + a.n_splits - 1) / a.n_splits;
    chunk = (chunk + NS - 1) / NS * NS;
    const int my_lo = min(lo + split * chunk, hi);
    const int my_hi = min(my_lo + chunk, hi);
    const int n_iter = (my_hi - my_lo + NS * U - 1) / (NS * U);

    // this lane's 8 channels of q and r
    float qf[8], rf[8];
    {
        const int64_t qi = (static_cast<int64_t>(b) * a.heads_q + hq) * D + sl * 8;
        unpack8<T>(*reinterpret_cast<const uint4 *>(static_cast<const T *>(a.q) + qi), qf);
        unpack8<T>(*reinterpret_cast<const uint4 *>(static_cast<const T *>(a.r) + qi), rf);
    }
    const bool paged = a.page_table != nullptr;      // uniform over the launch
    const int64_t row0 = (paged ? 0 : b * a.kv_sb) + hk * a.kv_sh + sl * 8;
    const T *kp = static_cast<const T *>(a.k) + row0;
    const T *vp = static_cast<const T *>(a.v) + row0;

    float m = -INFINITY, d1 = 0.f, d2 = 0.f, o1[8], o2[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o1[e] = o2[e] = 0.f;

    // rows of iteration `it` -> registers (keys past the range read nothing and count as masked)
    // (the first argument is a compile-time tag: std::true_type for a paged cache.  The dense sweep must
    // not carry the page-table branch inside its unrolled loads -- that cost 4 to 12 % of the bandwidth.)
    auto load = [&](auto paged_tag, int it, uint4 (&kr)[U], uint4 (&vr)[U]) {
        const int base = my_lo + it * NS * U + sid;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kj = base + u * NS;
            if (kj < my_hi) {
                const int64_t at = decltype(paged_tag)::value ? paged_key_offset(a, b, kj) : static_cast<int64_t>(kj) * a.kv_st;
                const T *pk = kp + at, *pv = vp + at;
                kr[u] = GQA ? __ldg(reinterpret_cast<const uint4 *>(pk)) : ld_stream16(pk);
                vr[u] = GQA ? __ldg(reinterpret_cast<const uint4 *>(pv)) : ld_stream16(pv);
            } else {
                kr[u] = make_uint4(0u, 0u, 0u, 0u);
                vr[u] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    auto compute = [&](int it, const uint4 (&kr)[U], const uint4 (&vr)[U]) {
        const int base = my_lo + it * NS * U + sid;
        float s1[U], s2[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float kf[8];
            unpack8<T>(kr[u], kf);
            float x = 0.f, y = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                x = fmaf(qf[e], kf[e], x);
                y = fmaf(rf[e], kf[e], y);
            }
            s1[u] = x;
            s2[u] = y;
        }
#pragma unroll
        for (int off = LPK / 2; off > 0; off >>= 1)
#pragma unroll
            for (int u = 0; u < U; ++u) {
                s1[u] += __shfl_xor_sync(0xffffffffu, s1[u], off);
                s2[u] += __shfl_xor_sync(0xffffffffu, s2[u], off);
            }
        float cmax = -INFINITY;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            s1[u] = (base + u * NS < my_hi) ? s1[u] * a.c2 : -INFINITY;
            cmax = fmaxf(cmax, s1[u]);
        }
        const float m_new = fmaxf(m, cmax);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = fast_exp2(m - m_safe);
        m = m_new;
        d1 *= alpha;
        d2 *= alpha;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            o1[e] *= alpha;
            o2[e] *= alpha;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const float p1 = fast_exp2(s1[u] - m_safe);
            const float p2 = p1 * s2[u];
            d1 += p1;
            d2 += p2;
            float vf[8];
            unpack8<T>(vr[u], vf);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                o1[e] = fmaf(p1, vf[e], o1[e]);
                o2[e] = fmaf(p2, vf[e], o2[e]);
            }
        }
    };
    // two register buffers: the rows of the next iteration are in flight while this one is reduced
    auto sweep = [&](auto paged_tag) {
        uint4 ka[U], va[U], kb[U], vb[U];
        if (n_iter > 0) load(paged_tag, 0, ka, va);
        for (int it = 0; it < n_iter; it += 2) {
            if (it + 1 < n_iter) load(paged_tag, it + 1, kb, vb);
            compute(it, ka, va);
            if (it + 1 < n_iter) {
                if (it + 2 < n_iter) load(paged_tag, it + 2, ka, va);
                compute(it + 1, kb, vb);
            }
        }
    };
    if (paged) sweep(std::true_type{});
    else sweep(std::false_type{});

    // merge the warp's streams (lanes that differ in bits >= log2(LPK) hold the same channels)
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1) {
        const float m_o = __shfl_xor_sync(0xffffffffu, m, off);
        const float big = fmaxf(m, m_o);
        const float safe = big == -INFINITY ? 0.f : big;
        const float wa = fast_exp2(m - safe), wb = fast_exp2(m_o - safe);
        d1 = wa * d1 + wb * __shfl_xor_sync(0xffffffffu, d1, off);
        d2 = wa * d2 + wb * __shfl_xor_sync(0xffffffffu, d2, off);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            o1[e] = wa * o1[e] + wb * __shfl_xor_sync(0xffffffffu, o1[e], off);
            o2[e] = wa * o2[e] + wb * __shfl_xor_sync(0xffffffffu, o2[e], off);
        }
        m = big;
    }
    // every lane now holds the warp's state for channels sl * 8 .. sl * 8 + 7; lanes < LPK write
    const int64_t bh = static_cast<int64_t>(b) * a.heads_q + hq;
    const bool writer = lane < LPK;

    auto emit = [&](float M, float D1, float D2, const float (&O1)[8], const float (&O2)[8]) {
        if (!writer) return;
        if (a.part_out) {
            float *rec = a.part_out + bh * REC;
            if (lane == 0) {
                rec[0] = M;
                rec[1] = D1;
                rec[2] = D2;
                rec[3] = 0.f;
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                rec[4 + sl * 8 + e] = O1[e];
                rec[4 + D + sl * 8 + e] = O2[e];
            }
        } else {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
                pk[e] = Elem<T>::pack(finalize(D1, D2, O1[2 * e], O2[2 * e]), finalize(D1, D2, O1[2 * e + 1], O2[2 * e + 1]));
            *reinterpret_cast<uint4 *>(static_cast<T *>(a.out) + bh * D + sl * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    };

    if constexpr (SG) {
        // ---- the eight splits of this CTA meet in shared memory
        static_assert(HG == 8, "a split group is eight warps");
        __shared__ __align__(16) float s_rec[HG][REC];
        __shared__ int s_last;
        if (writer) {
            if (lane == 0) *reinterpret_cast<float4 *>(&s_rec[warp][0]) = make_float4(m, d1, d2, 0.f);
#pragma unroll
            for (int e = 0; e < 8; e += 4) {
                *reinterpret_cast<float4 *>(&s_rec[warp][4 + sl * 8 + e]) = make_float4(o1[e], o1[e + 1], o1[e + 2], o1[e + 3]);
                *reinterpret_cast<float4 *>(&s_rec[warp][4 + D + sl * 8 + e]) = make_float4(o2[e], o2[e + 1], o2[e + 2], o2[e + 3]);
            }
        }
        __syncthreads();
        // thread c < 2 D owns element c of the concatenated [O1 | O2] from here on
        const int c = threadIdx.x;
        const bool active = c < 2 * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < HG; ++w) M = fmaxf(M, s_rec[w][0]);
        const float safe = M == -INFINITY ? 0.f : M;
        float S1 = 0.f, S2 = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < HG; ++w) {
            const float wt = fast_exp2(s_rec[w][0] - safe);
            S1 = fmaf(wt, s_rec[w][1], S1);
            S2 = fmaf(wt, s_rec[w][2], S2);
            if (active) A = fmaf(wt, s_rec[w][4 + c], A);
        }
        const int n_cta = gridDim.x;
        if (n_cta > 1 && cluster_size_x() == static_cast<uint32_t>(n_cta)) {
            // All CTAs of this (batch, head) form one thread-block cluster: the CTA records meet in the
            // shared memory of the cluster's first CTA (stores through distributed shared memory, one
            // cluster barrier) and never touch global memory -- no publish / fence / atomic / re-read.
            __shared__ __align__(16) float s_crec[8][REC];
            const uint32_t rank = cluster_rank_x();
            const uint32_t dst = cluster_map(smem_u32(&s_crec[rank][0]), 0);
            if (c == 0) {
                st_cluster_f32(dst, M);
                st_cluster_f32(dst + 4, S1);
                st_cluster_f32(dst + 8, S2);
            }
            if (active) st_cluster_f32(dst + 4u * (4 + c), A);
            cluster_sync();
            if (rank != 0) return;
            M = -INFINITY;
            for (int j = 0; j < n_cta; ++j) M = fmaxf(M, s_crec[j][0]);
            const float safe2 = M == -INFINITY ? 0.f : M;
            S1 = S2 = A = 0.f;
            for (int j = 0; j < n_cta; ++j) {
                const float wt = fast_exp2(s_crec[j][0] - safe2);
                S1 = fmaf(wt, s_crec[j][1], S1);
                S2 = fmaf(wt, s_crec[j][2], S2);
                if (active) A = fmaf(wt, s_crec[j][4 + c], A);
            }
        } else if (n_cta > 1) {
            // one record per CTA through global memory; the last CTA of the (batch, head) merges them
            float *rec = a.ws_parts + (bh * n_cta + blockIdx.x) * REC;
            if (c == 0) __stcg(reinterpret_cast<float4 *>(rec), make_float4(M, S1, S2, 0.f));
            if (active) __stcg(rec + 4 + c, A);
            __threadfence();
            __syncthreads();
            if (c == 0) s_last = atomicAdd(a.ws_counters + bh, 1) == n_cta - 1;
            __syncthreads();
            if (!s_last) return;
            __threadfence();
            const float *rec0 = a.ws_parts + bh * n_cta * REC;
            // all loads of all records in flight at once (n_cta <= 32): thread c its element of every
            // record, thread j < n_cta the header of record j, which then goes round through shared memory
            float x[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = (j < n_cta && active) ? __ldcg(rec0 + static_cast<int64_t>(j) * REC + 4 + c) : 0.f;
            float4 *s_head = reinterpret_cast<float4 *>(&s_rec[0][0]);     // the CTA's own records are spent
            if (c < 32)
                s_head[c] = c < n_cta ? __ldcg(reinterpret_cast<const float4 *>(rec0 + static_cast<int64_t>(c) * REC))
                                      : make_float4(-INFINITY, 0.f, 0.f, 0.f);
            __syncthreads();
            M = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; ++j) M = fmaxf(M, s_head[j].x);
            const float safe2 = M == -INFINITY ? 0.f : M;
            S1 = S2 = A = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float4 h = s_head[j];
                const float wt = fast_exp2(h.x - safe2);
                S1 = fmaf(wt, h.y, S1);
                S2 = fmaf(wt, h.z, S2);
                A = fmaf(wt, x[j], A);
            }
            if (c == 0) a.ws_counters[bh] = 0;  // ready for the next launch on this workspace
        }
        if (a.part_out) {
            float *rec = a.part_out + bh * REC;
            if (c == 0) *reinterpret_cast<float4 *>(rec) = make_float4(M, S1, S2, 0.f);
            if (active) rec[4 + c] = A;
        } else {
            // O1 and O2 of a channel sit in two threads: pair them up through shared memory
            float *s_out = &s_rec[2][0];
            __syncthreads();                 // everybody has read the headers / the CTA's records
            if (active) s_out[c] = A;
            __syncthreads();
            if (c < D) store_elem<T>(a.out, bh * D + c, finalize(S1, S2, s_out[c], s_out[D + c]));
        }
        return;
    }

    if (a.n_splits == 1) {
        emit(m, d1, d2, o1, o2);
        return;
    }

    // publish this split's state; the last warp of the (batch, head) to arrive merges all splits
    float *ws = a.ws_parts + (bh * a.n_splits + split) * REC;
    if (writer) {
        if (lane == 0) __stcg(reinterpret_cast<float4 *>(ws), make_float4(m, d1, d2, 0.f));
        __stcg(reinterpret_cast<float4 *>(ws + 4 + sl * 8), make_float4(o1[0], o1[1], o1[2], o1[3]));
        __stcg(reinterpret_cast<float4 *>(ws + 4 + sl * 8 + 4), make_float4(o1[4], o1[5], o1[6], o1[7]));
        __stcg(reinterpret_cast<float4 *>(ws + 4 + D + sl * 8), make_float4(o2[0], o2[1], o2[2], o2[3]));
        __stcg(reinterpret_cast<float4 *>(ws + 4 + D + sl * 8 + 4), make_float4(o2[4], o2[5], o2[6], o2[7]));
    }
    __threadfence();
    __syncwarp();

    // The merge is a chain of dependent L2 round trips if done record by record, and for small
    // batches it is most of the launch.  So the 32 lanes read the {m, d1, d2} headers of up to 32
    // records at once and reduce the maximum and the two sums with shuffles; for the O1 / O2 rows
    // every lane owns D / 32 channels and the loads of eight records are in flight together.  More
    // than 32 splits are merged in two levels, so that no warp walks more than 16 records.
    float big, D1, D2, O1[CH], O2[CH];
    auto arrive_last = [&](int *counter, int expected) -> bool {
        int last = 0;
        if (lane == 0) last = (atomicAdd(counter, 1) == expected - 1);
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) __threadfence();
        return last != 0;
    };
    if (a.n_groups == 0) {
        if (!arrive_last(a.ws_counters + bh, a.n_splits)) return;
        warp_merge<D>(a.ws_parts + bh * a.n_splits * REC, a.n_splits, lane, big, D1, D2, O1, O2);
    } else {
        const int group = split / PLX_DECODE_GROUP;
        const int first = group * PLX_DECODE_GROUP, size = min(PLX_DECODE_GROUP, a.n_splits - first);
        int *gc = a.ws_gcounters + bh * a.n_groups + group;
        if (!arrive_last(gc, size)) return;
        warp_merge<D>(a.ws_parts + (bh * a.n_splits + first) * REC, size, lane, big, D1, D2, O1, O2);
        float *grec = a.ws_gparts + (bh * a.n_groups + group) * REC;
        if (lane == 0) {
            __stcg(reinterpret_cast<float4 *>(grec), make_float4(big, D1, D2, 0.f));
            *gc = 0;   // ready for the next launch on this workspace
        }
#pragma unroll
        for (int e = 0; e < CH; ++e) {
            __stcg(grec + 4 + lane * CH + e, O1[e]);
            __stcg(grec + 4 + D + lane * CH + e, O2[e]);
        }
        __threadfence();
        __syncwarp();
        if (!arrive_last(a.ws_counters + bh, a.n_groups)) return;
        warp_merge<D>(a.ws_gparts + bh * a.n_groups * REC, a.n_groups, lane, big, D1, D2, O1, O2);
    }
    if (a.xch.world > 0) {
        exchange_merge_warp<T, D>(a, bh, lane, big, D1, D2, O1, O2);
    } else if (a.part_out) {
        float *rec = a.part_out + bh * REC;
        if (lane == 0) *reinterpret_cast<float4 *>(rec) = make_float4(big, D1, D2, 0.f);
#pragma unroll
        for (int e = 0; e < CH; ++e) {
            rec[4 + lane * CH + e] = O1[e];
            rec[4 + D + lane * CH + e] = O2[e];
        }
    } else {
        T *dst = static_cast<T *>(a.out) + bh * D + lane * CH;
        const uint32_t p0 = Elem<T>::pack(finalize(D1, D2, O1[0], O2[0]), finalize(D1, D2, O1[1], O2[1]));
        if (CH == 4) {
            const uint32_t p1 = Elem<T>::pack(finalize(D1, D2, O1[CH - 2], O2[CH - 2]), finalize(D1, D2, O1[CH - 1], O2[CH - 1]));
            *reinterpret_cast<uint2 *>(dst) = make_uint2(p0, p1);
        } else {
            *reinterpret_cast<uint32_t *>(dst) = p0;
        }
    }
    if (lane == 0) a.ws_counters[bh] = 0;  // ready for the next launch on this workspace
}

// n_parts arrays of n_records records each -> out
template <typename T, int D>
__global__ void __launch_bounds__(D) decode_merge_kernel(const float *parts, int n_parts, int n_records, void *out) {
    constexpr int REC = 2 * D + 4;
    const int i = blockIdx.x, d = threadIdx.x;
    float M, D1, D2, O1, O2;
    merge_records<D, false>(parts + static_cast<int64_t>(i) * REC, n_parts, static_cast<int64_t>(n_records) * REC, d, M,
                            D1, D2, O1, O2);
    store_elem<T>(out, static_cast<int64_t>(i) * D + d, finalize(D1, D2, O1, O2));
}

// ========================================================================= //
// Exchange + merge of the per-rank partial states of a KV-sharded decode, in one kernel over peer
// memory (NVLink loads / stores; no TMA, no multicast): instead of an all-gather followed by a
// merge kernel.
//
// Every rank owns an "inbox" that all ranks have mapped: [2 parities][world][n_records] records,
// then [2][world][n_records] 32-bit stamps, then [n_records] step counters (read only by their owner).  CTA i of rank g (1) stores record i of its partial
// array into slot (parity, g, i) of EVERY rank's inbox and then, after a system-wide fence, the
// stamp (step + 1) beside it; (2) waits -- bounded -- until its own inbox holds the stamps of record i
// from every other rank, and merges the `world` records into out[i].  A CTA waits only for CTAs of the
// same index on OTHER GPUs, which depend on nothing, so no CTA of a grid ever waits for another CTA
// of the same grid.  Two parities: a rank cannot start step e + 2 before every peer has finished
// merging step e (it needs their records of step e + 1, which they send after that merge).
//
// The wait is bounded (x.wait_ms).  A CTA whose wait runs out sets bit `src` of the caller's status
// word, reports (40 + src) through the error words, and writes NaN into its row of `out`, so that a
// result built on a missing record cannot pass for a number; the step counter advances all the same,
// which keeps the ranks in step for the next call.
// ========================================================================= //

template <typename T, int D>
__global__ void __launch_bounds__(D) decode_exchange_merge_kernel(const ExchangeArgs x, const float *part, void *out,
                                                                  const sm100::ErrSink err) {
    constexpr int REC = 2 * D + 4;
    const int i = blockIdx.x, d = threadIdx.x;
    const size_t rec_floats = static_cast<size_t>(2) * x.world * x.n_records * REC;
    // the step counter of record i lives beside this rank's stamps (so a captured launch can be replayed)
    uint32_t *my_epoch = reinterpret_cast<uint32_t *>(x.inbox[x.rank] + rec_floats) + static_cast<size_t>(2) * x.world * x.n_records + i;
    const uint32_t epoch = *my_epoch;
    const uint32_t parity = epoch & 1u, stamp = epoch + 1u;
    auto slot = [&](float *inbox, int src) -> float * {
        return inbox + ((static_cast<size_t>(parity) * x.world + src) * x.n_records + i) * REC;
    };
    auto stamp_of = [&](float *inbox, int src) -> uint32_t * {
        return reinterpret_cast<uint32_t *>(inbox + rec_floats) + (static_cast<size_t>(parity) * x.world + src) * x.n_records + i;
    };
    // (1) push record i to every rank (own inbox included)
    const float *mine = part + static_cast<size_t>(i) * REC;
    for (int p = 0; p < x.world; ++p) {
        float *dst = slot(x.inbox[p], x.rank);
        for (int c = d; c < REC; c += D) dst[c] = mine[c];
    }
    __threadfence_system();
    __syncthreads();
    if (d < x.world && d != x.rank) {
        uint32_t *f = stamp_of(x.inbox[d], x.rank);
        asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(f), "r"(stamp) : "memory");
    }
    // (2) wait for record i of every other rank, then merge
    __shared__ int s_bad;
    if (d == 0) s_bad = 0;
    __syncthreads();
    if (d < x.world && d != x.rank) {
        const uint32_t *f = stamp_of(x.inbox[x.rank], d);
        const uint64_t t0 = global_timer_ns(), limit = static_cast<uint64_t>(x.wait_ms) * 1000000ull;
        uint32_t seen;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(f) : "memory");
            if (seen == stamp) break;
            if (global_timer_ns() - t0 > limit) {
                sm100::report_error(err, ((40 + d) << 8) | 1);   // source rank d never delivered
                if (x.status) atomicOr(x.status, 1 << d);
                s_bad = 1;
                break;
            }
        }
    }
    __syncthreads();
    if (d == 0) *my_epoch = epoch + 1u;   // also after a time-out: the ranks stay in step
    if (s_bad) {
        store_elem<T>(out, static_cast<int64_t>(i) * D + d, __int_as_float(0x7fc00000));   // NaN: this row has no answer
        return;
    }
    float M, D1, D2, O1, O2;
    merge_records<D, true>(slot(x.inbox[x.rank], 0), x.world, static_cast<int64_t>(x.n_records) * REC, d, M, D1, D2, O1, O2);
    store_elem<T>(out, static_cast<int64_t>(i) * D + d, finalize(D1, D2, O1, O2));
}

template <typename T, int D>
static int launch_exchange_t(const ExchangeArgs &x, const float *part, void *out, const ErrorWords &ew, cudaStream_t stream) {
    decode_exchange_merge_kernel<T, D><<<x.n_records, D, 0, stream>>>(x, part, out, sm100::ErrSink{ew.word, ew.mirror});
    count_launch();
    return cudaGetLastError() == cudaSuccess ? PLX_OK : PLX_ERR_LAUNCH;
}

int launch_decode_exchange_merge(const ExchangeArgs &x, const float *part, int head_dim, int dtype, void *out,
                                 const ErrorWords &err, cudaStream_t stream) {
    if (dtype == PLX_BF16) {
        if (head_dim == 128) return launch_exchange_t<__nv_bfloat16, 128>(x, part, out, err, stream);
        if (head_dim == 64) return launch_exchange_t<__nv_bfloat16, 64>(x, part, out, err, stream);
    } else if (dtype == PLX_FP16) {
        if (head_dim == 128) return launch_exchange_t<__half, 128>(x, part, out, err, stream);
        if (head_dim == 64) return launch_exchange_t<__half, 64>(x, part, out, err, stream);
    }
    return PLX_ERR_UNSUPPORTED;
}

// ========================================================================= //
// Grouped-query decode on the warp-level tensor cores.
//
// With n_rep q heads per kv head, the per-key arithmetic of the kernel above grows n_rep-fold
// while the bytes stay the same: from n_rep = 4 on it is bound by the FMA pipe, not by HBM.  Here
// the q heads of a group are the M dimension of m16n8k16 MMAs (up to 16 rows, zero-padded), so
// K and V are read once per group and the arithmetic moves to the tensor cores.
//
// One warp per (split, kv head [x 16-row head group], batch row).  The warp stages 16-key tiles of
// K and V in its own shared memory (16-byte cp.async, kGqaStages deep, rows padded to D + 8
// elements; one bulk copy per row measured 1.6x slower: 32 small copies per tile queue up),
// forms S1 = Q_g K^T and S2 = R_g K^T, runs the online softmax per row in the accumulator
// fragments, and accumulates O1 += P1 V, O2 += P2 V with the P fragments as the A operand.  Warps
// never synchronise with each other; splits are merged as above.
// ========================================================================= //
constexpr int kGqaTile = 16;     // keys per staged tile
constexpr int kGqaStages = 3;
constexpr int kGqaWarps = kDecodeGqaWarps;   // warps (independent splits) per CTA

template <int D>
struct GqaSmem {
    static constexpr int kPerWarp = kGqaStages * 2 * kGqaTile * (D + 8) * 2;   // K and V tiles, 16-bit elements
};

template <typename T, int D>
__global__ void __launch_bounds__(kGqaWarps * 32, 1) decode_gqa_kernel(const DecodeArgs a, int n_hgroups) {
    constexpr int LD = D + 8;                       // padded row: ldmatrix without bank conflicts
    constexpr int REC = 2 * D + 4, CH = D / 32;
    constexpr int KS = D / 16;                      // k-steps of the score products
    constexpr uint32_t kTileBytes = kGqaTile * LD * 2;
    constexpr int CPR = D / 8;                      // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char gqa_smem[];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // warps are dealt out split-fastest over (batch, kv head, head group, split), so a CTA is full whatever the split count
    const int64_t wid = static_cast<int64_t>(blockIdx.x) * kGqaWarps + warp;
    const int64_t n_units = static_cast<int64_t>(a.batch) * a.heads_kv * n_hgroups;
    if (wid >= n_units * a.n_splits) return;
    const int split = static_cast<int>(wid % a.n_splits);
    const int unit = static_cast<int>(wid / a.n_splits);
    const int b = unit / (a.heads_kv * n_hgroups), hk = (unit / n_hgroups) % a.heads_kv, hgrp = unit % n_hgroups;
    const int hq0 = hk * a.n_rep + hgrp * 16;       // first q head of this warp's rows
    const int n_rows = min(16, a.n_rep - hgrp * 16);
    const uint32_t sbase = smem_u32(gqa_smem) + warp * GqaSmem<D>::kPerWarp;
    auto sK = [&](int st) -> uint32_t { return sbase + st * 2 * kTileBytes; };
    auto sV = [&](int st) -> uint32_t { return sbase + st * 2 * kTileBytes + kTileBytes; };

    // active key range of this batch row, then of this split (local key indices)
    int hi_g = a.total_len;
    if (a.seqused) hi_g = min(max(a.seqused[b], 1), a.total_len);
    int lo_g = a.cache_start ? max(a.cache_start[b], 0) : 0;
    if (a.window >= 0) lo_g = max(lo_g, hi_g - a.window);
    const int lo = min(max(lo_g - a.kv_offset, 0), a.cache_len);
    const int hi = min(max(hi_g - a.kv_offset, 0), a.cache_len);
    const int n = max(hi - lo, 0);
    int chunk = (n + a.n_splits - 1) / a.n_splits;
    chunk = (chunk + kGqaTile - 1) / kGqaTile * kGqaTile;
    const int my_lo = min(lo + split * chunk, hi);
    const int my_hi = min(my_lo + chunk, hi);
    const int n_tiles = (my_hi - my_lo + kGqaTile - 1) / kGqaTile;

    // ---- q and r of the group -> A fragments (staged through the first two tile buffers)
    uint32_t qa[KS][4], ra[KS][4];
    {
        const T *qg = static_cast<const T *>(a.q) + (static_cast<int64_t>(b) * a.heads_q + hq0) * D;
        const T *rg = static_cast<const T *>(a.r) + (static_cast<int64_t>(b) * a.heads_q + hq0) * D;
#pragma unroll
        for (int c = lane; c < 16 * CPR; c += 32) {
            const int row = c / CPR, col = c % CPR;
            const int bytes = row < n_rows ? 16 : 0;                      // rows past the group: zeros
            const int64_t at = static_cast<int64_t>(row < n_rows ? row : 0) * D + col * 8;
            cp_async16(sK(0) + (row * LD + col * 8) * 2, qg + at, bytes);
            cp_async16(sV(0) + (row * LD + col * 8) * 2, rg + at, bytes);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncwarp();
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            ldsm_x4(qa[ks], a_addr<LD>(sK(0), 0, ks * 16, lane));
            ldsm_x4(ra[ks], a_addr<LD>(sV(0), 0, ks * 16, lane));
        }
        __syncwarp();
    }

    // Tile i of this warp -> stage i % kGqaStages.  A lane copies the same 16-byte column of every
    // (32 / CPR)-th row, so its source and destination advance by constants; rows past my_hi (last tile
    // only) are zero-filled.
    constexpr int RPI = 32 / CPR;                                  // rows covered by one instruction of the warp
    const int my_row = lane / CPR, my_col = lane % CPR;
    const bool paged = a.page_table != nullptr;      // uniform over the launch
    const T *kp = static_cast<const T *>(a.k) + (paged ? 0 : b * a.kv_sb) + hk * a.kv_sh + my_col * 8;
    const T *vp = static_cast<const T *>(a.v) + (paged ? 0 : b * a.kv_sb) + hk * a.kv_sh + my_col * 8;
    const uint32_t my_dst = (my_row * LD + my_col * 8) * 2;
    auto load_tile = [&](int i) {
        if (i < n_tiles) {
            const int st = i % kGqaStages, key0 = my_lo + i * kGqaTile + my_row;
            const uint32_t dk = sK(st) + my_dst, dv = sV(st) + my_dst;
            const bool whole = key0 - my_row + kGqaTile <= my_hi;
            if (!paged) {
                const int64_t at = static_cast<int64_t>(key0) * a.kv_st, step = static_cast<int64_t>(RPI) * a.kv_st;
                if (whole) {
#pragma unroll
                    for (int j = 0; j < kGqaTile / RPI; ++j) {
                        cp_async16(dk + j * RPI * LD * 2, kp + at + j * step, 16);
                        cp_async16(dv + j * RPI * LD * 2, vp + at + j * step, 16);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < kGqaTile / RPI; ++j) {
                        const bool in = key0 + j * RPI < my_hi;
                        cp_async16(dk + j * RPI * LD * 2, kp + (in ? at + j * step : 0), in ? 16 : 0);
                        cp_async16(dv + j * RPI * LD * 2, vp + (in ? at + j * step : 0), in ? 16 : 0);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < kGqaTile / RPI; ++j) {
                    const bool in = whole || key0 + j * RPI < my_hi;
                    const int64_t at = in ? paged_key_offset(a, b, key0 + j * RPI) : 0;
                    cp_async16(dk + j * RPI * LD * 2, kp + at, in ? 16 : 0);
                    cp_async16(dv + j * RPI * LD * 2, vp + at, in ? 16 : 0);
                }
            }
        }
        cp_async_commit();             // always: keeps the group count uniform
    };

    // per-row state (rows g and g + 8 of the group); d1 / d2 are this thread's share until the end
    float m[2] = {-INFINITY, -INFINITY}, d1[2] = {0.f, 0.f}, d2[2] = {0.f, 0.f};
    float o1[D / 8][4], o2[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o1[i][e] = o2[i][e] = 0.f;

#pragma unroll
    for (int i = 0; i < kGqaStages - 1; ++i) load_tile(i);

    for (int i = 0; i < n_tiles; ++i) {
        const int st = i % kGqaStages, key0 = my_lo + i * kGqaTile;
        cp_async_wait<kGqaStages - 2>();
        __syncwarp();                    // tile i has landed for every lane, and every lane has left tile i - 1
        load_tile(i + kGqaStages - 1);   // into the stage that tile i - 1 has just left

        // S1, S2: 16 rows x 16 keys (two 8-key blocks)
        float s1[2][4], s2[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) s1[nb][e] = s2[nb][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t kb[4];
            ldsm_x4(kb, bn_addr<LD>(sK(st), 0, ks * 16, lane));
            Elem<T>::mma(s1[0], qa[ks], kb[0], kb[1]);
            Elem<T>::mma(s1[1], qa[ks], kb[2], kb[3]);
            Elem<T>::mma(s2[0], ra[ks], kb[0], kb[1]);
            Elem<T>::mma(s2[1], ra[ks], kb[2], kb[3]);
        }
        // scale, mask the keys past the range, row maxima (a row lives in the four lanes of a quad)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + nb * 8 + 2 * t + (e & 1);
                s1[nb][e] = key < my_hi ? s1[nb][e] * a.c2 : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s1[nb][e]);
            }
        uint32_t pa1[4], pa2[4];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
            const float m_new = fmaxf(m[hh], mx[hh]);
            const float m_safe = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = fast_exp2(m[hh] - m_safe);
            m[hh] = m_new;
            if (alpha != 1.f) {
                d1[hh] *= alpha;
                d2[hh] *= alpha;
#pragma unroll
                for (int i2 = 0; i2 < D / 8; ++i2) {
                    o1[i2][2 * hh] *= alpha;
                    o1[i2][2 * hh + 1] *= alpha;
                    o2[i2][2 * hh] *= alpha;
                    o2[i2][2 * hh + 1] *= alpha;
                }
            }
#pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
                const float p0 = fast_exp2(s1[nb][2 * hh] - m_safe), p1 = fast_exp2(s1[nb][2 * hh + 1] - m_safe);
                const float q0 = p0 * s2[nb][2 * hh], q1 = p1 * s2[nb][2 * hh + 1];
                // A fragment of the output products: {row g, keys 2t..}, {row g + 8, ..}, {row g, keys 8 + 2t..}, {row g + 8, ..}
                pa1[2 * nb + hh] = Elem<T>::pack(p0, p1);
                pa2[2 * nb + hh] = Elem<T>::pack(q0, q1);
                // The sums are those of the ROUNDED weights that multiply V: the output then cancels as in
                // exact arithmetic when a row sees few keys (one key returns v exactly).
                const float2 pr = Elem<T>::unpack(pa1[2 * nb + hh]), qr = Elem<T>::unpack(pa2[2 * nb + hh]);
                d1[hh] += pr.x + pr.y;
                d2[hh] += qr.x + qr.y;
            }
        }
        // O1 += P1 V, O2 += P2 V: 16 channels per step
#pragma unroll
        for (int db = 0; db < D / 16; ++db) {
            uint32_t vb[4];
            ldsm_x4_t(vb, bt_addr<LD>(sV(st), 0, db * 16, lane));
            Elem<T>::mma(o1[2 * db], pa1, vb[0], vb[1]);
            Elem<T>::mma(o1[2 * db + 1], pa1, vb[2], vb[3]);
            Elem<T>::mma(o2[2 * db], pa2, vb[0], vb[1]);
            Elem<T>::mma(o2[2 * db + 1], pa2, vb[2], vb[3]);
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        d1[hh] += __shfl_xor_sync(0xffffffffu, d1[hh], 1);
        d1[hh] += __shfl_xor_sync(0xffffffffu, d1[hh], 2);
        d2[hh] += __shfl_xor_sync(0xffffffffu, d2[hh], 1);
        d2[hh] += __shfl_xor_sync(0xffffffffu, d2[hh], 2);
    }

    // Row g + 8 hh of the group is q head hq0 + g + 8 hh; this thread holds its channels 8 i + 2 t, + 1.
    const bool row_ok[2] = {g < n_rows, g + 8 < n_rows};
    auto bh_of = [&](int row) -> int64_t { return static_cast<int64_t>(b) * a.heads_q + hq0 + row; };

    if (a.n_splits == 1) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            if (!row_ok[hh]) continue;
            const int64_t bh = bh_of(g + 8 * hh);
            if (a.part_out) {
                float *rec = a.part_out + bh * REC;
                if (t == 0) *reinterpret_cast<float4 *>(rec) = make_float4(m[hh], d1[hh], d2[hh], 0.f);
#pragma unroll
                for (int i = 0; i < D / 8; ++i) {
                    *reinterpret_cast<float2 *>(rec + 4 + 8 * i + 2 * t) = make_float2(o1[i][2 * hh], o1[i][2 * hh + 1]);
                    *reinterpret_cast<float2 *>(rec + 4 + D + 8 * i + 2 * t) = make_float2(o2[i][2 * hh], o2[i][2 * hh + 1]);
                }
            } else {
                T *dst = static_cast<T *>(a.out) + bh * D;
#pragma unroll
                for (int i = 0; i < D / 8; ++i)
                    *reinterpret_cast<uint32_t *>(dst + 8 * i + 2 * t) =
                        Elem<T>::pack(finalize(d1[hh], d2[hh], o1[i][2 * hh], o2[i][2 * hh]),
                                      finalize(d1[hh], d2[hh], o1[i][2 * hh + 1], o2[i][2 * hh + 1]));
            }
        }
        return;
    }

    // publish this split's state of every row
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        if (!row_ok[hh]) continue;
        float *ws = a.ws_parts + (bh_of(g + 8 * hh) * a.n_splits + split) * REC;
        if (t == 0) __stcg(reinterpret_cast<float4 *>(ws), make_float4(m[hh], d1[hh], d2[hh], 0.f));
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            __stcg(reinterpret_cast<float2 *>(ws + 4 + 8 * i + 2 * t), make_float2(o1[i][2 * hh], o1[i][2 * hh + 1]));
            __stcg(reinterpret_cast<float2 *>(ws + 4 + D + 8 * i + 2 * t), make_float2(o2[i][2 * hh], o2[i][2 * hh + 1]));
        }
    }
    __threadfence();
    __syncwarp();

    // Arrival: lane r < n_rows counts for row r (all rows at once, one round trip); the warp then merges
    // the rows for which it arrived last.
    float big, D1, D2, O1[CH], O2[CH];
    auto emit = [&](int64_t bh) {
        if (a.part_out) {
            float *rec = a.part_out + bh * REC;
            if (lane == 0) *reinterpret_cast<float4 *>(rec) = make_float4(big, D1, D2, 0.f);
#pragma unroll
            for (int e = 0; e < CH; ++e) {
                rec[4 + lane * CH + e] = O1[e];
                rec[4 + D + lane * CH + e] = O2[e];
            }
        } else {
            T *dst = static_cast<T *>(a.out) + bh * D + lane * CH;
            const uint32_t p0 = Elem<T>::pack(finalize(D1, D2, O1[0], O2[0]), finalize(D1, D2, O1[1], O2[1]));
            if (CH == 4) {
                const uint32_t p1 = Elem<T>::pack(finalize(D1, D2, O1[CH - 2], O2[CH - 2]), finalize(D1, D2, O1[CH - 1], O2[CH - 1]));
                *reinterpret_cast<uint2 *>(dst) = make_uint2(p0, p1);
            } else {
                *reinterpret_cast<uint32_t *>(dst) = p0;
            }
        }
    };
    // Merge, for every row in `rows`, its n <= 32 records (the first one of row r at first_rec(r)), and hand
    // each result to sink(r).  Record by record and row by row this is a chain of L2 round trips (three per
    // row); here the header loads of all rows are in flight together (parked in this warp's shared memory,
    // which the tiles no longer need) and every row then takes one round of 16 record loads.
    float *hpark = reinterpret_cast<float *>(gqa_smem + warp * GqaSmem<D>::kPerWarp);
    auto merge_rows = [&](unsigned rows, auto first_rec, int n, auto sink) {
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            float4 h = make_float4(-INFINITY, 0.f, 0.f, 0.f);
            if (((rows >> r) & 1) && lane < n) h = __ldcg(reinterpret_cast<const float4 *>(first_rec(r) + static_cast<int64_t>(lane) * REC));
            hpark[r * 32 + lane] = h.x;
            hpark[512 + r * 32 + lane] = h.y;
            hpark[1024 + r * 32 + lane] = h.z;
        }
#pragma unroll 1
        for (int r = 0; r < n_rows; ++r) {
            if (!((rows >> r) & 1)) continue;
            const float hm = hpark[r * 32 + lane];
            big = hm;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, off));
            const float safe = big == -INFINITY ? 0.f : big;
            const float wl = fast_exp2(hm - safe);   // weight of record `lane` (0 beyond n: m = -inf there)
            D1 = wl * hpark[512 + r * 32 + lane];
            D2 = wl * hpark[1024 + r * 32 + lane];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                D1 += __shfl_xor_sync(0xffffffffu, D1, off);
                D2 += __shfl_xor_sync(0xffffffffu, D2, off);
            }
#pragma unroll
            for (int e = 0; e < CH; ++e) O1[e] = O2[e] = 0.f;
            const float *col = first_rec(r) + 4 + lane * CH;
#pragma unroll
            for (int j0 = 0; j0 < 32; j0 += 16) {
                if (j0 >= n) break;
                float x[16][CH], y[16][CH];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float *pr = col + static_cast<int64_t>(min(j0 + j, n - 1)) * REC;   // weight 0 past the end
                    if (CH == 4) {
                        const float4 u = __ldcg(reinterpret_cast<const float4 *>(pr)), v = __ldcg(reinterpret_cast<const float4 *>(pr + D));
                        x[j][0] = u.x; x[j][1] = u.y; x[j][CH - 2] = u.z; x[j][CH - 1] = u.w;
                        y[j][0] = v.x; y[j][1] = v.y; y[j][CH - 2] = v.z; y[j][CH - 1] = v.w;
                    } else {
                        const float2 u = __ldcg(reinterpret_cast<const float2 *>(pr)), v = __ldcg(reinterpret_cast<const float2 *>(pr + D));
                        x[j][0] = u.x; x[j][1] = u.y;
                        y[j][0] = v.x; y[j][1] = v.y;
                    }
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float w = __shfl_sync(0xffffffffu, wl, j0 + j);
#pragma unroll
                    for (int e = 0; e < CH; ++e) {
                        O1[e] = fmaf(w, x[j][e], O1[e]);
                        O2[e] = fmaf(w, y[j][e], O2[e]);
                    }
                }
            }
            sink(r);
        }
    };
    const int group = split / PLX_DECODE_GROUP;
    const int first = group * PLX_DECODE_GROUP, gsize = min(PLX_DECODE_GROUP, a.n_splits - first);
    unsigned mine = 0;
    if (lane < n_rows) {
        int *counter = a.n_groups == 0 ? a.ws_counters + bh_of(lane) : a.ws_gcounters + bh_of(lane) * a.n_groups + group;
        if (atomicAdd(counter, 1) == (a.n_groups == 0 ? a.n_splits : gsize) - 1) mine = 1u << lane;
    }
    unsigned todo = __reduce_or_sync(0xffffffffu, mine);
    if (todo == 0) return;
    __threadfence();
    auto finish = [&](int row) {
        const int64_t bh = bh_of(row);
        emit(bh);
        if (lane == 0) a.ws_counters[bh] = 0;   // ready for the next launch on this workspace
    };
    if (a.n_groups == 0) {
        merge_rows(todo, [&](int row) { return a.ws_parts + bh_of(row) * a.n_splits * REC; }, a.n_splits, finish);
        return;
    }
    // two levels: merge this group's records of the rows in `todo`, then arrive for those rows at the second level
    merge_rows(todo, [&](int row) { return a.ws_parts + (bh_of(row) * a.n_splits + first) * REC; }, gsize, [&](int row) {
        const int64_t bh = bh_of(row);
        float *grec = a.ws_gparts + (bh * a.n_groups + group) * REC;
        if (lane == 0) {
            __stcg(reinterpret_cast<float4 *>(grec), make_float4(big, D1, D2, 0.f));
            a.ws_gcounters[bh * a.n_groups + group] = 0;
        }
#pragma unroll
        for (int e = 0; e < CH; ++e) {
            __stcg(grec + 4 + lane * CH + e, O1[e]);
            __stcg(grec + 4 + D + lane * CH + e, O2[e]);
        }
    });
    __threadfence();
    __syncwarp();
    mine = 0;
    if (lane < n_rows && ((todo >> lane) & 1) && atomicAdd(a.ws_counters + bh_of(lane), 1) == a.n_groups - 1) mine = 1u << lane;
    todo = __reduce_or_sync(0xffffffffu, mine);
    if (todo == 0) return;
    __threadfence();
    merge_rows(todo, [&](int row) { return a.ws_gparts + bh_of(row) * a.n_groups * REC; }, a.n_groups, finish);
}

template <typename T, int D>
static int launch_decode_gqa(const DecodeArgs &a, cudaStream_t stream) {
    const int n_hgroups = (a.n_rep + 15) / 16;
    constexpr int kSmem = kGqaWarps * GqaSmem<D>::kPerWarp;
    auto kern = decode_gqa_kernel<T, D>;
    {   // the shared-memory opt-in is a per-device function attribute: set it once per device
        constexpr int kMaxDevices = 64;
        static std::mutex mu;
        static bool done[kMaxDevices] = {};
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PLX_ERR_DEVICE;
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev]) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) {
                (void)cudaGetLastError();
                return PLX_ERR_LAUNCH;
            }
            done[dev] = true;
        }
    }
    const int64_t n_warps = static_cast<int64_t>(a.batch) * a.heads_kv * n_hgroups * a.n_splits;
    kern<<<static_cast<unsigned>((n_warps + kGqaWarps - 1) / kGqaWarps), kGqaWarps * 32, kSmem, stream>>>(a, n_hgroups);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? PLX_OK : PLX_ERR_LAUNCH;
}

template <typename T, int D, int HG>
static int launch_decode_hg(const DecodeArgs &a, cudaStream_t stream) {
    constexpr int U = 4;  // key rows per stream and register buffer (two buffers: 8 rows of K and of V in flight)
    dim3 grid(a.n_splits, a.heads_q / HG, a.batch);
    if (a.n_rep > 1)
        decode_kernel<T, D, HG, U, true, false><<<grid, HG * 32, 0, stream>>>(a);
    else
        decode_kernel<T, D, HG, U, false, false><<<grid, HG * 32, 0, stream>>>(a);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? PLX_OK : PLX_ERR_LAUNCH;
}

// number of SMs of the current device (cached per device; 0 on failure)
static int tma_free_sm_count() {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static int cached[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[dev] && cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        (void)cudaGetLastError();
        cached[dev] = 0;
    }
    return cached[dev];
}

// Few (batch, head) pairs, not many keys (the shapes that are bound by latency: the same test as in
// plx_decode_choose_splits) and a split count that is a multiple of eight, at most 256: split groups
// (see decode_kernel).  Both arrangements are correct for any problem; long sweeps stay with one warp per
// split, whose CTAs read contiguous memory.
static bool decode_split_groups(const DecodeArgs &a) {
    const int64_t bh = static_cast<int64_t>(a.batch) * a.heads_q;
    const int64_t n_keys = a.window >= 0 && a.window < a.cache_len ? a.window : a.cache_len;
    return a.n_rep == 1 && a.n_splits >= 8 && a.n_splits % 8 == 0 && a.n_splits <= 256 &&
           bh <= PLX_DECODE_SPLIT_GROUP_MAX_BH && bh * n_keys <= (static_cast<int64_t>(1) << 19);
}

template <typename T, int D>
static int launch_decode_sg(const DecodeArgs &a, cudaStream_t stream) {
    const int n_cta = a.n_splits / 8;
    dim3 grid(n_cta, a.heads_q, a.batch);
    // Up to eight CTAs per (batch, head): one thread-block cluster, merged through distributed shared memory.
    // (Sixteen, beyond the portable size, was measured too: 12.5 us against 10.8 at B = 1, H = 8, 4096 keys.)
    const bool cluster = n_cta == 2 || n_cta == 4 || n_cta == 8;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(n_cta);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    // When every CTA gets an SM of its own, a warp keeps 16 rows of K and of V in flight per buffer
    // (U = 8, more registers, one CTA per SM); otherwise 8 rows and two CTAs per SM.  The CTAs of a
    // cluster must sit in one GPC, so fewer clusters than (SM count / cluster size) are resident at
    // once: the occupancy calculator gives the number, asked once per device and cluster size.
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return PLX_ERR_DEVICE;
    const int64_t units = static_cast<int64_t>(a.heads_q) * a.batch;
    bool roomy = units * n_cta <= tma_free_sm_count();
    if (cluster) {
        // resident clusters of the U = 8 kernel: 0 = not asked yet, -1 = none / the query failed
        static std::atomic<int> resident[64][4] = {};
        const int slot = n_cta == 2 ? 1 : n_cta == 4 ? 2 : 3;
        int n = resident[dev][slot].load(std::memory_order_acquire);
        if (n == 0) {
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, decode_kernel<T, D, 8, 8, false, true>, &cfg) != cudaSuccess || n < 1) {
                (void)cudaGetLastError();
                n = -1;
            }
            resident[dev][slot].store(n, std::memory_order_release);
        }
        roomy = roomy && units <= n;
    }
    auto kern = roomy ? decode_kernel<T, D, 8, 8, false, true> : decode_kernel<T, D, 8, 4, false, true>;
    cfg.numAttrs = cluster ? 1 : 0;
    cudaError_t st = cudaLaunchKernelEx(&cfg, kern, a);
    count_launch();
    return st == cudaSuccess && cudaGetLastError() == cudaSuccess ? PLX_OK : PLX_ERR_LAUNCH;
}

template <typename T, int D>
static int launch_decode_t(const DecodeArgs &a, cudaStream_t stream) {
    if (a.n_rep >= 2) return launch_decode_gqa<T, D>(a, stream);   // grouped heads: tensor-core kernel
    if (decode_split_groups(a)) return launch_decode_sg<T, D>(a, stream);
    // adjacent q heads share a CTA (one warp each): the largest group that divides the head count
    if (a.heads_q % 8 == 0) return launch_decode_hg<T, D, 8>(a, stream);
    if (a.heads_q % 4 == 0) return launch_decode_hg<T, D, 4>(a, stream);
    if (a.heads_q % 2 == 0) return launch_decode_hg<T, D, 2>(a, stream);
    return launch_decode_hg<T, D, 1>(a, stream);
}

// The fused sweep + exchange exists in the one-warp-per-split arrangement with at least two splits.
bool decode_fused_exchange_supported(const DecodeArgs &a) {
    return a.n_rep == 1 && a.n_splits >= 2 && !decode_split_groups(a);
}

int launch_decode(const DecodeArgs &a, int dtype, int head_dim, cudaStream_t stream) {
    if (dtype == PLX_BF16) {
        if (head_dim == 128) return launch_decode_t<__nv_bfloat16, 128>(a, stream);
        if (head_dim == 64) return launch_decode_t<__nv_bfloat16, 64>(a, stream);
    } else if (dtype == PLX_FP16) {
        if (head_dim == 128) return launch_decode_t<__half, 128>(a, stream);
        if (head_dim == 64) return launch_decode_t<__half, 64>(a, stream);
    }
    return PLX_ERR_UNSUPPORTED;
}

template <typename T, int D>
static int launch_merge_t(const float *parts, int n_parts, int n_records, void *out, cudaStream_t stream) {
    decode_merge_kernel<T, D><<<n_records, D, 0, stream>>>(parts, n_parts, n_records, out);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? PLX_OK : PLX_ERR_LAUNCH;
}

int launch_decode_merge(const float *parts, int n_parts, int n_records, int head_dim, int dtype, void *out,
                        cudaStream_t stream) {
    if (dtype == PLX_BF16) {
        if (head_dim == 128) return launch_merge_t<__nv_bfloat16, 128>(parts, n_parts, n_records, out, stream);
        if (head_dim == 64) return launch_merge_t<__nv_bfloat16, 64>(parts, n_parts, n_records, out, stream);
    } else if (dtype == PLX_FP16) {
        if (head_dim == 128) return launch_merge_t<__half, 128>(parts, n_parts, n_records, out, stream);
        if (head_dim == 64) return launch_merge_t<__half, 64>(parts, n_parts, n_records, out, stream);
    }
    return PLX_ERR_UNSUPPORTED;
}

}  // namespace plx

// ========================================================================= //
// plx_decode_static: decode with the split-KV scratch built into the library,
// for callers that cannot allocate device memory.
// ========================================================================= //
// The scratch of all such calls on a device.  In HOST code this name is only a
// stand-in for the symbol -- it is not a device address and must never be handed
// to a kernel; the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_decode_static_scratch[PLX_DECODE_STATIC_SCRATCH_BYTES];

// Device address of the array on the CURRENT device, looked up once per device.
static int decode_static_scratch(void **ptr) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static void *cached[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PLX_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_decode_static_scratch) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return PLX_ERR_DEVICE;
        }
        cached[dev] = p;
    }
    *ptr = cached[dev];
    return PLX_OK;
}

// argument and device checks of plx_decode (defined beside it)
extern "C" int plx_decode_check_args(const plx_decode_problem *p, const void *q, const void *r, const void *k, const void *v,
                                     const void *out);

extern "C" int plx_decode_static(const plx_decode_problem *p, const void *q, const void *r, const void *k,
                                 const void *v, void *out, const int32_t *seqused_k, const int32_t *cache_start,
                                 plx_stream_t stream) {
    size_t need = 0;
    int st = plx_decode_workspace_bytes(p, &need);  // also validates the problem
    if (st != PLX_OK) return st;
    if (p->n_splits == 1)  // a single split publishes nothing: no scratch involved at all
        return plx_decode(p, q, r, k, v, out, seqused_k, cache_start, nullptr, 0, stream);
    if (need > PLX_DECODE_STATIC_SCRATCH_BYTES) return PLX_ERR_STATIC_SCRATCH;
    // everything plx_decode would refuse is refused here, before anything is enqueued on the stream
    if ((st = plx_decode_check_args(p, q, r, k, v, out)) != PLX_OK) return st;
    void *scratch = nullptr;
    if ((st = decode_static_scratch(&scratch)) != PLX_OK) return st;
    // The array keeps whatever the previous call (possibly of another shape) left in it.  Partial
    // records are fully rewritten before they are read; the arrival counters must start at zero.
    const size_t counter_bytes =
        static_cast<size_t>(p->batch) * p->heads_q * (1 + PLX_DECODE_GROUPS(p->n_splits)) * sizeof(int);
    if (cudaMemsetAsync(static_cast<unsigned char *>(scratch) + (need - counter_bytes), 0, counter_bytes,
                        reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) {
        (void)cudaGetLastError();
        return PLX_ERR_LAUNCH;
    }
    return plx_decode(p, q, r, k, v, out, seqused_k, cache_start, scratch, PLX_DECODE_STATIC_SCRATCH_BYTES, stream);
}
