// Parallax training kernels on warp-level tensor-core MMAs (mma.sync m16n8k16,
// fp32 accumulate): forward, backward row statistics, dq/dr and dk/dv.
//
// These kernels serve every shape the training entry points accept (head_dim 64
// and 128, bf16 and fp16, grouped-query heads, sliding window, packed sequences,
// len_q != len_k).  The math follows the upstream Triton kernels
// (parallax/triton/parallax_train.py:144-252 forward, :383-392 preprocess,
// :517-612 dq/dr, :737-889 dk/dv); the code shares nothing with them.
//
// Data layout in shared memory: every tile is row-major [rows][D + 8] 16-bit
// elements; the 16-byte row padding makes all ldmatrix reads conflict-free.
#include "plx_common.cuh"
#include "plx_launch.h"

namespace plx {

// ------------------------------------------------------------------------- //
// tile loader: rows [row0, row0 + ROWS) of one (batch, head) matrix whose rows
// are `row_stride` elements apart; rows >= n_rows are zero-filled.
// ------------------------------------------------------------------------- //
template <typename T, int ROWS, int D, int NT>
__device__ __forceinline__ void load_tile(T *smem, const T *gbase, int64_t row_stride, int row0,
                                          int n_rows) {
    constexpr int LD = D + 8;
    constexpr int CPR = D / 8;  // 16-byte chunks per row
    for (int c = threadIdx.x; c < ROWS * CPR; c += NT) {
        int rr = c / CPR, cc = c % CPR;
        int row = row0 + rr;
        bool ok = row < n_rows;
        const T *src = gbase + static_cast<int64_t>(ok ? row : 0) * row_stride + cc * 8;
        cp_async16(smem_u32(smem + rr * LD + cc * 8), src, ok ? 16 : 0);
    }
}

// 16 rows x D columns staged by ONE warp in shared memory -> global, 16 B per lane.
template <typename T, int D>
__device__ __forceinline__ void store_rows16(const T *smem_rows, T *gbase, int64_t row_stride,
                                             int row0, int n_rows, int lane) {
    constexpr int LD = D + 8;
    constexpr int CPR = D / 8;
    for (int c = lane; c < 16 * CPR; c += 32) {
        int rr = c / CPR, cc = c % CPR;
        int row = row0 + rr;
        if (row < n_rows) {
            uint4 val = *reinterpret_cast<const uint4 *>(smem_rows + rr * LD + cc * 8);
            *reinterpret_cast<uint4 *>(gbase + static_cast<int64_t>(row) * row_stride + cc * 8) = val;
        }
    }
}

__device__ __forceinline__ float quad_max(float x) {
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
    return fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
}
__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x + __shfl_xor_sync(0xffffffffu, x, 2);
}

// acc[SN/8][4] += A(16 x D, rows a_row0.. of tile sa) * B^T (SN x D, rows b_row0.. of tile sb)
template <typename T, int D, int SN>
__device__ __forceinline__ void gemm_nt(float (&acc)[SN / 8][4], uint32_t sa, int a_row0, uint32_t sb,
                                        int b_row0, int lane) {
    constexpr int LD = D + 8;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t a[4];
        ldsm_x4(a, a_addr<LD>(sa, a_row0, ks * 16, lane));
#pragma unroll
        for (int nb = 0; nb < SN / 16; ++nb) {
            uint32_t b[4];
            ldsm_x4(b, bn_addr<LD>(sb, b_row0 + nb * 16, ks * 16, lane));
            Elem<T>::mma(acc[2 * nb], a, b[0], b[1]);
            Elem<T>::mma(acc[2 * nb + 1], a, b[2], b[3]);
        }
    }
}

// Two products sharing the B operand: acc1 += A1 * B^T, acc2 += A2 * B^T.
template <typename T, int D, int SN>
__device__ __forceinline__ void gemm_nt2(float (&acc1)[SN / 8][4], float (&acc2)[SN / 8][4], uint32_t sa1,
                                         uint32_t sa2, int a_row0, uint32_t sb, int b_row0, int lane) {
    constexpr int LD = D + 8;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t a1[4], a2[4];
        ldsm_x4(a1, a_addr<LD>(sa1, a_row0, ks * 16, lane));
        ldsm_x4(a2, a_addr<LD>(sa2, a_row0, ks * 16, lane));
#pragma unroll
        for (int nb = 0; nb < SN / 16; ++nb) {
            uint32_t b[4];
            ldsm_x4(b, bn_addr<LD>(sb, b_row0 + nb * 16, ks * 16, lane));
            Elem<T>::mma(acc1[2 * nb], a1, b[0], b[1]);
            Elem<T>::mma(acc1[2 * nb + 1], a1, b[2], b[3]);
            Elem<T>::mma(acc2[2 * nb], a2, b[0], b[1]);
            Elem<T>::mma(acc2[2 * nb + 1], a2, b[2], b[3]);
        }
    }
}

// C fragments (16 x SN fp32) of one product -> A fragments (16 x SN 16-bit).
template <typename T, int SN>
__device__ __forceinline__ void to_a_frags(uint32_t (&a)[SN / 16][4], const float (&c)[SN / 8][4]) {
#pragma unroll
    for (int kk = 0; kk < SN / 16; ++kk) {
        a[kk][0] = Elem<T>::pack(c[2 * kk][0], c[2 * kk][1]);
        a[kk][1] = Elem<T>::pack(c[2 * kk][2], c[2 * kk][3]);
        a[kk][2] = Elem<T>::pack(c[2 * kk + 1][0], c[2 * kk + 1][1]);
        a[kk][3] = Elem<T>::pack(c[2 * kk + 1][2], c[2 * kk + 1][3]);
    }
}

// acc[D/8][4] += P (16 x SN, A fragments) * B (SN x D, rows b_row0.. of tile sb, read transposed)
template <typename T, int D, int SN>
__device__ __forceinline__ void gemm_pb(float (&acc)[D / 8][4], const uint32_t (&p)[SN / 16][4], uint32_t sb,
                                        int b_row0, int lane) {
    constexpr int LD = D + 8;
#pragma unroll
    for (int kk = 0; kk < SN / 16; ++kk) {
#pragma unroll
        for (int db = 0; db < D / 16; ++db) {
            uint32_t b[4];
            ldsm_x4_t(b, bt_addr<LD>(sb, b_row0 + kk * 16, db * 16, lane));
            Elem<T>::mma(acc[2 * db], p[kk], b[0], b[1]);
            Elem<T>::mma(acc[2 * db + 1], p[kk], b[2], b[3]);
        }
    }
}

// acc1 += P1 * B, acc2 += P2 * B  (shared B operand)
template <typename T, int D, int SN>
__device__ __forceinline__ void gemm_pb2(float (&acc1)[D / 8][4], float (&acc2)[D / 8][4],
                                         const uint32_t (&p1)[SN / 16][4], const uint32_t (&p2)[SN / 16][4],
                                         uint32_t sb, int b_row0, int lane) {
    constexpr int LD = D + 8;
#pragma unroll
    for (int kk = 0; kk < SN / 16; ++kk) {
#pragma unroll
        for (int db = 0; db < D / 16; ++db) {
            uint32_t b[4];
            ldsm_x4_t(b, bt_addr<LD>(sb, b_row0 + kk * 16, db * 16, lane));
            Elem<T>::mma(acc1[2 * db], p1[kk], b[0], b[1]);
            Elem<T>::mma(acc1[2 * db + 1], p1[kk], b[2], b[3]);
            Elem<T>::mma(acc2[2 * db], p2[kk], b[0], b[1]);
            Elem<T>::mma(acc2[2 * db + 1], p2[kk], b[2], b[3]);
        }
    }
}

// accumulator fragments of one warp (16 x D fp32) -> 16-bit rows in the warp's staging area
template <typename T, int D>
__device__ __forceinline__ void stage_rows16(T *smem_rows, const float (&acc)[D / 8][4], int lane) {
    constexpr int LD = D + 8;
    int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) {
        *reinterpret_cast<uint32_t *>(smem_rows + g * LD + nb * 8 + 2 * t) = Elem<T>::pack(acc[nb][0], acc[nb][1]);
        *reinterpret_cast<uint32_t *>(smem_rows + (g + 8) * LD + nb * 8 + 2 * t) =
            Elem<T>::pack(acc[nb][2], acc[nb][3]);
    }
}

// ========================================================================= //
// forward
// ========================================================================= //
// CTA: BM = 16 * NW query rows of one (batch, q head); loops over key tiles of
// BN keys (two cp.async stages), each processed in SN-key register sub-tiles.
template <typename T, int D, int NW, int BN, int SN>
__global__ void __launch_bounds__(NW * 32) fwd_mma_kernel(const TrainArgs a) {
    constexpr int BM = 16 * NW, LD = D + 8, NT = NW * 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T *sQ = reinterpret_cast<T *>(smem_raw);
    T *sR = sQ + BM * LD;
    T *sK = sR + BM * LD;        // [2][BN][LD]
    T *sV = sK + 2 * BN * LD;    // [2][BN][LD]
    __shared__ int s_loc[4];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) {
        Seq s;
        int tis = 0;
        bool ok = locate_tile(a, gridDim.x - 1 - blockIdx.x, BM, s, tis);
        s_loc[0] = ok ? s.bos : -1;
        s_loc[1] = s.nq;
        s_loc[2] = s.nk;
        s_loc[3] = tis;
    }
    __syncthreads();
    if (s_loc[0] < 0) return;
    const int bos = s_loc[0], nq = s_loc[1], nk = s_loc[2], r0 = s_loc[3] * BM;
    if (r0 >= nq) return;
    const int b = blockIdx.y / a.heads_q, h = blockIdx.y % a.heads_q, hk = h / a.n_rep;
    const Mask mask{nk - nq, a.window};

    const int64_t q_base = b * a.q_sb + h * a.q_sh + static_cast<int64_t>(bos) * a.q_st;
    const int64_t kv_base = b * a.kv_sb + hk * a.kv_sh + static_cast<int64_t>(bos) * a.kv_st;
    const T *gq = static_cast<const T *>(a.q) + q_base;
    const T *gr = static_cast<const T *>(a.r) + q_base;
    const T *gk = static_cast<const T *>(a.k) + kv_base;
    const T *gv = static_cast<const T *>(a.v) + kv_base;

    // visible key range of this row tile
    int hi_col = min(nk, r0 + BM + mask.off);
    int lo_col = a.window >= 0 ? max(0, r0 + mask.off - a.window + 1) : 0;
    const int jlo = lo_col / BN;
    const int jhi = hi_col > lo_col ? (hi_col + BN - 1) / BN : jlo;

    load_tile<T, BM, D, NT>(sQ, gq, a.q_st, r0, nq);
    load_tile<T, BM, D, NT>(sR, gr, a.q_st, r0, nq);
    if (jlo < jhi) {
        load_tile<T, BN, D, NT>(sK, gk, a.kv_st, jlo * BN, nk);
        load_tile<T, BN, D, NT>(sV, gv, a.kv_st, jlo * BN, nk);
    }
    cp_async_commit();

    float o1[D / 8][4], o2[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o1[i][e] = o2[i][e] = 0.f;
    // Two sets of row sums.  l1 / l2 are formed by the tensor cores from the SAME
    // 16-bit P that multiplies V (an all-ones B fragment) and normalise the OUTPUT:
    // with them bart * barv - O2 / d1 = sum_j P2_j (barv - v_j) / d1 cancels as it
    // does in exact arithmetic (identically 0 for a row that sees a single key).
    // row_d1 / row_d2 are the fp32 sums of the unrounded P; they are what the
    // backward recomputes, so they are the statistics that get saved.
    float l1[4] = {0.f, 0.f, 0.f, 0.f}, l2[4] = {0.f, 0.f, 0.f, 0.f};
    float row_m[2] = {-INFINITY, -INFINITY}, row_d1[2] = {0.f, 0.f}, row_d2[2] = {0.f, 0.f};
    const int i0 = r0 + warp * 16 + g;  // this thread's rows: i0 and i0 + 8
    const uint32_t uQ = smem_u32(sQ), uR = smem_u32(sR);

    for (int j = jlo; j < jhi; ++j) {
        const int st = (j - jlo) & 1;
        if (j + 1 < jhi) {
            load_tile<T, BN, D, NT>(sK + (st ^ 1) * BN * LD, gk, a.kv_st, (j + 1) * BN, nk);
            load_tile<T, BN, D, NT>(sV + (st ^ 1) * BN * LD, gv, a.kv_st, (j + 1) * BN, nk);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t uK = smem_u32(sK + st * BN * LD), uV = smem_u32(sV + st * BN * LD);

#pragma unroll 1
        for (int ss = 0; ss < BN / SN; ++ss) {
            const int c0 = j * BN + ss * SN;
            if (c0 >= hi_col || c0 + SN <= lo_col) continue;
            float s1[SN / 8][4], s2[SN / 8][4];
#pragma unroll
            for (int i = 0; i < SN / 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) s1[i][e] = s2[i][e] = 0.f;
            gemm_nt2<T, D, SN>(s1, s2, uQ, uR, warp * 16, uK, ss * SN, lane);

            // mask-free iff every row of the tile sees every key of the sub-tile
            const bool full = (c0 + SN - 1 <= r0 + mask.off) && (c0 + SN <= nk) &&
                              (a.window < 0 || c0 > r0 + BM - 1 + mask.off - a.window);
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < SN / 8; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float x = s1[nb][e] * a.c2;
                    if (!full) {
                        int col = c0 + nb * 8 + 2 * t + (e & 1);
                        int row = i0 + (e >> 1) * 8;
                        if (col >= nk || !mask(row, col)) x = -INFINITY;
                    }
                    s1[nb][e] = x;
                    mx[e >> 1] = fmaxf(mx[e >> 1], x);
                }
            float alpha[2], msafe[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                float mnew = fmaxf(row_m[hh], quad_max(mx[hh]));
                msafe[hh] = mnew == -INFINITY ? 0.f : mnew;
                alpha[hh] = fast_exp2(row_m[hh] - msafe[hh]);
                row_m[hh] = mnew;
            }
            float sum1[2] = {0.f, 0.f}, sum2[2] = {0.f, 0.f};
#pragma unroll
            for (int nb = 0; nb < SN / 8; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float p1 = fast_exp2(s1[nb][e] - msafe[e >> 1]);
                    float p2 = p1 * s2[nb][e];
                    sum1[e >> 1] += p1;
                    sum2[e >> 1] += p2;
                    s1[nb][e] = p1;
                    s2[nb][e] = p2;
                }
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                row_d1[hh] = row_d1[hh] * alpha[hh] + sum1[hh];
                row_d2[hh] = row_d2[hh] * alpha[hh] + sum2[hh];
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                l1[e] *= alpha[e >> 1];
                l2[e] *= alpha[e >> 1];
            }
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    o1[nb][e] *= alpha[e >> 1];
                    o2[nb][e] *= alpha[e >> 1];
                }
            uint32_t p1f[SN / 16][4], p2f[SN / 16][4];
            to_a_frags<T, SN>(p1f, s1);
            to_a_frags<T, SN>(p2f, s2);
#pragma unroll
            for (int kk = 0; kk < SN / 16; ++kk) {
                Elem<T>::mma(l1, p1f[kk], Elem<T>::kOnes, Elem<T>::kOnes);
                Elem<T>::mma(l2, p2f[kk], Elem<T>::kOnes, Elem<T>::kOnes);
            }
            gemm_pb2<T, D, SN>(o1, o2, p1f, p2f, uV, ss * SN, lane);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();  // (no key tile at all: the q / r copies of other threads must have landed)

    // epilogue: o = barv + bart * barv - O2 / d1
    float inv[2], bart[2], bart_saved[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        // every column of the ones-product holds the row sum; element 0 / 2 = rows g / g + 8
        const float dd1 = l1[2 * hh], dd2 = l2[2 * hh];
        inv[hh] = dd1 > 0.f ? 1.f / dd1 : 0.f;
        bart[hh] = dd2 * inv[hh];
        row_d1[hh] = quad_sum(row_d1[hh]);
        row_d2[hh] = quad_sum(row_d2[hh]);
        bart_saved[hh] = row_d1[hh] > 0.f ? row_d2[hh] / row_d1[hh] : 0.f;
    }
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float bv = o1[nb][e] * inv[e >> 1];
            o2[nb][e] = bv + bart[e >> 1] * bv - o2[nb][e] * inv[e >> 1];
            o1[nb][e] = bv;
        }
    // each warp re-uses its own 16 rows of the Q / R tiles as staging
    __syncwarp();
    T *stO = sQ + warp * 16 * LD, *stB = sR + warp * 16 * LD;
    stage_rows16<T, D>(stO, o2, lane);
    stage_rows16<T, D>(stB, o1, lane);
    __syncwarp();
    store_rows16<T, D>(stO, static_cast<T *>(a.o) + q_base, a.q_st, r0 + warp * 16, nq, lane);
    store_rows16<T, D>(stB, static_cast<T *>(a.barv) + q_base, a.q_st, r0 + warp * 16, nq, lane);
    if (t == 0) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            int row = i0 + hh * 8;
            if (row < nq) {
                int64_t si = b * a.st_sb + h * a.st_sh + static_cast<int64_t>(bos + row) * a.st_st;
                a.d1[si] = row_d1[hh];
                a.bart[si] = bart_saved[hh];
                a.m[si] = row_m[hh];
            }
        }
    }
}

// ========================================================================= //
// backward row statistics: one warp per 8 consecutive (batch, head, token) rows
//   bst = { m (finite), 1/d1, bart, t = go.o, b = go.barv, mL = m + log2 d1, 1 + bart, (b - t) * qk_scale }
// HBM-bound (three 16-bit rows in, 48 bytes out): every load of the warp's eight rows is issued
// before the first is used (16-byte loads, D / 8 lanes per row), lanes 0..7 then own one row each.
// ========================================================================= //
constexpr int kStatRowsPerWarp = 8;

template <typename T, int D>
// (four CTAs per SM: the kernel lives on loads in flight; 0.091 -> 0.078 ms against three at the benchmark size)
__global__ void __launch_bounds__(256, 4) bwd_stats_kernel(const TrainArgs a, int n_tok) {
    constexpr int R = kStatRowsPerWarp, LPR = D / 8, RPP = 32 / LPR, NP = R / RPP;   // lanes per row, rows per pass, passes
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(a.batch) * a.heads_q * n_tok;
    const int64_t first = (static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5)) * R;
    if (first >= total) return;
    // Row `gid` = first + off, off < R: the 64-bit division happens once per warp (for `first`), the rows
    // of the warp follow by stepping -- with a division per row the kernel was bound by integer
    // arithmetic, not by memory (0.100 ms for 435 MB at the benchmark size).
    const int64_t bh0 = first / n_tok;
    const int tok0 = static_cast<int>(first - bh0 * n_tok);
    auto locate = [&](int64_t gid, int64_t &base, int64_t &si) {
        int tok = tok0 + static_cast<int>(gid - first);
        int64_t bh = bh0;
        while (tok >= n_tok) {
            tok -= n_tok;
            ++bh;
        }
        const int b = static_cast<int>(bh / a.heads_q);
        const int h = static_cast<int>(bh - static_cast<int64_t>(b) * a.heads_q);
        base = b * a.q_sb + h * a.q_sh + static_cast<int64_t>(tok) * a.q_st;
        si = b * a.st_sb + h * a.st_sh + static_cast<int64_t>(tok) * a.st_st;
    };
    // lanes 0..R-1: the saved forward statistics of "their" row
    const bool owner = lane < R && first + lane < total;
    float m = 0.f, d1 = 0.f, bart = 0.f;
    if (owner) {
        int64_t base, si;
        locate(first + lane, base, si);
        m = a.m[si];
        d1 = a.d1[si];
        bart = a.bart[si];
    }
    uint4 xg[NP], xo[NP], xb[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) {
        const int64_t gid = first + p * RPP + lane / LPR;
        xg[p] = xo[p] = xb[p] = make_uint4(0u, 0u, 0u, 0u);
        if (gid < total) {
            int64_t base, si;
            locate(gid, base, si);
            const int64_t at = base + (lane % LPR) * 8;
            xg[p] = *reinterpret_cast<const uint4 *>(static_cast<const T *>(a.go) + at);
            xo[p] = *reinterpret_cast<const uint4 *>(static_cast<const T *>(a.o_in) + at);
            xb[p] = *reinterpret_cast<const uint4 *>(static_cast<const T *>(a.barv_in) + at);
        }
    }
    float t_row = 0.f, b_row = 0.f;   // lanes 0..R-1: t and b of their row
#pragma unroll
    for (int p = 0; p < NP; ++p) {
        const uint32_t wg[4] = {xg[p].x, xg[p].y, xg[p].z, xg[p].w}, wo[4] = {xo[p].x, xo[p].y, xo[p].z, xo[p].w},
                       wb[4] = {xb[p].x, xb[p].y, xb[p].z, xb[p].w};
        float tt = 0.f, bb = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 x = Elem<T>::unpack(wg[e]), y = Elem<T>::unpack(wo[e]), z = Elem<T>::unpack(wb[e]);
            tt += x.x * y.x + x.y * y.y;
            bb += x.x * z.x + x.y * z.y;
        }
#pragma unroll
        for (int sft = LPR / 2; sft > 0; sft >>= 1) {
            tt += __shfl_xor_sync(0xffffffffu, tt, sft);
            bb += __shfl_xor_sync(0xffffffffu, bb, sft);
        }
#pragma unroll
        for (int rr = 0; rr < RPP; ++rr) {
            const float tv = __shfl_sync(0xffffffffu, tt, rr * LPR), bv = __shfl_sync(0xffffffffu, bb, rr * LPR);
            if (lane == p * RPP + rr) {
                t_row = tv;
                b_row = bv;
            }
        }
    }
    if (owner) {
        const int64_t wid = first + lane;
        float4 lo = make_float4(m == -INFINITY ? 0.f : m, d1 > 0.f ? 1.f / d1 : 0.f, bart, t_row);
        // derived constants for the pipelined kernels: p = 2^(S1*c2 - mL) already carries 1/d1
        const float m_l = (d1 > 0.f && m != -INFINITY) ? m + log2f(d1) : INFINITY;
        float4 hi = make_float4(b_row, m_l, 1.f + bart, (b_row - t_row) * a.scale);
        float4 *dst = reinterpret_cast<float4 *>(a.bst + wid * 8);
        dst[0] = lo;
        dst[1] = hi;
        *reinterpret_cast<float4 *>(a.cst + wid * 4) = hi;
    }
}

// ========================================================================= //
// backward dq / dr
// ========================================================================= //
// CTA: BM = 16 * NW query rows; streams key tiles (K and V, two stages).
template <typename T, int D, int NW, int BN, int SN>
__global__ void __launch_bounds__(NW * 32) bwd_dqr_mma_kernel(const TrainArgs a, int n_tok) {
    constexpr int BM = 16 * NW, LD = D + 8, NT = NW * 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T *sQ = reinterpret_cast<T *>(smem_raw);
    T *sR = sQ + BM * LD;
    T *sG = sR + BM * LD;        // grad_o rows
    T *sK = sG + BM * LD;        // [2][BN][LD]
    T *sV = sK + 2 * BN * LD;    // [2][BN][LD]
    __shared__ int s_loc[4];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) {
        Seq s;
        int tis = 0;
        bool ok = locate_tile(a, gridDim.x - 1 - blockIdx.x, BM, s, tis);
        s_loc[0] = ok ? s.bos : -1;
        s_loc[1] = s.nq;
        s_loc[2] = s.nk;
        s_loc[3] = tis;
    }
    __syncthreads();
    if (s_loc[0] < 0) return;
    const int bos = s_loc[0], nq = s_loc[1], nk = s_loc[2], r0 = s_loc[3] * BM;
    if (r0 >= nq) return;
    const int b = blockIdx.y / a.heads_q, h = blockIdx.y % a.heads_q, hk = h / a.n_rep;
    const Mask mask{nk - nq, a.window};

    const int64_t q_base = b * a.q_sb + h * a.q_sh + static_cast<int64_t>(bos) * a.q_st;
    const int64_t kv_base = b * a.kv_sb + hk * a.kv_sh + static_cast<int64_t>(bos) * a.kv_st;
    const T *gk = static_cast<const T *>(a.k) + kv_base;
    const T *gv = static_cast<const T *>(a.v) + kv_base;

    int hi_col = min(nk, r0 + BM + mask.off);
    int lo_col = a.window >= 0 ? max(0, r0 + mask.off - a.window + 1) : 0;
    const int jlo = lo_col / BN;
    const int jhi = hi_col > lo_col ? (hi_col + BN - 1) / BN : jlo;

    load_tile<T, BM, D, NT>(sQ, static_cast<const T *>(a.q) + q_base, a.q_st, r0, nq);
    load_tile<T, BM, D, NT>(sR, static_cast<const T *>(a.r) + q_base, a.q_st, r0, nq);
    load_tile<T, BM, D, NT>(sG, static_cast<const T *>(a.go) + q_base, a.q_st, r0, nq);
    if (jlo < jhi) {
        load_tile<T, BN, D, NT>(sK, gk, a.kv_st, jlo * BN, nk);
        load_tile<T, BN, D, NT>(sV, gv, a.kv_st, jlo * BN, nk);
    }
    cp_async_commit();

    // per-row statistics of this thread's two rows
    const int i0 = r0 + warp * 16 + g;
    float rm[2], rinv[2], rbart[2], rt[2], rb[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        int row = i0 + hh * 8;
        rm[hh] = rinv[hh] = rbart[hh] = rt[hh] = rb[hh] = 0.f;
        if (row < nq) {
            const float *rec = a.bst + ((static_cast<int64_t>(b) * a.heads_q + h) * n_tok + bos + row) * 8;
            float4 lo = *reinterpret_cast<const float4 *>(rec);
            rm[hh] = lo.x;
            rinv[hh] = lo.y;
            rbart[hh] = lo.z;
            rt[hh] = lo.w;
            rb[hh] = rec[4];
        }
    }

    float dq[D / 8][4], dr[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) dq[i][e] = dr[i][e] = 0.f;
    const uint32_t uQ = smem_u32(sQ), uR = smem_u32(sR), uG = smem_u32(sG);

    for (int j = jlo; j < jhi; ++j) {
        const int st = (j - jlo) & 1;
        if (j + 1 < jhi) {
            load_tile<T, BN, D, NT>(sK + (st ^ 1) * BN * LD, gk, a.kv_st, (j + 1) * BN, nk);
            load_tile<T, BN, D, NT>(sV + (st ^ 1) * BN * LD, gv, a.kv_st, (j + 1) * BN, nk);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t uK = smem_u32(sK + st * BN * LD), uV = smem_u32(sV + st * BN * LD);

#pragma unroll 1
        for (int ss = 0; ss < BN / SN; ++ss) {
            const int c0 = j * BN + ss * SN;
            if (c0 >= hi_col || c0 + SN <= lo_col) continue;
            float s1[SN / 8][4], s2[SN / 8][4], av[SN / 8][4];
#pragma unroll
            for (int i = 0; i < SN / 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) s1[i][e] = s2[i][e] = av[i][e] = 0.f;
            gemm_nt2<T, D, SN>(s1, s2, uQ, uR, warp * 16, uK, ss * SN, lane);
            gemm_nt<T, D, SN>(av, uG, warp * 16, uV, ss * SN, lane);

            const bool full = (c0 + SN - 1 <= r0 + mask.off) && (c0 + SN <= nk) &&
                              (a.window < 0 || c0 > r0 + BM - 1 + mask.off - a.window);
#pragma unroll
            for (int nb = 0; nb < SN / 8; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int hh = e >> 1;
                    float w = fast_exp2(s1[nb][e] * a.c2 - rm[hh]);
                    if (!full) {
                        int col = c0 + nb * 8 + 2 * t + (e & 1);
                        int row = i0 + hh * 8;
                        if (col >= nk || !mask(row, col)) w = 0.f;
                    }
                    float p = w * rinv[hh];
                    float delta = av[nb][e] - rb[hh];
                    float gl = p * (av[nb][e] - rt[hh] + (rbart[hh] - s2[nb][e]) * delta);
                    s1[nb][e] = gl;
                    s2[nb][e] = -p * delta;
                }
            uint32_t glf[SN / 16][4], guf[SN / 16][4];
            to_a_frags<T, SN>(glf, s1);
            to_a_frags<T, SN>(guf, s2);
            gemm_pb2<T, D, SN>(dq, dr, glf, guf, uK, ss * SN, lane);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();

#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) dq[nb][e] *= a.scale;
    __syncwarp();
    T *stA = sQ + warp * 16 * LD, *stB = sR + warp * 16 * LD;
    stage_rows16<T, D>(stA, dq, lane);
    stage_rows16<T, D>(stB, dr, lane);
    __syncwarp();
    store_rows16<T, D>(stA, static_cast<T *>(a.dq) + q_base, a.q_st, r0 + warp * 16, nq, lane);
    store_rows16<T, D>(stB, static_cast<T *>(a.dr) + q_base, a.q_st, r0 + warp * 16, nq, lane);
}

// ========================================================================= //
// backward dk / dv
// ========================================================================= //
// CTA: BN = 16 * NW keys of one (batch, kv head); streams the query-row tiles
// (BR rows of q, r, grad_o + their statistics, two stages) of every q head of the
// group, so dk / dv leave the kernel already summed over the group.
// Scores are formed transposed (keys x rows) so that they feed the second MMA
// as the A operand without a register transpose.
template <typename T, int D, int NW, int BR, int SR>
__global__ void __launch_bounds__(NW * 32) bwd_dkv_mma_kernel(const TrainArgs a, int n_tok) {
    constexpr int BN = 16 * NW, LD = D + 8, NT = NW * 32;
    constexpr int STAGE = 3 * BR * LD;  // elements of q, r, grad_o per stage
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T *sK = reinterpret_cast<T *>(smem_raw);
    T *sV = sK + BN * LD;
    T *sQ = sV + BN * LD;  // [2][3][BR][LD]
    float *sS = reinterpret_cast<float *>(sQ + 2 * STAGE);  // [2][BR][8]
    __shared__ int s_loc[4];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) {
        Seq s;
        int tis = 0;
        bool ok = locate_tile(a, blockIdx.x, BN, s, tis);
        s_loc[0] = ok ? s.bos : -1;
        s_loc[1] = s.nq;
        s_loc[2] = s.nk;
        s_loc[3] = tis;
    }
    __syncthreads();
    if (s_loc[0] < 0) return;
    const int bos = s_loc[0], nq = s_loc[1], nk = s_loc[2], c0 = s_loc[3] * BN;
    if (c0 >= nk) return;
    const int b = blockIdx.y / a.heads_kv, hk = blockIdx.y % a.heads_kv;
    const Mask mask{nk - nq, a.window};
    const int64_t kv_base = b * a.kv_sb + hk * a.kv_sh + static_cast<int64_t>(bos) * a.kv_st;

    // query rows that can see any key of this tile
    const int i_lo = max(0, c0 - mask.off);
    const int i_hi = a.window >= 0 ? min(nq, min(nk, c0 + BN) - mask.off + a.window - 1) : nq;
    const int tlo = i_lo / BR;
    const int thi = i_hi > i_lo ? (i_hi + BR - 1) / BR : tlo;
    const int ntile = thi - tlo;
    const int nit = ntile * a.n_rep;  // iterations: (q head of the group, row tile)

    auto issue = [&](int it, int st) {
        const int hq = hk * a.n_rep + it / ntile;
        const int row0 = (tlo + it % ntile) * BR;
        const int64_t q_base = b * a.q_sb + hq * a.q_sh + static_cast<int64_t>(bos) * a.q_st;
        T *dst = sQ + st * STAGE;
        load_tile<T, BR, D, NT>(dst, static_cast<const T *>(a.q) + q_base, a.q_st, row0, nq);
        load_tile<T, BR, D, NT>(dst + BR * LD, static_cast<const T *>(a.r) + q_base, a.q_st, row0, nq);
        load_tile<T, BR, D, NT>(dst + 2 * BR * LD, static_cast<const T *>(a.go) + q_base, a.q_st, row0, nq);
        const float *rec = a.bst + ((static_cast<int64_t>(b) * a.heads_q + hq) * n_tok + bos) * 8;
        for (int c = threadIdx.x; c < BR * 2; c += NT) {
            int row = row0 + (c >> 1);
            bool ok = row < nq;
            cp_async16(smem_u32(sS + st * BR * 8 + c * 4), rec + static_cast<int64_t>(ok ? row : 0) * 8 + (c & 1) * 4,
                       ok ? 16 : 0);
        }
    };

    load_tile<T, BN, D, NT>(sK, static_cast<const T *>(a.k) + kv_base, a.kv_st, c0, nk);
    load_tile<T, BN, D, NT>(sV, static_cast<const T *>(a.v) + kv_base, a.kv_st, c0, nk);
    if (nit > 0) issue(0, 0);
    cp_async_commit();

    float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) dk[i][e] = dv[i][e] = 0.f;
    const uint32_t uK = smem_u32(sK), uV = smem_u32(sV);
    const int j0 = c0 + warp * 16 + g;  // this thread's keys: j0 and j0 + 8

    for (int it = 0; it < nit; ++it) {
        const int st = it & 1;
        if (it + 1 < nit) {
            issue(it + 1, st ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int row0 = (tlo + it % ntile) * BR;
        const uint32_t uQ = smem_u32(sQ + st * STAGE);
        const uint32_t uR = uQ + 2u * BR * LD, uG = uQ + 4u * BR * LD;
        const float *stats = sS + st * BR * 8;

#pragma unroll 1
        for (int ss = 0; ss < BR / SR; ++ss) {
            const int rr0 = row0 + ss * SR;  // first query row of the sub-tile
            if (rr0 >= i_hi || rr0 + SR <= i_lo) continue;
            float s1[SR / 8][4], s2[SR / 8][4], av[SR / 8][4];
#pragma unroll
            for (int i = 0; i < SR / 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) s1[i][e] = s2[i][e] = av[i][e] = 0.f;
            // transposed scores: rows = keys (A operand K or V), columns = query rows
            {
                constexpr int LDk = LD;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t ak[4], avf[4];
                    ldsm_x4(ak, a_addr<LDk>(uK, warp * 16, ks * 16, lane));
                    ldsm_x4(avf, a_addr<LDk>(uV, warp * 16, ks * 16, lane));
#pragma unroll
                    for (int nb = 0; nb < SR / 16; ++nb) {
                        uint32_t bq[4], br[4], bg[4];
                        ldsm_x4(bq, bn_addr<LDk>(uQ, ss * SR + nb * 16, ks * 16, lane));
                        ldsm_x4(br, bn_addr<LDk>(uR, ss * SR + nb * 16, ks * 16, lane));
                        ldsm_x4(bg, bn_addr<LDk>(uG, ss * SR + nb * 16, ks * 16, lane));
                        Elem<T>::mma(s1[2 * nb], ak, bq[0], bq[1]);
                        Elem<T>::mma(s1[2 * nb + 1], ak, bq[2], bq[3]);
                        Elem<T>::mma(s2[2 * nb], ak, br[0], br[1]);
                        Elem<T>::mma(s2[2 * nb + 1], ak, br[2], br[3]);
                        Elem<T>::mma(av[2 * nb], avf, bg[0], bg[1]);
                        Elem<T>::mma(av[2 * nb + 1], avf, bg[2], bg[3]);
                    }
                }
            }
            // mask-free iff every row of the sub-tile sees every key of the tile
            const bool full = (c0 + BN - 1 <= rr0 + mask.off) && (c0 + BN <= nk) && (rr0 + SR <= nq) &&
                              (a.window < 0 || c0 > rr0 + SR - 1 + mask.off - a.window);
#pragma unroll
            for (int nb = 0; nb < SR / 8; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int lr = ss * SR + nb * 8 + 2 * t + (e & 1);  // row inside the stage
                    const float4 sa = *reinterpret_cast<const float4 *>(stats + lr * 8);  // m, 1/d1, bart, t
                    const float sb = stats[lr * 8 + 4];
                    float w = fast_exp2(s1[nb][e] * a.c2 - sa.x);
                    if (!full) {
                        int row = row0 + lr;
                        int col = j0 + (e >> 1) * 8;
                        if (row >= nq || col >= nk || !mask(row, col)) w = 0.f;
                    }
                    float p = w * sa.y;
                    float delta = av[nb][e] - sb;
                    float cs = sa.z - s2[nb][e];
                    float gl = p * (av[nb][e] - sa.w + cs * delta) * a.scale;
                    s1[nb][e] = gl;
                    s2[nb][e] = -p * delta;
                    av[nb][e] = p * (1.f + cs);
                }
            uint32_t glf[SR / 16][4], guf[SR / 16][4], wf[SR / 16][4];
            to_a_frags<T, SR>(glf, s1);
            to_a_frags<T, SR>(guf, s2);
            to_a_frags<T, SR>(wf, av);
            gemm_pb<T, D, SR>(dk, glf, uQ, ss * SR, lane);
            gemm_pb<T, D, SR>(dk, guf, uR, ss * SR, lane);
            gemm_pb<T, D, SR>(dv, wf, uG, ss * SR, lane);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();

    // stage through the K / V tiles (every warp owns its 16 rows)
    T *stA = sK + warp * 16 * LD, *stB = sV + warp * 16 * LD;
    stage_rows16<T, D>(stA, dk, lane);
    stage_rows16<T, D>(stB, dv, lane);
    __syncwarp();
    store_rows16<T, D>(stA, static_cast<T *>(a.dk) + kv_base, a.kv_st, c0 + warp * 16, nk, lane);
    store_rows16<T, D>(stB, static_cast<T *>(a.dv) + kv_base, a.kv_st, c0 + warp * 16, nk, lane);
}

// ========================================================================= //
// launchers
// ========================================================================= //
template <typename K>
static cudaError_t set_smem(K kernel, size_t bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
}

static int n_row_tiles(const TrainArgs &a, int tile) {
    if (a.cu) return (a.len_q + tile - 1) / tile + a.n_seqs;
    return (a.len_q + tile - 1) / tile;
}
static int n_key_tiles(const TrainArgs &a, int tile) {
    if (a.cu) return (a.len_k + tile - 1) / tile + a.n_seqs;
    return (a.len_k + tile - 1) / tile;
}

template <typename T, int D>
static int launch_fwd_t(const TrainArgs &a, cudaStream_t stream) {
    constexpr int NW = 4, BN = 64, SN = (D == 128 ? 32 : 64), BM = 16 * NW, LD = D + 8;
    constexpr size_t smem = static_cast<size_t>(2 * BM + 4 * BN) * LD * sizeof(T);
    auto kern = fwd_mma_kernel<T, D, NW, BN, SN>;
    if (set_smem(kern, smem) != cudaSuccess) return PLX_ERR_LAUNCH;
    dim3 grid(n_row_tiles(a, BM), a.batch * a.heads_q);
    kern<<<grid, NW * 32, smem, stream>>>(a);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? PLX_OK : PLX_ERR_LAUNCH;
}

template <typename T, int D>
static int launch_bwd_t(const TrainArgs &a, int stages, cudaStream_t stream) {
    constexpr int LD = D + 8;
    const int n_tok = a.len_q;
    if (stages & PLX_BWD_STATS) {
        const int64_t rows = static_cast<int64_t>(a.batch) * a.heads_q * n_tok;
        bwd_stats_kernel<T, D><<<static_cast<unsigned>((rows + 8 * kStatRowsPerWarp - 1) / (8 * kStatRowsPerWarp)), 256, 0, stream>>>(a, n_tok);
        count_launch();
        if (cudaGetLastError() != cudaSuccess) return PLX_ERR_LAUNCH;
    }
    if (stages & PLX_BWD_DQR) {
        constexpr int NW = 4, BN = (D == 128 ? 32 : 64), SN = (D == 128 ? 16 : 32), BM = 16 * NW;
        constexpr size_t smem = static_cast<size_t>(3 * BM + 4 * BN) * LD * sizeof(T);
        auto kern = bwd_dqr_mma_kernel<T, D, NW, BN, SN>;
        if (set_smem(kern, smem) != cudaSuccess) return PLX_ERR_LAUNCH;
        dim3 grid(n_row_tiles(a, BM), a.batch * a.heads_q);
        kern<<<grid, NW * 32, smem, stream>>>(a, n_tok);
        count_launch();
        if (cudaGetLastError() != cudaSuccess) return PLX_ERR_LAUNCH;
    }
    if (stages & PLX_BWD_DKV) {
        constexpr int NW = 4, BR = 32, SR = 16, BN = 16 * NW;
        constexpr size_t smem = static_cast<size_t>(2 * BN + 6 * BR) * LD * sizeof(T) + 2 * BR * 8 * sizeof(float);
        auto kern = bwd_dkv_mma_kernel<T, D, NW, BR, SR>;
        if (set_smem(kern, smem) != cudaSuccess) return PLX_ERR_LAUNCH;
        dim3 grid(n_key_tiles(a, BN), a.batch * a.heads_kv);
        kern<<<grid, NW * 32, smem, stream>>>(a, n_tok);
        count_launch();
        if (cudaGetLastError() != cudaSuccess) return PLX_ERR_LAUNCH;
    }
    return PLX_OK;
}

int launch_train_fwd_mma(const TrainArgs &a, int dtype, int head_dim, cudaStream_t stream) {
    if (dtype == PLX_BF16) {
        if (head_dim == 128) return launch_fwd_t<__nv_bfloat16, 128>(a, stream);
        if (head_dim == 64) return launch_fwd_t<__nv_bfloat16, 64>(a, stream);
    } else if (dtype == PLX_FP16) {
        if (head_dim == 128) return launch_fwd_t<__half, 128>(a, stream);
        if (head_dim == 64) return launch_fwd_t<__half, 64>(a, stream);
    }
    return PLX_ERR_UNSUPPORTED;
}

int launch_train_bwd_mma(const TrainArgs &a, int dtype, int head_dim, int stages, cudaStream_t stream) {
    if (dtype == PLX_BF16) {
        if (head_dim == 128) return launch_bwd_t<__nv_bfloat16, 128>(a, stages, stream);
        if (head_dim == 64) return launch_bwd_t<__nv_bfloat16, 64>(a, stages, stream);
    } else if (dtype == PLX_FP16) {
        if (head_dim == 128) return launch_bwd_t<__half, 128>(a, stages, stream);
        if (head_dim == 64) return launch_bwd_t<__half, 64>(a, stages, stream);
    }
    return PLX_ERR_UNSUPPORTED;
}

}  // namespace plx
