// Shared device helpers for the Parallax sm_100a kernels: element traits,
// cp.async / ldmatrix / mma.sync wrappers, masking and the tile scheduler.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/plx_abi.h"

namespace plx {

constexpr float kLog2e = 1.4426950408889634f;

// ------------------------------------------------------------------------- //
// element traits
// ------------------------------------------------------------------------- //
template <typename T>
struct Elem;

template <>
struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t x) {
        return make_float2(__uint_as_float(x << 16), __uint_as_float(x & 0xffff0000u));
    }
    static constexpr uint32_t kOnes = 0x3f803f80u;  // {1.0, 1.0}
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

template <>
struct Elem<__half> {
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t x) {
        return __half22float2(*reinterpret_cast<__half2 *>(&x));
    }
    static constexpr uint32_t kOnes = 0x3c003c00u;  // {1.0, 1.0}
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

// ------------------------------------------------------------------------- //
// small PTX wrappers
// ------------------------------------------------------------------------- //
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 2^x, -inf -> +0
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 16-byte asynchronous copy global -> shared; bytes == 0 zero-fills the destination.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// ------------------------------------------------------------------------- //
// ldmatrix address helpers for a row-major [rows][LD] tile of 16-bit elements.
//
//  a_addr : 16x16 block used as the A operand (M = tile rows, K = tile columns)
//  bn_addr: 16x16 block used as B = tile^T (N = tile rows, K = tile columns);
//           registers {0,1} = N rows 0..7, {2,3} = N rows 8..15
//  bt_addr: 16x16 block used as B = tile (K = tile rows, N = tile columns), read
//           with the .trans form; registers {0,1} = N cols 0..7, {2,3} = cols 8..15
// ------------------------------------------------------------------------- //
template <int LD>
__device__ __forceinline__ uint32_t a_addr(uint32_t base, int row0, int col0, int lane) {
    return base + 2u * static_cast<uint32_t>((row0 + (lane & 15)) * LD + col0 + 8 * (lane >> 4));
}
template <int LD>
__device__ __forceinline__ uint32_t bn_addr(uint32_t base, int row0, int col0, int lane) {
    return base + 2u * static_cast<uint32_t>((row0 + (lane & 7) + 8 * (lane >> 4)) * LD + col0 +
                                             8 * ((lane >> 3) & 1));
}
template <int LD>
__device__ __forceinline__ uint32_t bt_addr(uint32_t base, int row0, int col0, int lane) {
    return base + 2u * static_cast<uint32_t>((row0 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + col0 +
                                             8 * (lane >> 4));
}

// ------------------------------------------------------------------------- //
// Kernel-side problem description (device copy of plx_train_problem + pointers)
// ------------------------------------------------------------------------- //
struct TrainArgs {
    const void *q, *r, *k, *v, *go, *o_in, *barv_in;
    void *o, *barv, *dq, *dr, *dk, *dv;
    float *d1, *bart, *m;
    float *bst;  // backward row statistics, 8 floats per (batch, head, token)
    float *cst;  // compact copy {b, mL, 1 + bart, (b - t) * scale}, 4 floats per (batch, head, token)
    const int32_t *cu;
    int n_seqs;
    int batch, heads_q, heads_kv, n_rep, len_q, len_k, window;
    float scale, c2;  // c2 = scale * log2(e)
    int64_t q_sb, q_sh, q_st, kv_sb, kv_sh, kv_st, st_sb, st_sh, st_st;
};

// One sequence as a kernel sees it.
struct Seq {
    int bos;  // first token (packed) or 0
    int nq;   // queries
    int nk;   // keys
};

// key j visible from query i?  (i, j relative to the sequence)
struct Mask {
    int off;     // nk - nq
    int window;  // -1 = off
    __device__ __forceinline__ bool operator()(int i, int j) const {
        int pos = i + off;
        return j <= pos && (window < 0 || j > pos - window);
    }
};

// Map a linear tile id to (sequence, tile inside the sequence) for tile_rows-row tiles.
// Dense: identity.  Packed: sequence i owns the ids
//     [cu[i] / tile_rows + i,  cu[i] / tile_rows + i + ceil(len_i / tile_rows)),
// which never overlap (a sequence has at most cu[i+1]/tile_rows - cu[i]/tile_rows + 1 tiles) and stay
// below total / tile_rows + n_seqs, the size the host gives the grid.  The first id of a sequence
// grows with i, so a tile finds its sequence by binary search over cu_seqlens alone -- no table of
// tile counts, no scan -- and ids that fall between two sequences return false.
__device__ __forceinline__ bool locate_tile(const TrainArgs &a, int tile_id, int tile_rows, Seq &s,
                                            int &tile_in_seq) {
    if (a.cu == nullptr) {
        s.bos = 0;
        s.nq = a.len_q;
        s.nk = a.len_k;
        tile_in_seq = tile_id;
        return true;
    }
    s.bos = 0;
    s.nq = s.nk = 0;
    tile_in_seq = 0;
    // last sequence whose first id is <= tile_id
    int lo = 0, hi = a.n_seqs - 1;
    if (tile_id < __ldg(a.cu) / tile_rows) return false;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldg(a.cu + mid) / tile_rows + mid <= tile_id) lo = mid;
        else hi = mid - 1;
    }
    const int b0 = __ldg(a.cu + lo), b1 = __ldg(a.cu + lo + 1);
    const int rest = tile_id - (b0 / tile_rows + lo);
    if (rest * tile_rows >= b1 - b0) return false;
    s.bos = b0;
    s.nq = s.nk = b1 - b0;
    tile_in_seq = rest;
    return true;
}

}  // namespace plx
