// Host-side helpers shared by the tcgen05 kernel files: tensor-map encoding with a small cache,
// and once-per-device caches of device attributes and kernel attributes.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

namespace plx {
namespace tma {

constexpr int kMaxDevices = 64;

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                              const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
inline EncodeFn encode_fn() {
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

// What a map of these kernels depends on: a (head_dim, tokens, heads, batch) view of a 16-bit tensor
// with a box of 64 channels x `rows` tokens, 128-byte swizzle.
struct MapKey {
    const void *ptr;
    int64_t st, sh, sb;
    int32_t head_dim, tokens, heads, batch, rows, dtype;
};

// Encoding a map is pure host arithmetic on the key, so maps are kept in a small direct-mapped
// cache: a training loop that calls with the same buffers (or a CUDA-graph capture loop) encodes
// each map once.  A changed pointer, shape or stride is simply a different key.
inline bool make_map(CUtensorMap *map, CUtensorMapDataType dt, const void *ptr, int head_dim, int tokens, int heads, int batch,
                     int64_t st, int64_t sh, int64_t sb, int rows) {
    constexpr int kSlots = 64;
    struct Slot {
        MapKey key;
        CUtensorMap map;
        bool used;
    };
    static std::mutex mu;
    static Slot slots[kSlots] = {};
    MapKey key;
    memset(&key, 0, sizeof(key));
    key.ptr = ptr; key.st = st; key.sh = sh; key.sb = sb;
    key.head_dim = head_dim; key.tokens = tokens; key.heads = heads; key.batch = batch; key.rows = rows;
    key.dtype = static_cast<int32_t>(dt);
    uint64_t h = reinterpret_cast<uintptr_t>(ptr) >> 4;
    h = (h ^ (h >> 17)) * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(rows) * 31u + static_cast<uint64_t>(tokens);
    Slot &s = slots[(h >> 20) % kSlots];
    {
        std::lock_guard<std::mutex> lock(mu);
        if (s.used && memcmp(&s.key, &key, sizeof(key)) == 0) {
            *map = s.map;
            return true;
        }
    }
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(heads),
                                static_cast<cuuint64_t>(batch)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(st) * 2, static_cast<cuuint64_t>(sh) * 2,
                                   static_cast<cuuint64_t>(sb) * 2};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(rows), 1, 1};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    if (fn(map, dt, 4, const_cast<void *>(ptr), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> lock(mu);
    s.key = key;
    s.map = *map;
    s.used = true;
    return true;
}

// number of SMs of the current device (0 on failure)
inline int sm_count() {
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

// The dynamic shared-memory opt-in is a per-device attribute of a kernel: set it once per (kernel,
// device).  `done` is the caller's per-kernel table (one static array per template instance).
template <typename Kernel>
inline bool opt_in_smem(Kernel kern, int bytes, bool (&done)[kMaxDevices], std::mutex &mu) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (!done[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        done[dev] = true;
    }
    return true;
}

}  // namespace tma
}  // namespace plx
