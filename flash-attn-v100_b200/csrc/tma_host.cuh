// Host-side construction of TMA tensor maps over the (B, N, H, D) layout.
// cuTensorMapEncodeTiled is fetched through the runtime's driver entry point
// query, so the library carries no link-time dependency on libcuda and builds
// on a machine without a GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>
#include <mutex>
#include <unordered_map>

namespace fa {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// Tensor map over a (B, N, H, D) tensor with element strides (sb, sn, sh, 1):
// dimensions ordered (D, H, N, B); a box is `box_rows` sequence positions of
// one head by `box_cols` elements of D; `swizzle`: 0 none, 1 the 128-byte swizzle (16-byte
// pieces; box_cols * elem size must be 128 bytes), 2 the 128-byte swizzle in 32-byte pieces (what
// tcgen05.mma wants for an MN-major 32-bit operand).  Out-of-range rows read as zero.
// Returns 0 on success, else the CUresult (or -1 if the driver entry point is missing).
inline int make_tmap_bnhd(CUtensorMap* map, const void* ptr, CUtensorMapDataType dt, size_t elem_bytes,
                          int64_t B, int64_t N, int64_t H, int64_t D, int64_t sb, int64_t sn, int64_t sh,
                          int box_rows, int box_cols, int swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return -1;
    // size-1 dimensions may carry arbitrary strides in a tensor view: give them a legal one
    if (H == 1) sh = D;
    if (N == 1) sn = (sh * H > D ? sh * H : D);
    if (B == 1) sb = sn * N;
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)N, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)(sh * elem_bytes), (cuuint64_t)(sn * elem_bytes),
                             (cuuint64_t)(sb * elem_bytes)};
    cuuint32_t box[4] = {(cuuint32_t)box_cols, 1u, (cuuint32_t)box_rows, 1u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = fn(map, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                 : (swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE),
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return (int)r;
}

// The same map, looked up in a process-wide cache first.  Encoding a map is a driver call of a
// microsecond or two and a backward pass needs seven of them; a training loop presents the same
// (pointer, shape, strides) again and again (PyTorch's allocator hands the same blocks back), so the
// steady state pays one hash lookup per map instead.  A map holds nothing but the numbers it was
// encoded from, so it is valid on whichever device the pointer belongs to and a stale entry is
// harmless: a freed and re-used address with the same key describes the same bytes.
struct TmapKey {
    uint64_t ptr;
    int64_t B, N, H, D, sb, sn, sh;
    int32_t dt, box_rows, box_cols, swizzle;
    bool operator==(const TmapKey& o) const { return memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapKeyHash {
    size_t operator()(const TmapKey& k) const {
        const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
        uint64_t h = 0x9E3779B97F4A7C15ull;
        for (size_t i = 0; i < sizeof(TmapKey) / 8; ++i) { h ^= w[i]; h *= 0xFF51AFD7ED558CCDull; h ^= h >> 32; }
        return (size_t)h;
    }
};
static_assert(sizeof(TmapKey) % 8 == 0, "the key is hashed and compared as 64-bit words");

inline int cached_tmap_bnhd(CUtensorMap* map, const void* ptr, CUtensorMapDataType dt, size_t elem_bytes,
                            int64_t B, int64_t N, int64_t H, int64_t D, int64_t sb, int64_t sn, int64_t sh,
                            int box_rows, int box_cols, int swizzle) {
    static std::mutex mu;
    static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
    TmapKey key;
    memset(&key, 0, sizeof(key));
    key.ptr = (uint64_t)(uintptr_t)ptr;
    key.B = B; key.N = N; key.H = H; key.D = D; key.sb = sb; key.sn = sn; key.sh = sh;
    key.dt = (int32_t)dt; key.box_rows = box_rows; key.box_cols = box_cols; key.swizzle = swizzle;
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *map = it->second; return 0; }
    }
    const int r = make_tmap_bnhd(map, ptr, dt, elem_bytes, B, N, H, D, sb, sn, sh, box_rows, box_cols, swizzle);
    if (r == 0) {
        std::lock_guard<std::mutex> lock(mu);
        if (cache.size() >= 4096) cache.clear();          // bounded: start over rather than grow for ever
        cache.emplace(key, *map);
    }
    return r;
}

// Raise a kernel's dynamic shared-memory limit once per device instead of on every launch.
// `done` is a per-kernel bit mask of the devices already served.
template <typename Kernel>
inline cudaError_t set_smem_limit_once(Kernel kernel, int smem_bytes, int device, uint64_t* done, std::mutex* mu) {
    if (device >= 0 && device < 64) {
        std::lock_guard<std::mutex> lock(*mu);
        if (*done & (1ull << device)) return cudaSuccess;
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e == cudaSuccess) *done |= 1ull << device;
        return e;
    }
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
}

}  // namespace fa
