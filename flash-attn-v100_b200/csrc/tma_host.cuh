// Host-side construction of TMA tensor maps over the (B, N, H, D) layout.
// cuTensorMapEncodeTiled is fetched through the runtime's driver entry point
// query, so the library carries no link-time dependency on libcuda and builds
// on a machine without a GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

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
// one head by `box_cols` elements of D, 128-byte swizzled (box_cols * elem
// size must be 128 bytes) or unswizzled.  Out-of-range rows read as zero.
// Returns 0 on success, else the CUresult (or -1 if the driver entry point is missing).
inline int make_tmap_bnhd(CUtensorMap* map, const void* ptr, CUtensorMapDataType dt, size_t elem_bytes,
                          int64_t B, int64_t N, int64_t H, int64_t D, int64_t sb, int64_t sn, int64_t sh,
                          int box_rows, int box_cols, bool swizzle128) {
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
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return (int)r;
}

}  // namespace fa
