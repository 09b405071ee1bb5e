// Host-side construction of TMA tensor maps (tiled mode, no multicast anywhere).
//
// cuTensorMapEncodeTiled is looked up through the runtime's driver entry point
// query so the library has no link-time dependency on libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace b200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) !=
                cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// 2-D bf16 tensor [outer, inner] with the given row pitch (bytes), copied in
// boxes of [box_outer, box_inner] elements laid out with the 128-byte swizzle
// (box_inner * 2 bytes must be <= 128).  Out-of-range elements read as zero.
inline int make_tmap_2d_bf16_sw128(CUtensorMap* out, const void* base, uint64_t inner,
                                   uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner,
                                   uint32_t box_outer) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        set_last_error("cuTensorMapEncodeTiled is not available from this driver");
        return B200_ERR_CUDA;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (row_pitch_bytes & 15u) != 0) {
        set_last_error("tensor map: base address and row pitch must be 16-byte aligned");
        return B200_ERR_INVALID_ARGUMENT;
    }
    if (box_inner * 2 > 128 || box_outer == 0 || box_outer > 256) {
        set_last_error("tensor map: box [%u, %u] outside the 128-byte swizzle limits", box_outer,
                       box_inner);
        return B200_ERR_INVALID_ARGUMENT;
    }
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_pitch_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t elem_strides[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                    strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
        return B200_ERR_CUDA;
    }
    return B200_OK;
}

}  // namespace b200
