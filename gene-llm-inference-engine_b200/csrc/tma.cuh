// Tensor maps for TMA and bounded mbarrier waits, shared by the kernels that use them.
#pragma once

#include "common.cuh"

#include <cuda.h>

namespace gi {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link libcuda).
inline EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        }
    }
    return fn;
}

// A row-major [rows, cols] matrix (row stride ld elements) as boxes of [box_rows, box_cols]; the
// swizzle follows the box's row bytes (128, 64 or 32). Reads outside give zeros, writes are clipped.
inline int make_tensor_map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elt_bytes,
                              unsigned long long rows, unsigned long long cols, unsigned long long ld, int box_rows,
                              int box_cols, CUtensorMapL2promotion promo, const char* what) {
    EncodeTiledFn fn = tensor_map_encoder();
    if (!fn) { set_error("%s: cuTensorMapEncodeTiled is not available from the driver", what); return 1; }
    const int row_bytes = box_cols * elt_bytes;
    CUtensorMapSwizzle swz = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                           : row_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * elt_bytes};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                    promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("%s: cuTensorMapEncodeTiled failed with code %d", what, static_cast<int>(r)); return 1; }
    return 0;
}

}  // namespace gi
