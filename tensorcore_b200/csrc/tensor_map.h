// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled), looked up through the
// runtime so that the library does not link against the driver library.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tcb {

// Tiled map over a row-major byte matrix [rows][row_bytes] (row_bytes a multiple of 16, base
// 16-byte aligned) with a box of box_rows x box_bytes (box_bytes a multiple of 16).  The matrix is
// described in elements of elem_bytes (1 or 4) because a box is limited to 256 elements per
// dimension: box_bytes / elem_bytes <= 256, box_rows <= 256; the load's x coordinate is in
// elements.  No swizzle, no interleave; parts of a box outside the matrix read as zeros.
inline bool encode_bytes_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                            uint32_t box_bytes, uint32_t box_rows, uint32_t elem_bytes = 1) {
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
    static EncodeFn encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return reinterpret_cast<EncodeFn>(fn);
    }();
    if (!encode) return false;
    if (elem_bytes != 1 && elem_bytes != 4) return false;
    if (row_bytes % elem_bytes || box_bytes % elem_bytes) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes / elem_bytes), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
    const cuuint32_t box[2] = {box_bytes / elem_bytes, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return encode(map, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tcb
