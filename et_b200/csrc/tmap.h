// Host-side construction of TMA tensor maps without linking libcuda: the encoder entry point is
// fetched from the driver through the runtime.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace et {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
                cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// 2-D fp16 row-major tensor [rows x cols] with row pitch `pitch_elems`; box = box_rows x box_cols.
// swizzle_bytes: 0 (none), 64 (box_cols must be 32) or 128 (box_cols must be 64). Out-of-range elements
// read as zero and are not written.
inline bool make_tmap_2d_f16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                             uint64_t pitch_elems, uint32_t box_rows, uint32_t box_cols,
                             int swizzle_bytes) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_elems * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box,
              estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
              : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same matrix seen as [cols/64 panels][rows][64 columns]: one box = `box_panels` adjacent 64-column
// panels of `box_rows` rows, each landing as its own 128-byte-swizzled [box_rows x 64] block, back to back.
// cols must be a multiple of 8; columns beyond `cols` in the last panel read as zero.
inline bool make_tmap_panels_f16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                                 uint64_t pitch_elems, uint32_t box_rows, uint32_t box_panels) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const uint64_t panels = (cols + 63) / 64;
    cuuint64_t dims[3] = {64, rows, panels};
    cuuint64_t strides[2] = {pitch_elems * 2, 128};
    cuuint32_t box[3] = {64, box_rows, box_panels};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace et
