/* tensormap.cuh — host-side construction of TMA tensor maps without linking libcuda.
 *
 * The driver's cuTensorMapEncodeTiled is reached through cudaGetDriverEntryPoint, so the library links the CUDA
 * runtime statically (as every SiLVANN family does, engine/scripts/build_silicon_families.sh:150-155) and needs only
 * the driver at run time.  Encoding is a pure host computation (no device work); a door encodes per call and hands the
 * 128-byte map to the kernel as a __grid_constant__ parameter. */
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sv {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
        if (q != cudaDriverEntryPointSuccess) return nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

/* A 2-D map over `rows` rows of `cols` 16-bit elements, `row_stride_bytes` apart, read in boxes of `box_cols` x
 * `box_rows` with the 128-byte swizzle (box_cols * 2 must be 128).  Out-of-range rows read as zero.
 * Requirements the caller has checked: base 16-byte aligned, row_stride_bytes a multiple of 16. */
inline bool make_map_2d_sw128(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                              uint64_t row_stride_bytes, uint32_t box_cols, uint32_t box_rows, bool bf16) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_stride_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2u,
              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

/* A 2-D map over `rows` rows of `cols` BYTES, `row_stride_bytes` apart, read in boxes of `box_bytes` x `box_rows` with the
 * swizzle whose span equals the box's width (32, 64 or 128 bytes).  Out-of-range rows read as zero.  Requirements the
 * caller has checked: base 16-byte aligned, row_stride_bytes a multiple of 16. */
inline bool make_map_2d_bytes(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride_bytes,
                              uint32_t box_bytes, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const CUtensorMapSwizzle sw = box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : box_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_stride_bytes};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2u, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace sv
