// Host-side construction of TMA tensor maps.  cuTensorMapEncodeTiled is fetched from the
// driver at run time, so the library links against the CUDA runtime only.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fmsa {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// bf16 matrix of `rows` rows and 128 columns, rows `row_stride_bytes` apart (a multiple of 16).
// The box is 64 columns x `box_rows` rows with the 128-byte swizzle, i.e. one panel of an operand tile.
inline bool make_tmap_rows(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_stride_bytes,
                           uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {128, rows};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Strided (B, H, S, 128) bf16 activation as a 4-D map {128, S, H, B}; element strides as in
// fmsa_tensor.  Box = 64 columns x `box_rows` sequence positions of one (batch, head).
inline bool make_tmap_bhsd(CUtensorMap* map, const void* base, uint64_t B, uint64_t H, uint64_t S, int64_t stride_b,
                           int64_t stride_h, int64_t stride_s, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {128, S, H, B};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(stride_s) * 2, static_cast<cuuint64_t>(stride_h) * 2,
                                   static_cast<cuuint64_t>(stride_b) * 2};
    const cuuint32_t box[4] = {64, box_rows, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Partial-row buffer [slots][heads][128] bf16 (heads = 1 gives the 2-D case) for tile STORES of
// 128 slots x one head x 128 elements from a dense row-major shared-memory tile (no swizzle).
inline bool make_tmap_partials(CUtensorMap* map, const void* base, uint64_t slots, uint64_t heads) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {128, heads, slots};
    const cuuint64_t strides[2] = {256, 256 * heads};
    const cuuint32_t box[3] = {128, 1, 128};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Row-gather view of a (B, H, S, 128) bf16 activation whose strides are all multiples of 128 elements: a
// 2-D matrix of 256-byte rows in which element row (b, h, s) has index (b*stride_b + h*stride_h +
// s*stride_s) / 128.  Box = 64 columns x 1 row, 128-byte swizzle: the form tile::gather4 loads take.
inline bool gather_compatible(const void* ptr, int64_t sb, int64_t sh, int64_t ss) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0 && sb > 0 && sh > 0 && ss > 0 && sb % 128 == 0 && sh % 128 == 0 &&
           ss % 128 == 0;
}
inline bool make_tmap_gather(CUtensorMap* map, const void* base, uint64_t nrows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn || nrows == 0 || nrows > 0x7fffffffull) return false;
    const cuuint64_t dims[2] = {128, nrows};
    const cuuint64_t strides[1] = {256};
    const cuuint32_t box[2] = {64, 1};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// Number of 256-byte rows the gather view of a (B, H, S, 128) activation spans.
inline uint64_t gather_rows(int64_t B, int64_t H, int64_t S, int64_t sb, int64_t sh, int64_t ss) {
    return static_cast<uint64_t>(((B - 1) * sb + (H - 1) * sh + (S - 1) * ss) / 128 + 1);
}

// Partial-row buffer [slots][heads][128] bf16 for tile STORES of 128 slots x one head from a shared-memory
// tile in the operand layout (two 64-column panels, 128-byte swizzle): one store per panel.
inline bool make_tmap_partials_swz(CUtensorMap* map, const void* base, uint64_t slots, uint64_t heads) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {128, heads, slots};
    const cuuint64_t strides[2] = {256, 256 * heads};
    const cuuint32_t box[3] = {64, 1, 128};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A TMA-loadable activation: last dimension contiguous, every stride a multiple of 8 elements
// (16 bytes), base 16-byte aligned.
inline bool tma_compatible(const void* ptr, int64_t sb, int64_t sh, int64_t ss) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0 && sb % 8 == 0 && sh % 8 == 0 && ss % 8 == 0 && ss >= 128 &&
           sb > 0 && sh > 0;
}

}  // namespace fmsa
