// Host-side helper for TMA descriptors. cuTensorMapEncodeTiled lives in the driver; it is fetched
// through cudaGetDriverEntryPoint so that the library has no link-time dependency on libcuda.
#include <mutex>

#include "sm100_ptx.cuh"
#include "w8a8_internal.h"

namespace w8a8 {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return static_cast<EncodeTiledFn>(nullptr);
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

}  // namespace

int make_tensor_map_2d_u8(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t row_pitch_bytes,
                          uint32_t box_cols, uint32_t box_rows, int swizzle_128b) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(W8A8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (row_pitch_bytes & 15u))
        return fail(W8A8_ERR_INVALID_ARG, "TMA needs a 16-byte aligned base and row pitch");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t elem_strides[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(W8A8_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return W8A8_OK;
}

int make_tensor_map_3d_u8(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                          uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                          int swizzle_128b) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(W8A8_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (pitch1_bytes & 15u) || (pitch2_bytes & 15u))
        return fail(W8A8_ERR_INVALID_ARG, "TMA needs a 16-byte aligned base and pitches");
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {pitch1_bytes, pitch2_bytes};
    cuuint32_t box[3] = {b0, b1, b2};
    cuuint32_t elem_strides[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem_strides,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(W8A8_ERR_CUDA, "cuTensorMapEncodeTiled (3d) failed with CUresult %d", (int)r);
    return W8A8_OK;
}

}  // namespace w8a8
