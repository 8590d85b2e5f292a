#pragma once
// Host-side creation of TMA tensor maps. The driver entry point is fetched through the runtime, so
// the library needs no link-time dependency on libcuda and loads on a machine without a GPU.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "fu_kernels.h"
#include "host_util.h"

namespace fu {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn()
{
    // The encoder is a driver call and wants a current context on the calling thread. A thread that
    // has made no runtime call yet (an autograd worker whose first CUDA work is one of these
    // launches) has none: a no-op runtime call binds the device's primary context to it.
    static thread_local bool bound = false;
    if (!bound) {
        cudaFree(nullptr);
        bound = true;
    }
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void*                           p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    }
    return fn;
}

// A row-major matrix of `rows` x `cols` elements (`elem_bytes` each, leading dimension `ld`
// elements) read in boxes of `box_rows` x `box_cols` with the 128-byte swizzle; out-of-range
// elements read as zero. `box_cols * elem_bytes` must be 128.
inline int make_map_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                       uint32_t box_rows, uint32_t box_cols)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        return fail(FU_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((ld * elem_bytes) & 15u)) {
        return fail(FU_E_ARG, "a TMA operand needs a 16-byte aligned base and row pitch (base %p, pitch %llu B)", base,
                    static_cast<unsigned long long>(ld * elem_bytes));
    }
    const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const cuuint64_t dims[2]    = {cols, rows};
    const cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
    const cuuint32_t box[2]     = {box_cols, box_rows};
    const cuuint32_t estr[2]    = {1, 1};
    const CUresult   rc = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        return fail(FU_E_CUDA, "cuTensorMapEncodeTiled failed with %d (rows %llu, cols %llu, ld %llu)", static_cast<int>(rc),
                    static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols),
                    static_cast<unsigned long long>(ld));
    }
    return FU_OK;
}

// A (batch, rows, cols) tensor with independent row and batch pitches (elements), boxes of
// 1 x box_rows x box_cols. Used for q/k/v/o laid out (b, s, heads, d): batch index = head.
inline int make_map_3d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t batch, uint64_t rows, uint64_t cols,
                       uint64_t row_pitch, uint64_t batch_pitch, uint32_t box_rows, uint32_t box_cols)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        return fail(FU_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((row_pitch * elem_bytes) & 15u)
        || ((batch_pitch * elem_bytes) & 15u)) {
        return fail(FU_E_ARG, "a TMA operand needs 16-byte aligned base and pitches");
    }
    const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const cuuint64_t dims[3]    = {cols, rows, batch};
    const cuuint64_t strides[2] = {row_pitch * static_cast<uint64_t>(elem_bytes),
                                   batch_pitch * static_cast<uint64_t>(elem_bytes)};
    const cuuint32_t box[3]     = {box_cols, box_rows, 1};
    const cuuint32_t estr[3]    = {1, 1, 1};
    const CUresult   rc = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        return fail(FU_E_CUDA, "cuTensorMapEncodeTiled (3d) failed with %d", static_cast<int>(rc));
    }
    return FU_OK;
}

// A (batch, rows, heads, 128) bf16 tensor such as q/k/v/o in the window layout, addressed as
// (x, row, head, batch) and read in boxes of `box_rows` rows x 64 columns of one head.
inline int make_map_bshd(CUtensorMap* map, const void* base, uint64_t batch, uint64_t rows, uint64_t heads,
                         uint64_t row_pitch, uint64_t head_pitch, uint64_t batch_pitch, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        return fail(FU_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((row_pitch * 2) & 15u) || ((head_pitch * 2) & 15u)
        || ((batch_pitch * 2) & 15u)) {
        return fail(FU_E_ARG, "a TMA operand needs 16-byte aligned base and pitches");
    }
    const cuuint64_t dims[4]    = {128, rows, heads, batch};
    const cuuint64_t strides[3] = {row_pitch * 2, head_pitch * 2, batch_pitch * 2};
    const cuuint32_t box[4]     = {64, box_rows, 1, 1};
    const cuuint32_t estr[4]    = {1, 1, 1, 1};
    const CUresult   rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        return fail(FU_E_CUDA, "cuTensorMapEncodeTiled (bshd) failed with %d", static_cast<int>(rc));
    }
    return FU_OK;
}

}  // namespace fu
