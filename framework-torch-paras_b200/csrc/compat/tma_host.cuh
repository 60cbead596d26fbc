// Host side of TMA: building CUtensorMap descriptors without linking libcuda (the encode
// function is fetched from the driver through the runtime).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "common.cuh"

namespace pb {

using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                       const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                       const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline TensorMapEncodeFn tensor_map_encode_fn() {
    static TensorMapEncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
                cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TensorMapEncodeFn>(sym);
        else
            cudaGetLastError();
    });
    return fn;
}

// Rank-3 map over 16-bit elements: dims {inner, rows, batch} (inner contiguous), element
// strides for rows and batch, box {box_inner, box_rows, 1}, 128-byte swizzle, zero fill for
// reads outside the tensor (writes outside it are dropped).  box_inner * 2 must be 128 bytes.
inline int make_tensor_map_3d(CUtensorMap* map, const void* base, int dtype, int64_t inner,
                              int64_t rows, int64_t batch, int64_t row_stride,
                              int64_t batch_stride, int box_inner, int box_rows) {
    TensorMapEncodeFn fn = tensor_map_encode_fn();
    if (!fn) return fail(PARAS_E_CUDA, "paras_b200: cuTensorMapEncodeTiled is unavailable");
    const cuuint64_t dims[3] = {cuuint64_t(inner), cuuint64_t(rows), cuuint64_t(batch)};
    // the stride of a size-1 dim is never used for addressing; keep it a legal multiple of 16
    const int64_t rs = rows > 1 ? row_stride : ((inner + 7) / 8) * 8;
    const int64_t bs = batch > 1 ? batch_stride : rs * rows;
    const cuuint64_t strides[2] = {cuuint64_t(rs) * 2, cuuint64_t(bs) * 2};
    const cuuint32_t box[3] = {cuuint32_t(box_inner), cuuint32_t(box_rows), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, dtype == PARAS_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                          3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(PARAS_E_CUDA, "paras_b200: cuTensorMapEncodeTiled failed with code %d", int(r));
    return PARAS_OK;
}

// Rank-4 map over a 16-bit [B, H, L, inner] tensor with element strides st = {B, H, L} and a
// contiguous inner dim: box {64, box_rows, 1, 1}, 128-byte swizzle, rows outside the tensor read
// as zero and are not written.
inline int make_tensor_map_bhld(CUtensorMap* map, const void* base, int dtype, int B, int H, int L,
                                int inner, const int64_t* st, int box_rows, int box_heads = 1) {
    TensorMapEncodeFn fn = tensor_map_encode_fn();
    if (!fn) return fail(PARAS_E_CUDA, "paras_b200: cuTensorMapEncodeTiled is unavailable");
    const cuuint64_t dims[4] = {cuuint64_t(inner), cuuint64_t(L), cuuint64_t(H), cuuint64_t(B)};
    // the stride of a size-1 dim is never used for addressing; keep it a legal multiple of 16
    const int64_t sl = L > 1 ? st[2] : inner;
    const int64_t sh = H > 1 ? st[1] : sl * L;
    const int64_t sb = B > 1 ? st[0] : sh * H;
    const cuuint64_t strides[3] = {cuuint64_t(sl) * 2, cuuint64_t(sh) * 2, cuuint64_t(sb) * 2};
    const cuuint32_t box[4] = {64, cuuint32_t(box_rows), cuuint32_t(box_heads), 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(map, dtype == PARAS_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                          4, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(PARAS_E_CUDA, "paras_b200: cuTensorMapEncodeTiled failed with code %d", int(r));
    return PARAS_OK;
}

}  // namespace pb
