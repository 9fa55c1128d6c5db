// Host helper: 2-D TMA tensor maps over row-major bf16 matrices, 128-byte swizzle, 64-column boxes.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/ittai_b200.h"

namespace ittai {

void set_error(const char* fmt, ...);

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tmap_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// [rows, cols] bf16 with leading dimension ld (elements); boxes of box_rows rows x box_cols columns (64 columns with the
// 128-byte swizzle, 32 columns with the 64-byte swizzle); out-of-range reads give 0, out-of-range writes are dropped.
inline int make_tmap_bf16(CUtensorMap* tm, const void* ptr, long long rows, long long cols, long long ld, int box_rows, int box_cols = 64) {
    EncodeTiledFn fn = tmap_encode_fn();
    if (fn == nullptr) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return ITTAI_E_CUDA; }
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with %d (rows %lld cols %lld ld %lld)", (int)r, rows, cols, ld); return ITTAI_E_CUDA; }
    return ITTAI_OK;
}

}  // namespace ittai
