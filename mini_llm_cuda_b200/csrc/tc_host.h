// Host helpers for the tensor-core GEMM: tensor-map encoding through the driver entry point
// (no link dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/mlb.h"
#include "errors.h"
#include "gemm_tc.cuh"

namespace mlb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D bf16 tensor map over a row-major [rows][cols] matrix, box = [box_rows][64 columns], 128-byte swizzle.
static inline int make_bf16_map(EncodeTiledFn enc, CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)kTcKB, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MLB_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return MLB_OK;
}

// 2-D map over a row-major [rows][cols] matrix of e4m3 codes (one byte each), box = [box_rows][64 codes], no swizzle:
// the tile is widened to bf16 by the kernel before the MMA reads it.
static inline int make_u8_map(EncodeTiledFn enc, CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols};
    cuuint32_t box[2] = {(cuuint32_t)kTcKB, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MLB_E_CUDA, "cuTensorMapEncodeTiled (e4m3 codes) failed with code %d", (int)r);
    return MLB_OK;
}

static inline EncodeTiledFn get_encode_tiled() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
        qres != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(fn);
}

}  // namespace mlb
