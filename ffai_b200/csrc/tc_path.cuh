// Host glue for the tcgen05 grouped GEMM: tensor-map encoding and launch.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "grouped_gemm_sm100.cuh"

namespace ffai {
namespace g100 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is fetched through the runtime, so the library links no libcuda.
inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

// Packed weights [rows, words_per_row] u32; box = 32 words (256 x 4-bit = 128 B) x 128 rows, 128-byte swizzle.
inline bool make_weight_map(CUtensorMap* m, const uint32_t* w, uint64_t rows, uint64_t words_per_row) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {words_per_row, rows};
    cuuint64_t strides[1] = {words_per_row * 4};
    cuuint32_t box[2] = {(cuuint32_t)(KS / 8), (cuuint32_t)BM};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(w), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Activations [rows, K] bf16; box = 64 k x box_rows rows, 128-byte swizzle (K-major MMA operand).
inline bool make_act_map(CUtensorMap* m, const uint16_t* x, uint64_t rows, uint64_t K, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(x), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool FUSED, typename TOut, bool WBF16 = false>
int launch_grouped_gemm(const CUtensorMap& w, const CUtensorMap& w2, const CUtensorMap& x, const Params& p,
                        int n_ctas, cudaStream_t st) {
    using L = SmemLayout<WBF16>;
    auto k = grouped_gemm_kernel<FUSED, TOut, WBF16>;
    static SmemOptIn opt_in;
    if (!opt_in.ensure(k, L::TOTAL)) return -1;
    k<<<n_ctas, THREADS, L::TOTAL, st>>>(w, w2, x, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace g100
}  // namespace ffai
