// Host side of the specialized GEMV / small-batch kernels: which kernel serves a job, the one-time
// set-up of their shared-memory sizes, and the TMA tensor maps they all use.
//   Q4_K, 1..8 tokens:           i8_kernel<Q4K>   (gemv_q4k_i8.cu, i8_q4k.cuh, i8_kernel.cuh)
//   planar Q6_K, 1..8 tokens:    i8_kernel<Q6K>   (gemv_q6k_i8.cu, i8_q6k.cuh)
//   planar Q8_0, 1..8 tokens:    i8_kernel<Q80>   (gemv_q8_0_i8.cu, i8_q8_0.cuh)
//   planar Q5_0 / Q5_1 / Q4_0 / IQ4_NL: i8_kernel<Block32<>> (gemv_block32_i8.cu, i8_block32.cuh)
//   Q5_K, 1..8 tokens:           i8_kernel<Q5K>   (gemv_q5k_i8.cu, i8_q5k.cuh)
//   planar Q2_K / Q3_K:          i8_kernel<Q2K / Q3K> (gemv_q23k_i8.cu, i8_q2k.cuh, i8_q3k.cuh)
//   runs of one-token jobs:      chain_kernel     (gemv_chain.cu; opt-in)
// Everything else (F32 / F16 / BF16, unaligned views, the GGUF forms of the encodings that have a planar one) is declined here and
// served by the generic kernels (kernels_generic.cu).
#include <cuda.h>

#include "kernels.hpp"

namespace nu {

// cuTensorMapEncodeTiled through the runtime's driver entry point: no link against libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    }
    return fn;
}

// A two-dimensional tensor [outer][inner] of `elem_bytes`-wide elements, `stride_bytes` between rows.
bool encode_tiled_map(CUtensorMap *map, CUtensorMapDataType type, uint32_t elem_bytes, const void *base, uint64_t inner, uint64_t outer,
                      uint64_t stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    (void)elem_bytes;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, type, 2, (void *)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A uint8 tensor [rows][row_bytes] with `stride` bytes between rows, copied in boxes of box_rows x box_bytes.
bool encode_weight_map(CUtensorMap *map, const uint8_t *base, uint64_t row_bytes, uint64_t rows, uint64_t stride, uint32_t box_bytes, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {stride};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool fast_supported(const FastJob &job) {
    return q4k_i8_supported(job) || q6k_i8_supported(job) || q8_0_i8_supported(job) || block32_i8_supported(job) || q5k_i8_supported(job) || q23k_i8_supported(job);
}

bool fast_configure() {
    return q4k_i8_configure() && q6k_i8_configure() && q8_0_i8_configure() && block32_i8_configure() && q5k_i8_configure() && q23k_i8_configure() && prefill_configure() && expert_gemv_configure() && chain_configure();
}

int launch_fast(cudaStream_t s, const FastJob &job) {
    if (q4k_i8_supported(job)) return launch_q4k_i8(s, job);
    if (q6k_i8_supported(job)) return launch_q6k_i8(s, job);
    if (q8_0_i8_supported(job)) return launch_q8_0_i8(s, job);
    if (block32_i8_supported(job)) return launch_block32_i8(s, job);
    if (q5k_i8_supported(job)) return launch_q5k_i8(s, job);
    if (q23k_i8_supported(job)) return launch_q23k_i8(s, job);
    return 0;
}

}  // namespace nu
