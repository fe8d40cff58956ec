// Q5_K GEMV and small-batch GEMM (1..8 activation rows) for sm_100a on the integer tensor path: the kernel behind
// Backend.matvec, matvecRows, small matmul and matvecSegments on Q5_K weights as GGUF stores them (176-byte
// superblocks). The reference runs this encoding on its generic nu_matvec
// (inference/src/backends/metal/kernels/matvec.metal:5-21; decoder inference/src/quant/decode.zig:147-170).
// The scheme is that of i8_kernel.cuh and gemv_q4k_i8.cu; i8_q5k.cuh says what the fifth bits change.
#include "i8_q5k.cuh"

namespace nu {
namespace i8 {

static bool fill_q5k(const FastJob &job, Params &p, Plan &plan, bool maps) {
    if (job.enc != Q5_K || job.layout != 0) return false;
    const bool ok = job.tokens == 1 ? fill_geometry<Q5K, Q5KPlain, 1>(job, p, plan) : job.tokens == 2 ? fill_geometry<Q5K, Q5KPlain, 2>(job, p, plan) : job.tokens <= 4 ? fill_geometry<Q5K, Q5KDense, 4>(job, p, plan) : fill_geometry<Q5K, Q5KDense, 8>(job, p, plan);
    if (!ok) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.stride % 16 != 0) return false;
        if (maps && !encode_tiled_map(&p.map[s], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, g.w, (uint64_t)p.ksb * 44, g.rows, g.stride, Q5K::ROW_PITCH / 4, 16, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
    }
    return true;
}

static int launch_q5k(cudaStream_t s, const FastJob &job, const Params &p, const Plan &plan) {
    return plan.nt == 1 ? launch_geometry<Q5K, Q5KPlain, 1>(s, job, p, plan) : plan.nt == 2 ? launch_geometry<Q5K, Q5KPlain, 2>(s, job, p, plan) : plan.nt == 4 ? launch_geometry<Q5K, Q5KDense, 4>(s, job, p, plan) : launch_geometry<Q5K, Q5KDense, 8>(s, job, p, plan);
}

}  // namespace i8

bool q5k_i8_configure() {
    return i8::configure_geometry<i8::Q5K, i8::Q5KPlain, 1>() && i8::configure_geometry<i8::Q5K, i8::Q5KPlain, 2>() && i8::configure_geometry<i8::Q5K, i8::Q5KDense, 4>() &&
           i8::configure_geometry<i8::Q5K, i8::Q5KDense, 8>();
}

bool q5k_i8_supported(const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    return i8::fill_q5k(job, p, plan, false);
}

int launch_q5k_i8(cudaStream_t s, const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    if (!i8::fill_q5k(job, p, plan, true)) return 0;
    return i8::launch_q5k(s, job, p, plan);
}

}  // namespace nu
