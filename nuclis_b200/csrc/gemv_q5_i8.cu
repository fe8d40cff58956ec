// Q5_0 / Q5_1 GEMV and small-batch GEMM (1..8 activation rows) for sm_100a on the integer tensor path, reading
// the planar forms that launch_prepare writes at load time (prepare.cu: GGUF blocks of 22 and 24 bytes start on
// 2-byte boundaries). The kernel behind Backend.matvec, matvecRows, small matmul and matvecSegments on prepared
// Q5_0 / Q5_1 weights; the reference runs these encodings on its generic nu_matvec
// (inference/src/backends/metal/kernels/matvec.metal:5-21; decoders inference/src/quant/decode.zig:125-143).
// The scheme is that of i8_kernel.cuh and gemv_q4k_i8.cu; i8_q5.cuh says what these encodings change: 5-bit
// codes assembled as bytes (nibble | fifth bit << 4) on m16n8k32 u8 x s8, f16 block scales applied in F32,
// the offset (-16 d, or m) through the group sums of X.
#include "i8_q5.cuh"

namespace nu {
namespace i8 {

using Plain = Q5Plain;

template <bool OFFSET>
static bool fill_q5(const FastJob &job, Params &p, Plan &plan, bool maps) {
    using E = Q5<OFFSET>;
    const bool ok = job.tokens == 1 ? fill_geometry<E, Plain, 1>(job, p, plan) : job.tokens == 2 ? fill_geometry<E, Plain, 2>(job, p, plan) : job.tokens <= 4 ? fill_geometry<E, Plain, 4>(job, p, plan) : fill_geometry<E, Plain, 8>(job, p, plan);
    if (!ok) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows % 16 != 0) return false;  // the planar form is made of 16-row tiles
        const uint8_t *scales = g.w + (size_t)g.rows * p.ksb * 160;
        if (maps && !encode_tiled_map(&p.map[s], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, g.w, (uint64_t)p.ksb * 40, g.rows, (uint64_t)p.ksb * 160, E::ROW_PITCH / 4, 16,
                                      CU_TENSOR_MAP_SWIZZLE_NONE))
            return false;
        if (maps && !encode_tiled_map(&p.map2[s], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, scales, (uint64_t)g.rows * (E::SC_ROW / 4), p.ksb, (uint64_t)g.rows * E::SC_ROW,
                                      16 * E::SC_ROW / 4, E::STAGE_SBS, CU_TENSOR_MAP_SWIZZLE_NONE))
            return false;
    }
    return true;
}

static bool fill(const FastJob &job, Params &p, Plan &plan, bool maps) {
    if (job.enc == Q5_0 && job.layout == 3) return fill_q5<false>(job, p, plan, maps);
    if (job.enc == Q5_1 && job.layout == 4) return fill_q5<true>(job, p, plan, maps);
    return false;
}

template <bool OFFSET>
static int launch_q5(cudaStream_t s, const FastJob &job, const Params &p, const Plan &plan) {
    using E = Q5<OFFSET>;
    return plan.nt == 1 ? launch_geometry<E, Plain, 1>(s, job, p, plan) : plan.nt == 2 ? launch_geometry<E, Plain, 2>(s, job, p, plan) : plan.nt == 4 ? launch_geometry<E, Plain, 4>(s, job, p, plan) : launch_geometry<E, Plain, 8>(s, job, p, plan);
}

template <bool OFFSET>
static bool configure_q5() {
    using E = Q5<OFFSET>;
    return configure_geometry<E, Plain, 1>() && configure_geometry<E, Plain, 2>() && configure_geometry<E, Plain, 4>() && configure_geometry<E, Plain, 8>();
}

}  // namespace i8

bool q5_i8_configure() { return i8::configure_q5<false>() && i8::configure_q5<true>(); }

bool q5_i8_supported(const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    return i8::fill(job, p, plan, false);
}

int launch_q5_i8(cudaStream_t s, const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    if (!i8::fill(job, p, plan, true)) return 0;
    return job.enc == Q5_1 ? i8::launch_q5<true>(s, job, p, plan) : i8::launch_q5<false>(s, job, p, plan);
}

}  // namespace nu
