// GEMV and small-batch GEMM (1..8 activation rows) for sm_100a on the integer tensor path for the encodings made
// of 32-element blocks under an f16 scale (Q5_0, Q5_1, Q4_0, IQ4_NL) and IQ4_XS, reading the planar forms that
// launch_prepare writes at load time (prepare.cu: GGUF blocks of 18, 22 and 24 bytes start on 2-byte boundaries, IQ4_XS superblocks of 136 on 8-byte ones).
// The kernel behind Backend.matvec, matvecRows, small matmul and matvecSegments on prepared weights of these
// encodings; the reference runs them on its generic nu_matvec
// (inference/src/backends/metal/kernels/matvec.metal:5-21; decoders inference/src/quant/decode.zig:46-53, 73-81, 125-143, 214-228).
// The scheme is that of i8_kernel.cuh and gemv_q4k_i8.cu; i8_block32.cuh says what these encodings change: codes
// assembled as bytes (nibble | fifth bit << 4, or the IQ4_NL table value) on m16n8k32, f16 block scales applied in
// F32, the offset (-16 d, -8 d, or m) through the group sums of X.
#include "i8_block32.cuh"

namespace nu {
namespace i8 {

using Plain = Block32Plain;

template <int KIND>
static bool fill_kind(const FastJob &job, Params &p, Plan &plan, bool maps) {
    using E = Block32<KIND>;
    const bool ok = job.tokens == 1 ? fill_geometry<E, Plain, 1>(job, p, plan) : job.tokens == 2 ? fill_geometry<E, Plain, 2>(job, p, plan) : job.tokens <= 4 ? fill_geometry<E, Plain, 4>(job, p, plan) : fill_geometry<E, Plain, 8>(job, p, plan);
    if (!ok) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows % 16 != 0) return false;  // the planar form is made of 16-row tiles
        const uint8_t *scales = g.w + (size_t)g.rows * p.ksb * E::ROW_BYTES;
        if (maps && !encode_tiled_map(&p.map[s], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, g.w, (uint64_t)p.ksb * (E::ROW_BYTES / 4), g.rows, (uint64_t)p.ksb * E::ROW_BYTES,
                                      E::ROW_PITCH / 4, 16, CU_TENSOR_MAP_SWIZZLE_NONE))
            return false;
        if (maps && !encode_tiled_map(&p.map2[s], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, scales, (uint64_t)g.rows * (E::SC_ROW / 4), p.ksb, (uint64_t)g.rows * E::SC_ROW,
                                      16 * E::SC_ROW / 4, E::STAGE_SBS, CU_TENSOR_MAP_SWIZZLE_NONE))
            return false;
    }
    return true;
}

// The kind a job is served as; -1 when it is none of this family's prepared forms.
static int kind_of(const FastJob &job) {
    if (job.enc == Q5_0 && job.layout == 3) return KIND_Q5_0;
    if (job.enc == Q5_1 && job.layout == 4) return KIND_Q5_1;
    if (job.enc == Q4_0 && job.layout == 5) return KIND_Q4_0;
    if (job.enc == IQ4_NL && job.layout == 5) return KIND_IQ4_NL;
    if (job.enc == IQ4_XS && job.layout == 6) return KIND_IQ4_XS;
    return -1;
}

static bool fill(const FastJob &job, Params &p, Plan &plan, bool maps) {
    switch (kind_of(job)) {
    case KIND_Q5_0: return fill_kind<KIND_Q5_0>(job, p, plan, maps);
    case KIND_Q5_1: return fill_kind<KIND_Q5_1>(job, p, plan, maps);
    case KIND_Q4_0: return fill_kind<KIND_Q4_0>(job, p, plan, maps);
    case KIND_IQ4_NL: return fill_kind<KIND_IQ4_NL>(job, p, plan, maps);
    case KIND_IQ4_XS: return fill_kind<KIND_IQ4_XS>(job, p, plan, maps);
    default: return false;
    }
}

template <int KIND>
static int launch_kind(cudaStream_t s, const FastJob &job, const Params &p, const Plan &plan) {
    using E = Block32<KIND>;
    return plan.nt == 1 ? launch_geometry<E, Plain, 1>(s, job, p, plan) : plan.nt == 2 ? launch_geometry<E, Plain, 2>(s, job, p, plan) : plan.nt == 4 ? launch_geometry<E, Plain, 4>(s, job, p, plan) : launch_geometry<E, Plain, 8>(s, job, p, plan);
}

template <int KIND>
static bool configure_kind() {
    using E = Block32<KIND>;
    return configure_geometry<E, Plain, 1>() && configure_geometry<E, Plain, 2>() && configure_geometry<E, Plain, 4>() && configure_geometry<E, Plain, 8>();
}

}  // namespace i8

bool block32_i8_configure() {
    return i8::configure_kind<i8::KIND_Q5_0>() && i8::configure_kind<i8::KIND_Q5_1>() && i8::configure_kind<i8::KIND_Q4_0>() && i8::configure_kind<i8::KIND_IQ4_NL>() &&
           i8::configure_kind<i8::KIND_IQ4_XS>();
}

bool block32_i8_supported(const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    return i8::fill(job, p, plan, false);
}

int launch_block32_i8(cudaStream_t s, const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    if (!i8::fill(job, p, plan, true)) return 0;
    switch (i8::kind_of(job)) {
    case i8::KIND_Q5_0: return i8::launch_kind<i8::KIND_Q5_0>(s, job, p, plan);
    case i8::KIND_Q5_1: return i8::launch_kind<i8::KIND_Q5_1>(s, job, p, plan);
    case i8::KIND_Q4_0: return i8::launch_kind<i8::KIND_Q4_0>(s, job, p, plan);
    case i8::KIND_IQ4_NL: return i8::launch_kind<i8::KIND_IQ4_NL>(s, job, p, plan);
    default: return i8::launch_kind<i8::KIND_IQ4_XS>(s, job, p, plan);
    }
}

}  // namespace nu
