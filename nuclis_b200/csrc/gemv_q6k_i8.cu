// Q6_K GEMV and small-batch GEMM (1..8 activation rows) for sm_100a on the integer tensor path, reading the
// planar form that launch_prepare writes at load time (prepare.cu): the kernel behind Backend.matvec,
// matvecRows, small matmul and matvecSegments on prepared Q6_K weights (the reference's kernel for this is
// nu_matvec_q6_k, inference/src/backends/metal/kernels/matvec.metal:227-264). The scheme is that of
// i8_kernel.cuh and gemv_q4k_i8.cu; what Q6_K changes:
//
//  * A scale group is 16 columns, so a group is one mma.sync.m16n8k16.s32.u8.s8 step: lane t of a quad
//    supplies the group's columns 4t..4t+3, one word per row. The planar record keeps, per (half hh, column
//    half ch) of the superblock, 16 bytes of low nibbles of quarters 0 / 2, 16 of quarters 1 / 3 and 16 of high
//    bits: word t of each is what lane t needs for the four quarters. A code is assembled as bytes
//    low4 | high2 << 4 (0..63) with two logic operations per four codes and stays unsigned; the bias of 32
//    is folded into the sum of X over the group (kernels/matvec.metal:252): d * sc * (sum(q * X) - 32 * sum(X)).
//  * The signed 8-bit group scale multiplies the int32 sums after the mma; the bias term is an m16n8k16 f16
//    step whose A holds the row's 16 scales (exact in fp16) and whose B holds the 16 group sums of X
//    (times 2^-11, as fp16 pieces hi + lo).
//  * A stage is 16 rows x three records (624 contiguous bytes per row) plus a 3 x 16 box of the f16 super-scales
//    from the transposed plane; a unit slot is three warps, a block 18 warps = 6 slots x 3 (15 = 5 x 3 in the wide
//    form). 624 bytes = 156 words put the rows 4 banks apart: the 4-byte loads of a warp (8 rows x 4 lanes)
//    hit 32 different banks. The digit rows are 16 bytes apart round the banks for the same reason.
#include "i8_q6k.cuh"

namespace nu {
namespace i8 {

using Plain = Q6KPlain;
using Dense = Q6KDense;
using Quad = Q6KDense;  // three or four tokens: the 15-warp geometry (two mmas a group want the wide form's registers), no K cut forced by the digit rows

static bool fill(const FastJob &job, Params &p, Plan &plan, bool maps) {
    if (job.enc != Q6_K || job.layout != 1) return false;
    const bool ok = job.tokens == 1 ? fill_geometry<Q6K, Plain, 1>(job, p, plan) : job.tokens == 2 ? fill_geometry<Q6K, Plain, 2>(job, p, plan) : job.tokens <= 4 ? fill_geometry<Q6K, Quad, 4>(job, p, plan) : fill_geometry<Q6K, Dense, 8>(job, p, plan);
    if (!ok) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows % 16 != 0) return false;  // the planar form is made of 16-row tiles
        const uint8_t *dplane = g.w + (size_t)g.rows * p.ksb * 208;
        if (maps && !encode_tiled_map(&p.map[s], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, g.w, (uint64_t)p.ksb * 52, g.rows, (uint64_t)p.ksb * 208, Q6K::ROW_PITCH / 4, 16,
                                      CU_TENSOR_MAP_SWIZZLE_NONE))
            return false;
        if (maps && !encode_weight_map(&p.map2[s], dplane, (uint64_t)g.rows * 2, p.ksb, (uint64_t)g.rows * 2, 32, Q6K::STAGE_SBS)) return false;
    }
    return true;
}

static int launch(cudaStream_t s, const FastJob &job, const Params &p, const Plan &plan) {
    return plan.nt == 1 ? launch_geometry<Q6K, Plain, 1>(s, job, p, plan) : plan.nt == 2 ? launch_geometry<Q6K, Plain, 2>(s, job, p, plan) : plan.nt == 4 ? launch_geometry<Q6K, Quad, 4>(s, job, p, plan) : launch_geometry<Q6K, Dense, 8>(s, job, p, plan);
}

}  // namespace i8

bool q6k_i8_fill(const FastJob &job, i8::Params &p, i8::Plan &plan, bool maps) { return i8::fill(job, p, plan, maps); }

bool q6k_i8_configure() {
    return i8::configure_geometry<i8::Q6K, i8::Plain, 1>() && i8::configure_geometry<i8::Q6K, i8::Plain, 2>() && i8::configure_geometry<i8::Q6K, i8::Quad, 4>() &&
           i8::configure_geometry<i8::Q6K, i8::Dense, 8>();
}

bool q6k_i8_supported(const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    return i8::fill(job, p, plan, false);
}

int launch_q6k_i8(cudaStream_t s, const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    if (!i8::fill(job, p, plan, true)) return 0;
    return i8::launch(s, job, p, plan);
}

}  // namespace nu
