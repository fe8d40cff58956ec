// Q8_0 GEMV and small-batch GEMM (1..8 activation rows) for sm_100a on the integer tensor path, reading the
// planar form that launch_prepare writes at load time (prepare.cu: the codes as a [rows][columns] int8 plane, the
// scales as a transposed [columns / 32][rows] f16 plane): the kernel behind Backend.matvec, matvecRows, small
// matmul and matvecSegments on prepared Q8_0 weights. The reference has no specialized Q8_0 matvec: it runs the
// generic nu_matvec (inference/src/backends/metal/kernels/matvec.metal:5-21, docs/engine/metal-backend.md:198-201).
// The scheme is that of i8_kernel.cuh and gemv_q4k_i8.cu; what Q8_0 changes:
//
//  * The codes are signed bytes as they lie: a block of 32 is one mma.sync.m16n8k32.s32.s8.s8 step against the
//    digit planes, with no unpacking at all; lane t of a quad supplies the block's columns 8t..8t+7 (one 64-bit
//    shared load per row).
//  * The block's scale is an f16, not an integer: it multiplies the int32 sums in F32 (one conversion and one
//    multiply-add per accumulator register and block). There are no minima and no bias, so the sums of X over
//    the groups are not staged.
//  * A stage is 16 rows x two superblocks of codes, copied as boxes of 16 x 544 bytes: 512 bytes of codes and 32
//    more, so that consecutive rows lie 8 banks apart in shared memory (rows of exactly 512 bytes would all start
//    in bank 0 and the warp's loads would conflict eight ways), plus a 16 x 16 box of the f16 scales. A unit slot is
//    two warps, a block 12 warps = 6 slots x 2.
#include "i8_q8_0.cuh"

namespace nu {
namespace i8 {

using Plain = Q80Plain;

static bool fill(const FastJob &job, Params &p, Plan &plan, bool maps) {
    if (job.enc != Q8_0 || job.layout != 2) return false;
    const bool ok = job.tokens == 1 ? fill_geometry<Q80, Plain, 1>(job, p, plan) : job.tokens == 2 ? fill_geometry<Q80, Plain, 2>(job, p, plan) : job.tokens <= 4 ? fill_geometry<Q80, Plain, 4>(job, p, plan) : fill_geometry<Q80, Plain, 8>(job, p, plan);
    if (!ok) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows % 16 != 0) return false;  // the planar form is made of 16-row tiles
        const uint8_t *scales = g.w + (size_t)g.rows * job.columns;
        if (maps && !encode_tiled_map(&p.map[s], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, g.w, (uint64_t)job.columns / 4, g.rows, (uint64_t)job.columns, Q80::ROW_PITCH / 4, 16,
                                      CU_TENSOR_MAP_SWIZZLE_NONE))
            return false;
        if (maps && !encode_weight_map(&p.map2[s], scales, (uint64_t)g.rows * 2, (uint64_t)job.columns / 32, (uint64_t)g.rows * 2, 32, Q80::STAGE_SBS * 8)) return false;
    }
    return true;
}

static int launch(cudaStream_t s, const FastJob &job, const Params &p, const Plan &plan) {
    return plan.nt == 1 ? launch_geometry<Q80, Plain, 1>(s, job, p, plan) : plan.nt == 2 ? launch_geometry<Q80, Plain, 2>(s, job, p, plan) : plan.nt == 4 ? launch_geometry<Q80, Plain, 4>(s, job, p, plan) : launch_geometry<Q80, Plain, 8>(s, job, p, plan);
}

}  // namespace i8

bool q8_0_i8_configure() {
    return i8::configure_geometry<i8::Q80, i8::Plain, 1>() && i8::configure_geometry<i8::Q80, i8::Plain, 2>() && i8::configure_geometry<i8::Q80, i8::Plain, 4>() &&
           i8::configure_geometry<i8::Q80, i8::Plain, 8>();
}

bool q8_0_i8_supported(const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    return i8::fill(job, p, plan, false);
}

int launch_q8_0_i8(cudaStream_t s, const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    if (!i8::fill(job, p, plan, true)) return 0;
    return i8::launch(s, job, p, plan);
}

}  // namespace nu
