// Q2_K and Q3_K GEMV and small-batch GEMM (1..8 activation rows) for sm_100a on the integer tensor path, reading the
// planar forms that launch_prepare writes at load time (prepare.cu: GGUF superblocks of 84 and 110 bytes start on
// 4- and 2-byte boundaries). The kernel behind Backend.matvec, matvecRows, small matmul and matvecSegments on prepared
// weights of these encodings; the reference runs them on its generic nu_matvec
// (inference/src/backends/metal/kernels/matvec.metal:5-21; decoders inference/src/quant/decode.zig:174-196, 260-275).
// The scheme is that of i8_kernel.cuh and gemv_q4k_i8.cu; i8_q2k.cuh and i8_q3k.cuh say what these encodings change.
#include "i8_q2k.cuh"
#include "i8_q3k.cuh"

namespace nu {
namespace i8 {

template <class E, class G>
static bool fill_planes(const FastJob &job, Params &p, Plan &plan, bool maps, uint32_t tail_words_per_row16) {
    const bool ok = job.tokens == 1 ? fill_geometry<E, G, 1>(job, p, plan) : job.tokens == 2 ? fill_geometry<E, G, 2>(job, p, plan) : job.tokens <= 4 ? fill_geometry<E, G, 4>(job, p, plan) : fill_geometry<E, G, 8>(job, p, plan);
    if (!ok) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows % 16 != 0) return false;  // the planar form is made of 16-row tiles
        const uint8_t *tail = g.w + (size_t)g.rows * p.ksb * E::ROW_BYTES;
        if (maps && !encode_tiled_map(&p.map[s], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, g.w, (uint64_t)p.ksb * (E::ROW_BYTES / 4), g.rows, (uint64_t)p.ksb * E::ROW_BYTES,
                                      E::ROW_PITCH / 4, 16, CU_TENSOR_MAP_SWIZZLE_NONE))
            return false;
        // the second plane: per superblock, tail_words_per_row16 words for each tile of 16 rows
        const uint64_t inner = (uint64_t)(g.rows / 16) * tail_words_per_row16;
        if (maps && !encode_tiled_map(&p.map2[s], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, tail, inner, p.ksb, inner * 4, tail_words_per_row16, E::STAGE_SBS, CU_TENSOR_MAP_SWIZZLE_NONE))
            return false;
    }
    return true;
}

static bool fill(const FastJob &job, Params &p, Plan &plan, bool maps) {
    if (job.enc == Q2_K && job.layout == 7) return fill_planes<Q2K, Q2KPlain>(job, p, plan, maps, 16);
    if (job.enc == Q3_K && job.layout == 8) return fill_planes<Q3K, Q3KPlain>(job, p, plan, maps, Q3K::TAIL_BYTES / 4);
    return false;
}

template <class E, class G>
static int launch_planes(cudaStream_t s, const FastJob &job, const Params &p, const Plan &plan) {
    return plan.nt == 1 ? launch_geometry<E, G, 1>(s, job, p, plan) : plan.nt == 2 ? launch_geometry<E, G, 2>(s, job, p, plan) : plan.nt == 4 ? launch_geometry<E, G, 4>(s, job, p, plan) : launch_geometry<E, G, 8>(s, job, p, plan);
}

template <class E, class G>
static bool configure_planes() {
    return configure_geometry<E, G, 1>() && configure_geometry<E, G, 2>() && configure_geometry<E, G, 4>() && configure_geometry<E, G, 8>();
}

}  // namespace i8

bool q23k_i8_configure() { return i8::configure_planes<i8::Q2K, i8::Q2KPlain>() && i8::configure_planes<i8::Q3K, i8::Q3KPlain>(); }

bool q23k_i8_supported(const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    return i8::fill(job, p, plan, false);
}

int launch_q23k_i8(cudaStream_t s, const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    if (!i8::fill(job, p, plan, true)) return 0;
    return job.enc == Q2_K ? i8::launch_planes<i8::Q2K, i8::Q2KPlain>(s, job, p, plan) : i8::launch_planes<i8::Q3K, i8::Q3KPlain>(s, job, p, plan);
}

}  // namespace nu
