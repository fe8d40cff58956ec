// Q8_0 GEMM for 2..8 token rows on the planar form (prepare.cu), on the shared skeleton
// (rows_kernel.cuh; the scheme is described in gemv_q4k_rows.cu). The reference has no
// specialized Q8_0 kernel: it runs the generic nu_matvec
// (inference/src/backends/metal/kernels/matvec.metal:5-21).
//
// A Q8_0 scale is an f16 per 32 columns and a code has eight bits, so the scale cannot be folded
// into the fp16 A operand. As in the Q6_K kernel a k16 step of the mma covers columns of one scale
// block only: step (block b, half s) takes the 16 codes of 16-byte chunk 2b + s, lane t of a quad
// supplying word t of the chunk. The two steps of a block share an accumulator that starts from
// zero and is added to the task's sums with the block's scale as an F32 factor. The bias of 128
// (codes are used as code + 128, an fp16 subnormal) goes through the tensor core: one m16n8k8
// step whose A holds the eight scales of a row (f16 as stored) and whose B holds the eight block
// sums of x (times 2^-6, split hi + lo). Per superblock and row:
// out += sum_b d_b * 2^24 * C_b - 128 * 64 * C_bias.
//
// Rows of the code plane are 256 bytes apart in a 16 x 256 task, so the eight rows a warp reads with
// one instruction would all fall on the same banks. The task is therefore fetched as two TMA boxes
// of 16 rows x 128 bytes in the 128-byte swizzle (16-byte chunk c of row r sits at chunk c ^ (r & 7)),
// which spreads those eight rows over all banks; the 256 bytes of scales travel in the small
// second part of the stage so that the swizzled boxes stay on 1024-byte boundaries.
#include "rows_kernel.cuh"

namespace nu {

bool encode_tiled_map(CUtensorMap *map, CUtensorMapDataType type, uint32_t elem_bytes, const void *base, uint64_t inner, uint64_t outer,
                      uint64_t stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle);

namespace rows {

struct Q80 {
    static constexpr int TASK_BYTES = 4096;  // two swizzled boxes of 16 rows x 128 codes
    static constexpr bool SWIZZLED = true;  // whether the task's TMA boxes use a shared-memory swizzle
    static constexpr int AUX_BYTES = 256;    // 8 blocks x 16 rows of f16 scales
    static constexpr int GS_BYTES = 16;      // staged block sums per (B column, 256 columns): eight fp16

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t aux, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, TASK_BYTES + AUX_BYTES);
        tma_load_2d(dst, &p.map[seg], sb * 256, row0, bar, policy);
        tma_load_2d(dst + 2048, &p.map[seg], sb * 256 + 128, row0, bar, policy);
        tma_load_2d(aux, &p.map2[seg], row0 * 2, sb * 8, bar, policy);
    }
    // Float4 ci of a 256-column unit (columns 4ci..4ci+3): chunk c = ci >> 2 (16 columns), word m = ci & 3.
    // Lane m of a quad keeps its 16 steps (one per chunk) as 8 bytes each, 128 bytes in all.
    __device__ static __forceinline__ uint32_t x_offset(uint32_t i) {
        const uint32_t sb = i >> 6, ci = i & 63u;
        return (sb * 4 + (ci & 3u)) * PITCH + (ci >> 2) * 8;
    }
    // Sum of a 32-column block (eight consecutive lanes), times 2^-6, as fp16 pieces.
    __device__ static __forceinline__ void group_sum(uint8_t *gs_hi, uint8_t *gs_lo, uint32_t i, float sum, uint32_t lane) {
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if ((lane & 7) == 0) {
            sum *= 0.015625f;
            const __half sh = __float2half_rn(sum), sl = __float2half_rn(sum - __half2float(sh));
            const uint32_t blk = i >> 3;  // block within the window
            *(__half *)(gs_hi + blk * 2) = sh;
            *(__half *)(gs_lo + blk * 2) = sl;
        }
    }

    // One task: rows g and g+8 of the tile against every token column; see rows_kernel.cuh for the arguments.
    template <bool WIDE>
    __device__ static __forceinline__ void task(const uint8_t *task, const uint8_t *aux, const uint8_t *xb, uint32_t lo_off, const uint8_t *gsb, uint32_t gs_lo_off,
                                                uint32_t g, uint32_t t, float o[4]) {
        // rows g and g + 8 share the swizzle term (row & 7 == g); chunk c of a row sits at chunk c ^ g of its 128-byte line
        const uint8_t *line = task + g * 128 + t * 4;
        const __half *scales = (const __half *)aux;  // [block][row]
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            float cs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                const int c = 2 * b + s;  // 16-byte chunk of the row's 256 codes
                const uint8_t *src = line + (c >> 3) * 2048 + (((c & 7) ^ g) << 4);
                uint32_t a[4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t w = *(const uint32_t *)(src + h * 1024) ^ 0x80808080u;  // code + 128, 0..255
                    a[h] = __byte_perm(w, 0u, 0x4240);      // columns +0, +2 as fp16 subnormals
                    a[2 + h] = __byte_perm(w, 0u, 0x4341);  // columns +1, +3
                }
                const uint2 bb = *(const uint2 *)(xb + c * 8);
                mma16816(cs, a, bb.x, bb.y);
                if (WIDE) {
                    const uint2 ll = *(const uint2 *)(xb + lo_off + c * 8);
                    mma16816(cs, a, ll.x, ll.y);
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float d = __half2float(scales[b * 16 + g + 8 * h]);
                acc[2 * h] = fmaf(d, cs[2 * h], acc[2 * h]);
                acc[2 * h + 1] = fmaf(d, cs[2 * h + 1], acc[2 * h + 1]);
            }
        }
        // the bias: A = the row's eight scales (k = block: 2t, 2t+1), B = the block sums
        uint32_t am[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t lo = __half_as_ushort(scales[(2 * t) * 16 + g + 8 * h]), hi = __half_as_ushort(scales[(2 * t + 1) * 16 + g + 8 * h]);
            am[h] = lo | (hi << 16);
        }
        float cb[4] = {0.f, 0.f, 0.f, 0.f};
        mma1688(cb, am[0], am[1], *(const uint32_t *)(gsb + t * 4));
        if (WIDE) mma1688(cb, am[0], am[1], *(const uint32_t *)(gsb + gs_lo_off + t * 4));
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = fmaf(16777216.0f, acc[j], fmaf(-8192.0f, cb[j], o[j]));
    }
};

static bool fill_q8_0(const FastJob &job, Params &p, Plan &plan, bool maps) {
    if (job.enc != Q8_0 || job.layout != 2) return false;
    if (!fill_common<Q80>(job, p, plan)) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows % 16 != 0) return false;
        const uint8_t *dplane = g.w + (size_t)g.rows * job.columns;
        if (maps && !encode_tiled_map(&p.map[s], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g.w, job.columns, g.rows, job.columns, 128, 16, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
        if (maps && !encode_weight_map(&p.map2[s], dplane, (uint64_t)g.rows * 2, job.columns / 32, (uint64_t)g.rows * 2, 32, 8)) return false;
    }
    return true;
}

}  // namespace rows

bool q8_0_rows_configure() { return rows::configure<rows::Q80>(); }

bool q8_0_rows_supported(const FastJob &job) {
    if (job.tokens < 2) return false;
    rows::Params p;
    rows::Plan plan;
    return rows::fill_q8_0(job, p, plan, false);
}

int launch_q8_0_rows(cudaStream_t s, const FastJob &job) {
    rows::Params p;
    rows::Plan plan;
    if (!rows::fill_q8_0(job, p, plan, true)) return 0;
    return rows::launch<rows::Q80>(s, job, p, plan);
}

}  // namespace nu
