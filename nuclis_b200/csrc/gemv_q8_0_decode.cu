// Q8_0 decode GEMV (one activation row) for sm_100a, on the shared decode skeleton
// (decode_kernel.cuh; the scheme is described in gemv_q4k_decode.cu). The reference has no
// specialized Q8_0 matvec: it runs the generic nu_matvec
// (inference/src/backends/metal/kernels/matvec.metal:5-21, docs/engine/metal-backend.md:198-201).
//
// Q8_0 blocks are 34 bytes (f16 scale + 32 int8 codes): GGUF rows start on 2-byte boundaries, so
// this kernel reads the planar form launch_prepare writes at load time (prepare.cu): the codes as a
// [rows][columns] int8 plane and the scales as a transposed [columns/32][rows] f16 plane. Same bytes,
// same values. A task is 16 rows x 256 columns: one 4096-byte TMA box of codes and a 256-byte box
// of the 8 x 16 scales.
//
// Lane t of a quad owns the 16-byte chunks t, t+4, t+8, t+12 of a row's 256 codes (so the four lanes
// of a quad read 64 contiguous bytes at a time): half of each of four blocks. Codes become the fp16
// subnormals (code + 128) * 2^-24 by one XOR and two byte permutes per four codes; the bias of 128 is
// folded into the sum of x over the lane's 16 columns: d * (sum((code+128) * x) - 128 * sum(x)).
#include "decode_kernel.cuh"

namespace nu {
namespace dec {

struct Q80 {
    static constexpr int ROW_BYTES = 256;                 // 256 codes of one row
    static constexpr int MAIN_BYTES = 16 * ROW_BYTES;     // 4096
    static constexpr int TASK_BYTES = MAIN_BYTES + 256;   // + 8 blocks x 16 rows of f16 scales
    static constexpr int GSUMS = 16;                      // activation sums per 256 columns: one per 16-column chunk

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, TASK_BYTES);
        tma_load_2d(dst, &p.map[seg], sb * ROW_BYTES, row0, bar, policy);
        tma_load_2d(dst + MAIN_BYTES, &p.map2[seg], row0 * 2, sb * 8, bar, policy);
    }
    // Float4 ci of a 256-column unit: chunk c = ci >> 2 (16 columns), word m = ci & 3; lane t = c & 3 keeps
    // chunk j = c >> 2 of its four as words (j, m) -> 8 bytes each, 128 bytes in all.
    __device__ static __forceinline__ uint32_t x_offset(uint32_t i) {
        const uint32_t sb = i >> 6, ci = i & 63u;
        const uint32_t c = ci >> 2, m = ci & 3u;
        return (sb * 4 + (c & 3u)) * PAIR_PITCH + ((c >> 2) * 4 + m) * 8;
    }
    // 16-column chunk sum: four consecutive threads hold a chunk; lane t reads its four chunks as one float4.
    __device__ static __forceinline__ void group_sum(float *gsum, uint32_t i, float s, uint32_t lane) {
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if ((lane & 3) == 0) {
            const uint32_t sb = i >> 6, c = (i & 63u) >> 2;
            gsum[sb * 16 + (c & 3u) * 4 + (c >> 2)] = s;
        }
    }
    __device__ static __forceinline__ void task(const uint8_t *task, const uint8_t *xb, const float *gsum, uint32_t g, uint32_t t, float acc[2]) {
        const float4 gs = *(const float4 *)(gsum + t * 4);
        const float gsv[4] = {gs.x, gs.y, gs.z, gs.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint4 q[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) q[h] = *(const uint4 *)(task + (g + 8 * h) * ROW_BYTES + (4 * j + t) * 16);
            float c[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                uint32_t a[4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t w = (m == 0 ? q[h].x : m == 1 ? q[h].y : m == 2 ? q[h].z : q[h].w) ^ 0x80808080u;  // code + 128, 0..255
                    a[h] = __byte_perm(w, 0u, 0x4240);      // columns +0, +2 as fp16 subnormals
                    a[2 + h] = __byte_perm(w, 0u, 0x4341);  // columns +1, +3
                }
                const uint2 b = *(const uint2 *)(xb + (j * 4 + m) * 8);
                if (m == 0) mma16816_first(c, a, b.x, b.y);
                else mma16816(c, a, b.x, b.y);
            }
            // chunk 4j + t lies in block 2j + (t >> 1) of the eight
            const uint32_t blk = 2 * j + (t >> 1);
            const float bias = -128.0f * gsv[j];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float d = __half2float(*(const __half *)(task + MAIN_BYTES + (blk * 16 + g + 8 * h) * 2));
                acc[h] = fmaf(d, fmaf(c[2 * h] + c[2 * h + 1], 16777216.0f, bias), acc[h]);
            }
        }
    }
};

static bool fill(const FastJob &job, Params &p, bool maps) {
    if (job.enc != Q8_0 || job.layout != 2) return false;
    if (!fill_common<Q80>(job, p)) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows % 16 != 0) return false;
        const uint8_t *dplane = g.w + (size_t)g.rows * job.columns;
        if (maps && !encode_weight_map(&p.map[s], g.w, job.columns, g.rows, job.columns, 256, 16)) return false;
        if (maps && !encode_weight_map(&p.map2[s], dplane, (uint64_t)g.rows * 2, job.columns / 32, (uint64_t)g.rows * 2, 32, 8)) return false;
    }
    return true;
}

}  // namespace dec

bool q8_0_decode_configure() { return dec::configure<dec::Q80>(); }

bool q8_0_decode_supported(const FastJob &job) {
    dec::Params p;
    return dec::fill(job, p, false);
}

int launch_q8_0_decode(cudaStream_t s, const FastJob &job) {
    dec::Params p;
    if (!dec::fill(job, p, true)) return 0;
    return dec::launch<dec::Q80>(s, job, p);
}

}  // namespace nu
