// The planar Q2_K policy of the integer-path skeleton (i8_kernel.cuh): the bytes of a task, the copies that fetch a
// stage, and the mma loop over one task. gemv_q23k_i8.cu has the host side.
//
// A Q2_K superblock (inference/src/quant/decode.zig:260-275) holds 16 groups of 16 two-bit codes, each under a
// four-bit scale and a four-bit minimum: value = d * s_g * q - dmin * m_g. A code times its scale is at most 45 and
// still a byte, so the scale is folded into the codes before the tensor core sees them (one 32-bit multiply scales four
// codes): one int32 accumulator serves the whole superblock, an m16n8k32 step covers two groups, and nothing is
// applied per group afterwards. The minima go through an f16 m16n8k16 step against the group sums of X.
#pragma once
#include "i8_kernel.cuh"

namespace nu {
namespace i8 {

// C += A(16 x 32, unsigned bytes) x B(32 x 8, signed bytes), int32.
__device__ __forceinline__ void imma_u8_acc(int c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct Q2K {
    static constexpr int ROW_BYTES = 80;                     // one planar record: 16 scale bytes, 64 code bytes
    static constexpr int STAGE_SBS = 4;
    static constexpr int ROW_PITCH = STAGE_SBS * ROW_BYTES + 16;  // 336 bytes = 84 words: the eight rows a warp's 4-byte loads touch start
                                                             // 20 banks apart round the banks, all distinct. The 16 bytes more are the
                                                             // row's next bytes.
    static constexpr int MAIN_BYTES = 16 * ROW_PITCH;        // 5,376 = 42 x 128
    static constexpr int STAGE_BYTES = MAIN_BYTES + STAGE_SBS * 64;  // + (d, dmin) of 16 rows per superblock: 5,632 = 44 x 128
    static constexpr int GROUP = 16;
    static constexpr bool GROUP_SUMS = true;                 // the minima meet the sums of X over the groups
    static constexpr int GS_BYTES = 32;                      // sixteen fp16 group sums per superblock and B column
    static constexpr float GS_SCALE = 0.00048828125f;        // 2^-11: a group sum of X (below 2^26) fits fp16
    static constexpr int PLANE_SKEW = 16;
    static constexpr int LANE_BYTES = 4;
    static constexpr float UNIT = 1.0f;

    __device__ static __forceinline__ uint32_t row(uint32_t g) { return g; }

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, STAGE_BYTES);
        tma_load_2d(dst, &p.map[seg], sb * (ROW_BYTES / 4), row0, bar, policy);
        tma_load_2d(dst + MAIN_BYTES, &p.map2[seg], row0, sb, bar, policy);
    }

    // One task (record `part` of the stage): task rows gr and gr + 8 against every B column. Columns 32 m .. 32 m + 31 of
    // the superblock (groups 2m and 2m + 1) are the two-bit field j = m % 4 of the 32 code bytes of half n = m / 4; lane t
    // holds bytes 4t.. (group 2m) and 16 + 4t.. (group 2m + 1), the k order of an m16n8k32.
    template <int NT>
    __device__ static __forceinline__ void task(const uint8_t *stage, uint32_t part, const uint8_t *xb, uint32_t bstep, const uint8_t *gsb, uint32_t gs_step, const float *iv,
                                                const float (&wl)[3], uint32_t gr, uint32_t t, float acc[4]) {
        constexpr bool WIDE = NT == 8;
        constexpr int NC = mma_count<NT>();
        constexpr int STEP = NT == 1 ? 2 : 1;
        const uint8_t *r0 = stage + gr * ROW_PITCH + part * ROW_BYTES, *r1 = r0 + 8 * ROW_PITCH;
        const uint4 h0 = *(const uint4 *)r0, h1 = *(const uint4 *)r1;   // scale (low nibble) and minimum (high nibble) of the 16 groups
        const uint32_t sl0[4] = {h0.x & 0x0f0f0f0fu, h0.y & 0x0f0f0f0fu, h0.z & 0x0f0f0f0fu, h0.w & 0x0f0f0f0fu};
        const uint32_t sl1[4] = {h1.x & 0x0f0f0f0fu, h1.y & 0x0f0f0f0fu, h1.z & 0x0f0f0f0fu, h1.w & 0x0f0f0f0fu};
        int is[NC][4];
#pragma unroll
        for (int j = 0; j < NC; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) is[j][i] = 0;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const uint32_t wa0 = *(const uint32_t *)(r0 + 16 + n * 32 + t * 4), wb0 = *(const uint32_t *)(r0 + 32 + n * 32 + t * 4);
            const uint32_t wa1 = *(const uint32_t *)(r1 + 16 + n * 32 + t * 4), wb1 = *(const uint32_t *)(r1 + 32 + n * 32 + t * 4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int ge = 8 * n + 2 * j, go = ge + 1;   // the two groups; their scales are bytes ge and go of the 16
                const uint32_t e0 = __byte_perm(sl0[ge / 4], 0u, 0x4440 + ge % 4), o0 = __byte_perm(sl0[ge / 4], 0u, 0x4440 + go % 4);
                const uint32_t e1 = __byte_perm(sl1[ge / 4], 0u, 0x4440 + ge % 4), o1 = __byte_perm(sl1[ge / 4], 0u, 0x4440 + go % 4);
                const uint32_t a[4] = {((wa0 >> (2 * j)) & 0x03030303u) * e0, ((wa1 >> (2 * j)) & 0x03030303u) * e1,
                                       ((wb0 >> (2 * j)) & 0x03030303u) * o0, ((wb1 >> (2 * j)) & 0x03030303u) * o1};
#pragma unroll
                for (int jj = 0; jj < NC; ++jj) {
                    const uint32_t b0 = *(const uint32_t *)(xb + jj * bstep + ge * 16), b1 = *(const uint32_t *)(xb + jj * bstep + go * 16);
                    imma_u8_acc(is[jj], a, b0, b1);
                }
            }
        }
        // the minima: sum_g m_g * (group sum of X * 2^-11), pieces hi + lo. A of the f16 step: row r holds its 16 minima,
        // lane t the pairs (2t, 2t + 1) and (8 + 2t, 9 + 2t); a byte b under the exponent byte 0x64 is the fp16 1024 + b.
        const uint32_t sel = (t & 1u) ? 0x4342 : 0x4140;
        const uint32_t ma0 = ((t & 2u) ? h0.y : h0.x) >> 4 & 0x0f0f0f0fu, ma1 = ((t & 2u) ? h1.y : h1.x) >> 4 & 0x0f0f0f0fu;
        const uint32_t mb0 = ((t & 2u) ? h0.w : h0.z) >> 4 & 0x0f0f0f0fu, mb1 = ((t & 2u) ? h1.w : h1.z) >> 4 & 0x0f0f0f0fu;
        const uint32_t a[4] = {hsub2(__byte_perm(ma0, 0x64646464u, sel), 0x64006400u), hsub2(__byte_perm(ma1, 0x64646464u, sel), 0x64006400u),
                               hsub2(__byte_perm(mb0, 0x64646464u, sel), 0x64006400u), hsub2(__byte_perm(mb1, 0x64646464u, sel), 0x64006400u)};
        float cm[4] = {0.f, 0.f, 0.f, 0.f};
        dec::mma16816(cm, a, *(const uint32_t *)gsb, *(const uint32_t *)(gsb + 16));
        if (WIDE) dec::mma16816(cm, a, *(const uint32_t *)(gsb + gs_step), *(const uint32_t *)(gsb + gs_step + 16));
        const float iv0 = iv[0], iv1 = NT == 1 ? 0.0f : iv[1];
        const uint32_t *tail = (const uint32_t *)(stage + MAIN_BYTES) + part * 16;   // (d, dmin) as an f16 pair per row
        const uint32_t dd0 = tail[gr], dd1 = tail[gr + 8];
        const float d0 = __half2float(__ushort_as_half((unsigned short)(dd0 & 0xffffu))), d1 = __half2float(__ushort_as_half((unsigned short)(dd1 & 0xffffu)));
        const float dm0 = -2048.0f * __half2float(__ushort_as_half((unsigned short)(dd0 >> 16))), dm1 = -2048.0f * __half2float(__ushort_as_half((unsigned short)(dd1 >> 16)));
#pragma unroll
        for (int i = 0; i < 4; i += STEP) {
            float f = (float)is[0][i] * wl[0];
#pragma unroll
            for (int j = 1; j < NC; ++j) f = fmaf((float)is[j][i], wl[j], f);
            const float ivi = (i & 1) ? iv1 : iv0;
            acc[i] = fmaf(f, (i < 2 ? d0 : d1) * ivi, acc[i]);
            acc[i] = fmaf(cm[i], (i < 2 ? dm0 : dm1) * ivi, acc[i]);
        }
    }
};

// 16 warps = 4 unit slots x 4 K parts for every number of token rows.
using Q2KPlain = Geometry<16, 4>;

}  // namespace i8
}  // namespace nu
