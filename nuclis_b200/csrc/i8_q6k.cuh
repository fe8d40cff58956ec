// The planar Q6_K policy of the integer-path skeleton (i8_kernel.cuh): the bytes of a task, the copies that
// fetch a stage, and the mma loop over one task. gemv_q6k_i8.cu has the scheme and the host side.
#pragma once
#include "i8_kernel.cuh"

namespace nu {
namespace i8 {

__device__ __forceinline__ void imma_k16_u8(int c[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// Byte k of w as a sign-extended int: one permute (a selector nibble with its top bit set copies the sign).
template <int K>
__device__ __forceinline__ int sbyte(uint32_t w) {
    // prmt by name: selector nibbles with bit 3 set replicate the byte's sign, which the byte-permute intrinsic masks off
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "n"(((8 | K) << 12) | ((8 | K) << 8) | ((8 | K) << 4) | K));
    return (int)r;
}
// Bytes 2h and 2h + 1 of w (int8) as an f16 pair: biased to 0..255 they sit under the exponent byte 0x64 as 1024 + b.
__device__ __forceinline__ uint32_t scale_pair(uint32_t w, uint32_t h) {
    return hsub2(__byte_perm(w ^ 0x80808080u, 0x64646464u, h ? 0x4342 : 0x4140), 0x64806480u);
}

struct Q6K {
    static constexpr int ROW_BYTES = 208;                    // one planar record
    static constexpr int STAGE_SBS = 3;
    static constexpr int ROW_PITCH = STAGE_SBS * ROW_BYTES;  // 624
    static constexpr int MAIN_BYTES = 16 * ROW_PITCH;        // 9,984 = 78 x 128
    static constexpr int STAGE_BYTES = MAIN_BYTES + 128;     // + the 3 x 16 super-scales (96 bytes)
    static constexpr int GROUP = 16;
    static constexpr bool GROUP_SUMS = true;               // the minima / the bias need the sums of X over the scale groups
    static constexpr int GS_BYTES = 32;                      // sixteen fp16 group sums per superblock and B column
    static constexpr float GS_SCALE = 0.00048828125f;        // 2^-11: a group sum of X (below 2^26) fits fp16
    static constexpr int PLANE_SKEW = 16;
    static constexpr int LANE_BYTES = 4;
    static constexpr float UNIT = 1.0f;

    __device__ static __forceinline__ uint32_t row(uint32_t g) { return row_of(g); }

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, MAIN_BYTES + STAGE_SBS * 32);
        tma_load_2d(dst, &p.map[seg], sb * (ROW_BYTES / 4), row0, bar, policy);
        tma_load_2d(dst + MAIN_BYTES, &p.map2[seg], row0 * 2, sb, bar, policy);
    }

    // One task (record `part` of the stage): task rows gr and gr + 8 against every B column. xb: this lane's four
    // bytes of group 0 in its digit row; gsb: its first word of the group sums (the second lies 16 bytes further).
    template <int NT>
    __device__ static __forceinline__ void task(const uint8_t *stage, uint32_t part, const uint8_t *xb, uint32_t bstep, const uint8_t *gsb, uint32_t gs_step, const float *iv,
                                                const float (&wl)[3], uint32_t gr, uint32_t t, float acc[4]) {
        constexpr bool WIDE = NT == 8;
        constexpr int NC = mma_count<NT>();
        constexpr int STEP = NT == 1 ? 2 : 1;
        const uint8_t *r0 = stage + gr * ROW_PITCH + part * ROW_BYTES, *r1 = r0 + 8 * ROW_PITCH;
        int acci[NC][4];
#pragma unroll
        for (int j = 0; j < NC; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acci[j][i] = 0;
#pragma unroll
        for (int tb = 0; tb < 4; ++tb) {  // (half, column half) of the superblock: the record's 48-byte chunk
            // the eight group scales of this half of the superblock (registers are short: they are read again per half, and
            // once more for the bias below, rather than kept)
            const uint2 sc0 = *(const uint2 *)(r0 + 192 + (tb >> 1) * 8), sc1 = *(const uint2 *)(r1 + 192 + (tb >> 1) * 8);
            const uint32_t la0 = *(const uint32_t *)(r0 + tb * 48 + t * 4), lb0 = *(const uint32_t *)(r0 + tb * 48 + 16 + t * 4), hb0 = *(const uint32_t *)(r0 + tb * 48 + 32 + t * 4);
            const uint32_t la1 = *(const uint32_t *)(r1 + tb * 48 + t * 4), lb1 = *(const uint32_t *)(r1 + tb * 48 + 16 + t * 4), hb1 = *(const uint32_t *)(r1 + tb * 48 + 32 + t * 4);
#pragma unroll
            for (int qr = 0; qr < 4; ++qr) {
                const uint32_t lo0 = (qr & 1) ? lb0 : la0, lo1 = (qr & 1) ? lb1 : la1;
                const uint32_t n0 = (qr >> 1) ? lo0 >> 4 : lo0, n1 = (qr >> 1) ? lo1 >> 4 : lo1;
                const uint32_t h0 = qr == 0 ? hb0 << 4 : qr == 1 ? hb0 << 2 : qr == 2 ? hb0 : hb0 >> 2;
                const uint32_t h1 = qr == 0 ? hb1 << 4 : qr == 1 ? hb1 << 2 : qr == 2 ? hb1 : hb1 >> 2;
                const uint32_t v0 = (n0 & 0x0f0f0f0fu) | (h0 & 0x30303030u), v1 = (n1 & 0x0f0f0f0fu) | (h1 & 0x30303030u);
                const int gi = (tb >> 1) * 8 + qr * 2 + (tb & 1);  // the group's index in the row: columns 16 gi .. 16 gi + 15
                const uint32_t w0 = (gi & 7) < 4 ? sc0.x : sc0.y, w1 = (gi & 7) < 4 ? sc1.x : sc1.y;
                const int s0 = (gi & 3) == 0 ? sbyte<0>(w0) : (gi & 3) == 1 ? sbyte<1>(w0) : (gi & 3) == 2 ? sbyte<2>(w0) : sbyte<3>(w0);
                const int s1 = (gi & 3) == 0 ? sbyte<0>(w1) : (gi & 3) == 1 ? sbyte<1>(w1) : (gi & 3) == 2 ? sbyte<2>(w1) : sbyte<3>(w1);
#pragma unroll
                for (int j = 0; j < NC; ++j) {
                    const uint32_t b = *(const uint32_t *)(xb + j * bstep + gi * 16);
                    int c[4];
                    imma_k16_u8(c, v0, v1, b);
#pragma unroll
                    for (int i = 0; i < 4; i += STEP) acci[j][i] += (i < 2 ? s0 : s1) * c[i];
                }
            }
        }
        // the bias: sum_g sc_g * (group sum of X * 2^-11), pieces hi + lo
        // A of the f16 step: row r holds its 16 scales, lane t the pairs (2t, 2t + 1) and (8 + 2t, 9 + 2t): bytes 2t.. of each half
        const uint32_t sw0 = *(const uint32_t *)(r0 + 192 + (t >> 1) * 4), sw1 = *(const uint32_t *)(r1 + 192 + (t >> 1) * 4);
        const uint32_t sw2 = *(const uint32_t *)(r0 + 200 + (t >> 1) * 4), sw3 = *(const uint32_t *)(r1 + 200 + (t >> 1) * 4);
        const uint32_t a[4] = {scale_pair(sw0, t & 1u), scale_pair(sw1, t & 1u), scale_pair(sw2, t & 1u), scale_pair(sw3, t & 1u)};
        float cm[4] = {0.f, 0.f, 0.f, 0.f};
        dec::mma16816(cm, a, *(const uint32_t *)gsb, *(const uint32_t *)(gsb + 16));
        if (WIDE) dec::mma16816(cm, a, *(const uint32_t *)(gsb + gs_step), *(const uint32_t *)(gsb + gs_step + 16));
        const float iv0 = iv[0], iv1 = NT == 1 ? 0.0f : iv[1];
        const __half *dsc = (const __half *)(stage + MAIN_BYTES) + part * 16;
        const float d0 = __half2float(dsc[gr]), d1 = __half2float(dsc[gr + 8]);
#pragma unroll
        for (int i = 0; i < 4; i += STEP) {
            float f = (float)acci[0][i] * wl[0];
#pragma unroll
            for (int j = 1; j < NC; ++j) f = fmaf((float)acci[j][i], wl[j], f);
            const float ivi = (i & 1) ? iv1 : iv0, d = i < 2 ? d0 : d1;
            acc[i] = fmaf(f, d * ivi, acc[i]);
            acc[i] = fmaf(cm[i], -65536.0f * d * ivi, acc[i]);  // 32 * 2^11
        }
    }
};

// 18 warps = 6 unit slots x 3 K parts; the wide form (three to eight tokens) 15 = 5 x 3.
using Q6KPlain = Geometry<18, 3>;
using Q6KDense = Geometry<15, 3>;

}  // namespace i8
}  // namespace nu
