// The planar Q3_K policy of the integer-path skeleton (i8_kernel.cuh): the bytes of a task, the copies that fetch a
// stage, and the mma loop over one task. gemv_q23k_i8.cu has the host side.
//
// A Q3_K superblock (inference/src/quant/decode.zig:174-196) holds 16 groups of 16 codes: two low bits in the code
// bytes, a third bit in a mask plane (clear means subtract four), under a six-bit scale biased by 32:
// value = d * (s_g - 32) * (c - 4) with c = low | bit << 2 in 0..7. This is Q6_K's shape (signed group scales, unsigned
// codes, a bias through the group sums of X) with another way of assembling the codes: one m16n8k16 step per group,
// the scale on the int32 sums, the bias -4 (s_g - 32) sum(X_g) through an f16 m16n8k16 step.
#pragma once
#include "i8_q6k.cuh"

namespace nu {
namespace i8 {

// The sixteen scales of a row, minus 32, as signed bytes: s[k] holds groups 4k .. 4k + 3. w0, w1: the low nibbles of
// groups 0..7 and, in the high nibbles, of groups 8..15; w2: byte k holds the top two bits of groups k, k + 4, k + 8, k + 12.
__device__ __forceinline__ void q3k_scales(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t s[4]) {
    const uint32_t x[4] = {(w0 & 0x0f0f0f0fu) | ((w2 << 4) & 0x30303030u), (w1 & 0x0f0f0f0fu) | ((w2 << 2) & 0x30303030u),
                           ((w0 >> 4) & 0x0f0f0f0fu) | (w2 & 0x30303030u), ((w1 >> 4) & 0x0f0f0f0fu) | ((w2 >> 2) & 0x30303030u)};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        // x - 32 for a six-bit x, byte by byte: flip bit 5; where it is now set (x was below 32) the byte is negative: set bits 6 and 7
        const uint32_t f = x[k] ^ 0x20202020u;
        s[k] = f | ((f & 0x20202020u) * 6u);
    }
}

struct Q3K {
    static constexpr int ROW_BYTES = 96;                     // one planar record: 32 mask bytes, 64 code bytes
    static constexpr int STAGE_SBS = 4;
    static constexpr int ROW_PITCH = STAGE_SBS * ROW_BYTES + 16;  // 400 bytes = 100 words: the eight rows a warp's 4-byte loads touch start
                                                             // 4 banks apart, all distinct. The 16 bytes more are the row's next bytes.
    static constexpr int MAIN_BYTES = 16 * ROW_PITCH;        // 6,400 = 50 x 128
    static constexpr int TAIL_BYTES = 224;                   // per superblock and 16 rows: 16 x 12 scale bytes, then 16 f16 d
    static constexpr int STAGE_BYTES = MAIN_BYTES + STAGE_SBS * TAIL_BYTES;  // 7,296 = 57 x 128
    static constexpr int GROUP = 16;
    static constexpr bool GROUP_SUMS = true;
    static constexpr int GS_BYTES = 32;
    static constexpr float GS_SCALE = 0.00048828125f;        // 2^-11
    static constexpr int PLANE_SKEW = 16;
    static constexpr int LANE_BYTES = 4;
    static constexpr float UNIT = 1.0f;

    __device__ static __forceinline__ uint32_t row(uint32_t g) { return g; }

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, STAGE_BYTES);
        tma_load_2d(dst, &p.map[seg], sb * (ROW_BYTES / 4), row0, bar, policy);
        tma_load_2d(dst + MAIN_BYTES, &p.map2[seg], (row0 / 16) * (TAIL_BYTES / 4), sb, bar, policy);
    }

    // One task (record `part` of the stage): task rows gr and gr + 8 against every B column. Group gi (columns 16 gi ..)
    // is the two-bit field (gi % 8) / 2 of code bytes 32 (gi / 8) + 16 (gi % 2) .., with bit gi / 2 of mask bytes 16 (gi % 2) ..
    template <int NT>
    __device__ static __forceinline__ void task(const uint8_t *stage, uint32_t part, const uint8_t *xb, uint32_t bstep, const uint8_t *gsb, uint32_t gs_step, const float *iv,
                                                const float (&wl)[3], uint32_t gr, uint32_t t, float acc[4]) {
        constexpr bool WIDE = NT == 8;
        constexpr int NC = mma_count<NT>();
        constexpr int STEP = NT == 1 ? 2 : 1;
        const uint8_t *r0 = stage + gr * ROW_PITCH + part * ROW_BYTES, *r1 = r0 + 8 * ROW_PITCH;
        const uint8_t *tail = stage + MAIN_BYTES + part * TAIL_BYTES;
        const uint32_t *tw0 = (const uint32_t *)(tail + gr * 12), *tw1 = (const uint32_t *)(tail + (gr + 8) * 12);
        uint32_t s0[4], s1[4];
        q3k_scales(tw0[0], tw0[1], tw0[2], s0);
        q3k_scales(tw1[0], tw1[1], tw1[2], s1);
        int acci[NC][4];
#pragma unroll
        for (int j = 0; j < NC; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acci[j][i] = 0;
#pragma unroll
        for (int half = 0; half < 2; ++half) {  // the column half of a 32-column chunk: bytes 16 half .. of the mask and code planes
            const uint32_t m0 = *(const uint32_t *)(r0 + half * 16 + t * 4), m1 = *(const uint32_t *)(r1 + half * 16 + t * 4);
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const uint32_t q0 = *(const uint32_t *)(r0 + 32 + n * 32 + half * 16 + t * 4), q1 = *(const uint32_t *)(r1 + 32 + n * 32 + half * 16 + t * 4);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int gi = 8 * n + 2 * j + half, bit = 4 * n + j;   // the mask bit of this group's 32-column chunk
                    const uint32_t k0 = bit <= 2 ? m0 << (2 - bit) : m0 >> (bit - 2), k1 = bit <= 2 ? m1 << (2 - bit) : m1 >> (bit - 2);
                    const uint32_t v0 = ((q0 >> (2 * j)) & 0x03030303u) | (k0 & 0x04040404u), v1 = ((q1 >> (2 * j)) & 0x03030303u) | (k1 & 0x04040404u);
                    const uint32_t w0 = s0[gi / 4], w1 = s1[gi / 4];
                    const int c0 = (gi & 3) == 0 ? sbyte<0>(w0) : (gi & 3) == 1 ? sbyte<1>(w0) : (gi & 3) == 2 ? sbyte<2>(w0) : sbyte<3>(w0);
                    const int c1 = (gi & 3) == 0 ? sbyte<0>(w1) : (gi & 3) == 1 ? sbyte<1>(w1) : (gi & 3) == 2 ? sbyte<2>(w1) : sbyte<3>(w1);
#pragma unroll
                    for (int jj = 0; jj < NC; ++jj) {
                        const uint32_t b = *(const uint32_t *)(xb + jj * bstep + gi * 16);
                        int c[4];
                        imma_k16_u8(c, v0, v1, b);
#pragma unroll
                        for (int i = 0; i < 4; i += STEP) acci[jj][i] += (i < 2 ? c0 : c1) * c[i];
                    }
                }
            }
        }
        // the bias: sum_g (s_g - 32) * (group sum of X * 2^-11), pieces hi + lo, times -4
        const bool up = (t & 2u) != 0;   // selects, not indexing: the scale words stay in registers
        const uint32_t a[4] = {scale_pair(up ? s0[1] : s0[0], t & 1u), scale_pair(up ? s1[1] : s1[0], t & 1u), scale_pair(up ? s0[3] : s0[2], t & 1u), scale_pair(up ? s1[3] : s1[2], t & 1u)};
        float cm[4] = {0.f, 0.f, 0.f, 0.f};
        dec::mma16816(cm, a, *(const uint32_t *)gsb, *(const uint32_t *)(gsb + 16));
        if (WIDE) dec::mma16816(cm, a, *(const uint32_t *)(gsb + gs_step), *(const uint32_t *)(gsb + gs_step + 16));
        const float iv0 = iv[0], iv1 = NT == 1 ? 0.0f : iv[1];
        const __half *dsc = (const __half *)(tail + 192);
        const float d0 = __half2float(dsc[gr]), d1 = __half2float(dsc[gr + 8]);
#pragma unroll
        for (int i = 0; i < 4; i += STEP) {
            float f = (float)acci[0][i] * wl[0];
#pragma unroll
            for (int j = 1; j < NC; ++j) f = fmaf((float)acci[j][i], wl[j], f);
            const float ivi = (i & 1) ? iv1 : iv0, d = i < 2 ? d0 : d1;
            acc[i] = fmaf(f, d * ivi, acc[i]);
            acc[i] = fmaf(cm[i], -8192.0f * d * ivi, acc[i]);  // 4 * 2^11
        }
    }
};

// 16 warps = 4 unit slots x 4 K parts for every number of token rows.
using Q3KPlain = Geometry<16, 4>;

}  // namespace i8
}  // namespace nu
