// The Q5_K policy of the integer-path skeleton (i8_kernel.cuh). A Q5_K superblock is a Q4_K superblock with 32 bytes
// of fifth bits between the header and the nibbles (176 bytes, still a multiple of 16, so the GGUF rows are read as
// they are): bit g of byte j of those 32 is the fifth bit of element j of group g
// (inference/src/quant/decode.zig:147-170). gemv_q5k_i8.cu has the host side.
#pragma once
#include "i8_q4k.cuh"

namespace nu {
namespace i8 {

struct Q5K {
    static constexpr int ROW_BYTES = 176;
    static constexpr int STAGE_SBS = 5;
    static constexpr int ROW_PITCH = STAGE_SBS * ROW_BYTES;  // 880 bytes = 220 words: rows two apart lie 24 banks apart, the four rows of a
                                                             // half-warp at 0, 24, 16, 8 (row_of)
    static constexpr int STAGE_BYTES = 16 * ROW_PITCH;       // 14080, a multiple of 128
    static constexpr int GROUP = 32;
    static constexpr bool GROUP_SUMS = true;
    static constexpr int GS_BYTES = 16;
    static constexpr float GS_SCALE = 0.000244140625f;
    static constexpr int PLANE_SKEW = 32;
    static constexpr int LANE_BYTES = 8;
    static constexpr float UNIT = 1.0f;                      // the codes enter as they are: 0..31

    __device__ static __forceinline__ uint32_t row(uint32_t g) { return row_of(g); }

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, STAGE_BYTES);
        tma_load_2d(dst, &p.map[seg], sb * (ROW_BYTES / 4), row0, bar, policy);
    }

    // The fifth bits of group g of four elements (bit g of each byte of h), moved to bit 4 of their bytes.
    __device__ static __forceinline__ uint32_t fifth(uint32_t h, int g) { return (g <= 4 ? h << (4 - g) : h >> (g - 4)) & 0x10101010u; }

    // The arguments are those of Q4K::task. Lane t of a quad holds the group's columns 8t..8t+7: eight nibble bytes
    // per chunk and the eight bytes of fifth bits that serve all eight groups.
    template <int NT>
    __device__ static __forceinline__ void task(const uint8_t *stage, uint32_t part, const uint8_t *xb, uint32_t bstep, const uint8_t *gsb, uint32_t gs_step, const float *iv,
                                                const float (&wl)[3], uint32_t gr, uint32_t t, float acc[4]) {
        const uint8_t *task = stage + part * ROW_BYTES;
        constexpr bool WIDE = NT == 8;
        constexpr int NC = mma_count<NT>();
        constexpr int STEP = NT == 1 ? 2 : 1;
        const uint8_t *r0 = task + gr * ROW_PITCH, *r1 = r0 + 8 * ROW_PITCH;
        const uint4 h0 = *(const uint4 *)r0, h1 = *(const uint4 *)r1;
        const RowInts a = row_ints(h0, t), b = row_ints(h1, t);
        const uint2 f0 = *(const uint2 *)(r0 + 16 + t * 8), f1 = *(const uint2 *)(r1 + 16 + t * 8);
        int is[NC][4];
#pragma unroll
        for (int j = 0; j < NC; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) is[j][i] = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint2 q0 = *(const uint2 *)(r0 + 48 + c * 32 + t * 8), q1 = *(const uint2 *)(r1 + 48 + c * 32 + t * 8);
            const int ge = 2 * c, go = 2 * c + 1;
            const uint32_t ae[4] = {(q0.x & 0x0f0f0f0fu) | fifth(f0.x, ge), (q1.x & 0x0f0f0f0fu) | fifth(f1.x, ge), (q0.y & 0x0f0f0f0fu) | fifth(f0.y, ge),
                                    (q1.y & 0x0f0f0f0fu) | fifth(f1.y, ge)};
            const uint32_t ao[4] = {((q0.x >> 4) & 0x0f0f0f0fu) | fifth(f0.x, go), ((q1.x >> 4) & 0x0f0f0f0fu) | fifth(f1.x, go),
                                    ((q0.y >> 4) & 0x0f0f0f0fu) | fifth(f0.y, go), ((q1.y >> 4) & 0x0f0f0f0fu) | fifth(f1.y, go)};
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                const uint2 be = *(const uint2 *)(xb + j * bstep + ge * 32);
                const uint2 bo = *(const uint2 *)(xb + j * bstep + go * 32);
                int ce[4], co[4];
                imma_u8(ce, ae, be.x, be.y);
                imma_u8(co, ao, bo.x, bo.y);
#pragma unroll
                for (int i = 0; i < 4; i += STEP) {
                    is[j][i] += (i < 2 ? a.s[ge] : b.s[ge]) * ce[i];
                    is[j][i] += (i < 2 ? a.s[go] : b.s[go]) * co[i];
                }
            }
        }
        float cm[4] = {0.f, 0.f, 0.f, 0.f};
        hmma_k8(cm, a.mm, b.mm, *(const uint32_t *)gsb);
        if (WIDE) hmma_k8(cm, a.mm, b.mm, *(const uint32_t *)(gsb + gs_step));
        const float iv0 = iv[0], iv1 = NT == 1 ? 0.0f : iv[1];
        const float dm0 = -4096.0f * a.dmin, dm1 = -4096.0f * b.dmin;
#pragma unroll
        for (int i = 0; i < 4; i += STEP) {
            // sum_g s_g * sum(q * digit) per plane (below 2^27), each plane with the weight of its digits, met in F32
            float f = (float)is[0][i] * wl[0];
#pragma unroll
            for (int j = 1; j < NC; ++j) f = fmaf((float)is[j][i], wl[j], f);
            const float ivi = (i & 1) ? iv1 : iv0;
            acc[i] = fmaf(f, (i < 2 ? a.d : b.d) * ivi, acc[i]);
            acc[i] = fmaf(cm[i], (i < 2 ? dm0 : dm1) * ivi, acc[i]);
        }
    }
};

// 4 unit slots x 5 K parts for one and two tokens, 3 x 5 for the wider forms: the Q4_K geometries.
using Q5KPlain = Geometry<20, 5>;
using Q5KDense = Geometry<15, 5>;

}  // namespace i8
}  // namespace nu
