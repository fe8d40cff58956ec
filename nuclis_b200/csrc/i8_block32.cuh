// The policy of the integer-path skeleton (i8_kernel.cuh) for the planar forms of the encodings made of 32-element
// blocks under an f16 scale: Q5_0, Q5_1, Q4_0 and IQ4_NL, and for IQ4_XS (IQ4_NL's codes, eight blocks under one f16
// scale and eight six-bit ones). The bytes of a task, the copies that fetch a stage, and the
// mma loop over one task. gemv_block32_i8.cu has the scheme and the host side.
#pragma once
#include "i8_kernel.cuh"

namespace nu {
namespace i8 {

// The eight six-bit scales of an IQ4_XS superblock row (decode.zig:214-228: block g has four bits in nibble g of the
// header's second word and two bits at 2g of the first word's upper half) as bytes: blocks 0, 2, 4, 6 in even,
// 1, 3, 5, 7 in odd.
__device__ __forceinline__ void xs_scales(const uint2 &hdr, uint32_t &even, uint32_t &odd) {
    uint32_t h = hdr.x >> 16;                // nibble k: the top bits of blocks 2k (low pair) and 2k + 1 (high pair)
    h = (h | (h << 8)) & 0x00ff00ffu;
    h = (h | (h << 4)) & 0x0f0f0f0fu;        // nibble k now in byte k
    even = (hdr.y & 0x0f0f0f0fu) | ((h & 0x03030303u) << 4);
    odd = ((hdr.y >> 4) & 0x0f0f0f0fu) | ((h & 0x0c0c0c0cu) << 2);
}

enum Block32Kind : int { KIND_Q5_0 = 0, KIND_Q5_1 = 1, KIND_Q4_0 = 2, KIND_IQ4_NL = 3, KIND_IQ4_XS = 4 };

// Q5_1: value = d * q + m; Q5_0: d * (q - 16); Q4_0: d * (q - 8); IQ4_NL: d * table[q]; IQ4_XS: d * (s - 32) * table[q].
template <int KIND>
struct Block32 {
    static constexpr bool FIFTH = KIND == KIND_Q5_0 || KIND == KIND_Q5_1;   // a plane of fifth bits follows the nibbles
    static constexpr bool OFFSET = KIND == KIND_Q5_1;
    static constexpr bool TABLE = KIND == KIND_IQ4_NL || KIND == KIND_IQ4_XS;
    static constexpr bool SUPER = KIND == KIND_IQ4_XS;       // the header of a superblock row: d, two bits of each scale, four bits of each
    static constexpr int ROW_BYTES = FIFTH ? 160 : 128;      // one planar record: 8 x 16 nibble bytes (then 8 x 4 bytes of high bits)
    static constexpr int STAGE_SBS = 2;
    static constexpr int ROW_PITCH = STAGE_SBS * ROW_BYTES + 16;  // 336 (272) bytes = 84 (68) words: the eight rows a warp's 4-byte
                                                             // loads touch start 20 (4) banks apart round the banks, all distinct
                                                             // (320 or 256 would put them 16 or 0 apart). The 16 bytes more are the
                                                             // row's next bytes.
    static constexpr int MAIN_BYTES = 16 * ROW_PITCH;        // 5,376 = 42 x 128 (4,352 = 34 x 128)
    static constexpr int SC_ROW = OFFSET ? 32 : SUPER ? 8 : 16;  // scale bytes per row and superblock: eight d (and eight m); the IQ4_XS header
    static constexpr int STAGE_BYTES = MAIN_BYTES + STAGE_SBS * 16 * SC_ROW;
    static constexpr int GROUP = 32;                         // one block
    static constexpr bool GROUP_SUMS = !TABLE;               // the offset (16 d, 8 d, or m) meets the sums of X over the blocks
    static constexpr int GS_BYTES = 16;                      // staged group sums per superblock and B column: eight fp16
    static constexpr float GS_SCALE = 0.000244140625f;       // 2^-12: a group sum of X (below 2^27) fits fp16
    static constexpr int PLANE_SKEW = 16;                    // digit rows 16 bytes apart round the banks: 4-byte loads, 4 lanes a row
    static constexpr int LANE_BYTES = 4;                     // digits a lane supplies per mma: columns 4t..4t+3 and 16+4t..16+4t+3 of the block
    static constexpr float UNIT = 1.0f;

    __device__ static __forceinline__ uint32_t row(uint32_t g) { return g; }

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, STAGE_BYTES);
        tma_load_2d(dst, &p.map[seg], sb * (ROW_BYTES / 4), row0, bar, policy);
        tma_load_2d(dst + MAIN_BYTES, &p.map2[seg], row0 * (SC_ROW / 4), sb, bar, policy);
    }

    // One task (record `part` of the stage): task rows gr and gr + 8 against every B column. A block of 32 codes is one
    // m16n8k32 step: byte i of the block's 16 nibble bytes holds column i in its low and column 16 + i in its high nibble,
    // which is exactly how the mma's k index runs over a lane's two operand words (k = 4t.. and 16 + 4t..), so one 32-bit
    // load feeds both; the fifth bits come from the block's 32-bit plane, four at a time. The f16 block scale multiplies
    // the int32 sums in F32; the offset goes through an m16n8k8 f16 step against the group sums of X.
    // IQ4_NL: the table lookup leaves the values of a half-word's nibbles in nibble order (columns 4t, 16 + 4t, 4t + 1,
    // 16 + 4t + 1); the order of k inside an mma is free as long as both operands share it, so the two digit words are
    // permuted the same way (two permutes per block and plane instead of two per row).
    template <int NT>
    __device__ static __forceinline__ void task(const uint8_t *stage, uint32_t part, const uint8_t *xb, uint32_t bstep, const uint8_t *gsb, uint32_t gs_step, const float *iv,
                                                const float (&wl)[3], uint32_t gr, uint32_t t, float acc[4]) {
        constexpr bool WIDE = NT == 8;
        constexpr int NC = mma_count<NT>();
        constexpr int STEP = NT == 1 ? 2 : 1;
        const uint8_t *r0 = stage + gr * ROW_PITCH + part * ROW_BYTES, *r1 = r0 + 8 * ROW_PITCH;
        const uint8_t *sc0 = stage + MAIN_BYTES + (part * 16 + gr) * SC_ROW, *sc1 = sc0 + 8 * SC_ROW;
        uint2 hd0 = make_uint2(0u, 0u), hd1 = hd0;
        uint32_t se0 = 0, so0 = 0, se1 = 0, so1 = 0;  // the six-bit scales of the even and of the odd blocks, a byte each
        if (SUPER) {
            hd0 = *(const uint2 *)sc0, hd1 = *(const uint2 *)sc1;
            xs_scales(hd0, se0, so0);
            xs_scales(hd1, se1, so1);
        }
        float f[NC][4];
#pragma unroll
        for (int j = 0; j < NC; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) f[j][i] = 0.0f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint32_t n0 = *(const uint32_t *)(r0 + c * 16 + t * 4), n1 = *(const uint32_t *)(r1 + c * 16 + t * 4);
            uint32_t a[4];
            if (TABLE) {
                a[0] = iq4_lookup4(n0), a[1] = iq4_lookup4(n1), a[2] = iq4_lookup4(n0 >> 16), a[3] = iq4_lookup4(n1 >> 16);
            } else {
                a[0] = n0 & 0x0f0f0f0fu, a[1] = n1 & 0x0f0f0f0fu, a[2] = (n0 >> 4) & 0x0f0f0f0fu, a[3] = (n1 >> 4) & 0x0f0f0f0fu;
            }
            if (FIFTH) {
                const uint32_t h0 = *(const uint32_t *)(r0 + 128 + c * 4) >> (4 * t), h1 = *(const uint32_t *)(r1 + 128 + c * 4) >> (4 * t);
                a[0] |= bits4_to_bit4(h0 & 15u), a[1] |= bits4_to_bit4(h1 & 15u), a[2] |= bits4_to_bit4((h0 >> 16) & 15u), a[3] |= bits4_to_bit4((h1 >> 16) & 15u);
            }
            float d0, d1;
            if (SUPER) {
                // byte c / 2 of the even or odd scales as a float through the 2^23 magic number, minus 32
                d0 = __uint_as_float(prmt_b32((c & 1) ? so0 : se0, 0x4b000000u, 0x7650u + c / 2)) - 8388640.0f;
                d1 = __uint_as_float(prmt_b32((c & 1) ? so1 : se1, 0x4b000000u, 0x7650u + c / 2)) - 8388640.0f;
            } else {
                d0 = __half2float(*(const __half *)(sc0 + c * 2)), d1 = __half2float(*(const __half *)(sc1 + c * 2));
            }
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                const uint32_t b0 = *(const uint32_t *)(xb + j * bstep + c * 32), b1 = *(const uint32_t *)(xb + j * bstep + c * 32 + 16);
                int s[4];
                if (TABLE) imma_s8(s, a, prmt_b32(b0, b1, 0x5140u), prmt_b32(b0, b1, 0x7362u));
                else imma_u8(s, a, b0, b1);
#pragma unroll
                for (int i = 0; i < 4; i += STEP) f[j][i] = fmaf((float)s[i], i < 2 ? d0 : d1, f[j][i]);
            }
        }
        // the offset: sum_c coef_c * (group sum of X * 2^-12), pieces hi + lo; coef = m (Q5_1) or d (times -16 or -8 below)
        float cm[4] = {0.f, 0.f, 0.f, 0.f};
        if (GROUP_SUMS) {
            const uint32_t m0 = *(const uint32_t *)(sc0 + (OFFSET ? 16 : 0) + t * 4), m1 = *(const uint32_t *)(sc1 + (OFFSET ? 16 : 0) + t * 4);
            hmma_k8(cm, m0, m1, *(const uint32_t *)gsb);
            if (WIDE) hmma_k8(cm, m0, m1, *(const uint32_t *)(gsb + gs_step));
        }
        const float iv0 = iv[0], iv1 = NT == 1 ? 0.0f : iv[1];
        constexpr float OFF = OFFSET ? 4096.0f : KIND == KIND_Q5_0 ? -65536.0f : -32768.0f;  // 2^12, times -16 for Q5_0, -8 for Q4_0
#pragma unroll
        for (int i = 0; i < 4; i += STEP) {
            float v = f[0][i] * wl[0];
#pragma unroll
            for (int j = 1; j < NC; ++j) v = fmaf(f[j][i], wl[j], v);
            const float ivi = (i & 1) ? iv1 : iv0;
            if (SUPER) v *= __half2float(__ushort_as_half((unsigned short)((i < 2 ? hd0.x : hd1.x) & 0xffffu)));
            acc[i] = fmaf(v, ivi, acc[i]);
            if (GROUP_SUMS) acc[i] = fmaf(cm[i], OFF * ivi, acc[i]);
        }
    }
};

// 16 warps = 8 unit slots x 2 K parts for every number of token rows (the task is heavy on unpacking: 12 warps left the
// issue slots a third idle: 18.9 us for Q5_0 17408 x 5120 at one token, 17.6 with 16).
using Block32Plain = Geometry<16, 2>;

}  // namespace i8
}  // namespace nu
