// The Q4_K policy of the integer-path skeleton (i8_kernel.cuh): the bytes of a task, the copy that fetches a
// stage, and the mma loop over one task. gemv_q4k_i8.cu has the scheme and the host side.
#pragma once
#include "i8_kernel.cuh"

namespace nu {
namespace i8 {

// The integer scales of one superblock row, its minima as an f16 pair for this lane's k slots, d and dmin.
struct RowInts {
    int s[8];
    uint32_t mm;
    float d, dmin;
};
__device__ __forceinline__ RowInts row_ints(const uint4 &hdr, uint32_t t) {
    const uint32_t y = hdr.y, z = hdr.z, w = hdr.w;
    // groups 0..3: low six bits of bytes 0..3 / 4..7; groups 4..7: nibbles of bytes 8..11 plus the top two bits of bytes 0..7
    const uint32_t s_lo = y & 0x3f3f3f3fu, s_hi = (w & 0x0f0f0f0fu) | ((y >> 2) & 0x30303030u);
    const uint32_t m_lo = z & 0x3f3f3f3fu, m_hi = ((w >> 4) & 0x0f0f0f0fu) | ((z >> 2) & 0x30303030u);
    RowInts r;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        r.s[i] = (int)__byte_perm(s_lo, 0u, 0x4440 + i);      // byte i alone: one permute
        r.s[4 + i] = (int)__byte_perm(s_hi, 0u, 0x4440 + i);
    }
    // minima of groups 2t, 2t + 1: a byte b under the exponent byte 0x64 is the fp16 1024 + b
    const uint32_t m4 = t < 2 ? m_lo : m_hi;
    r.mm = hsub2(__byte_perm(m4, 0x64646464u, (t & 1u) ? 0x4342 : 0x4140), 0x64006400u);
    r.d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
    r.dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    return r;
}

struct Q4K {
    static constexpr int ROW_BYTES = 144;                 // one superblock of one row
    static constexpr int STAGE_SBS = 5;                   // superblocks of a row a stage holds: one per warp of a slot
    static constexpr int ROW_PITCH = STAGE_SBS * ROW_BYTES;  // 720 bytes = 180 words between the rows of a stage: rows two apart
                                                          // lie 8 banks apart, which the lanes' 8-byte loads need (row_of)
    static constexpr int STAGE_BYTES = 16 * ROW_PITCH;    // 11520, a multiple of 128
    static constexpr int GROUP = 32;                      // columns per scale group
    static constexpr bool GROUP_SUMS = true;               // the minima / the bias need the sums of X over the scale groups
    static constexpr int GS_BYTES = 16;                   // staged group sums per superblock and B column: eight fp16
    static constexpr float GS_SCALE = 0.000244140625f;    // 2^-12: a group sum of X (below 2^27) fits fp16
    static constexpr int PLANE_SKEW = 32;                 // digit rows 32 bytes apart round the banks: 8-byte loads, 4 lanes a row
    static constexpr int LANE_BYTES = 8;                  // digits a lane supplies per mma: columns 8t..8t+7 of the group
    static constexpr float UNIT = 0.0625f;                // the integer sums carry 16 (high nibbles left in place)

    // One box of 16 rows x 720 bytes. Measured on B200: boxes of 16 x 144 bytes stream at 3.3 TB/s however many are
    // in flight (the copy engine's cost is per row of a box), 16 x 720 bytes at 6.2 TB/s. The tensor map counts in
    // 4-byte elements (a box side is at most 256 elements). Superblocks past the row are filled with zeros.
    __device__ static __forceinline__ uint32_t row(uint32_t g) { return row_of(g); }

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, STAGE_BYTES);
        tma_load_2d(dst, &p.map[seg], sb * (ROW_BYTES / 4), row0, bar, policy);
    }

    // One task (superblock `part` of the stage): task rows gr and gr + 8 against every B column. xb: this lane's digit row at the task's
    // superblock (its 8 bytes of group 0); the digit rows of the next mma lie `bstep` bytes further.
    // gsb: this lane's word of the group sums. iv: 1 / the activation scale of the lane's token(s) at this superblock.
    // acc: (row gr, token a), (gr, a + 1), (gr + 8, a), (gr + 8, a + 1); with one token the odd entries stay untouched.
    template <int NT>
    __device__ static __forceinline__ void task(const uint8_t *stage, uint32_t part, const uint8_t *xb, uint32_t bstep, const uint8_t *gsb, uint32_t gs_step, const float *iv,
                                                const float (&wl)[3], uint32_t gr, uint32_t t, float acc[4]) {
        const uint8_t *task = stage + part * ROW_BYTES;
        constexpr bool WIDE = NT == 8;
        constexpr int NC = mma_count<NT>();
        constexpr int STEP = NT == 1 ? 2 : 1;  // one token: accumulator columns 0 and 2 only
        const uint8_t *r0 = task + gr * ROW_PITCH, *r1 = r0 + 8 * ROW_PITCH;
        const uint4 h0 = *(const uint4 *)r0, h1 = *(const uint4 *)r1;
        const RowInts a = row_ints(h0, t), b = row_ints(h1, t);
        int ie[NC][4], io[NC][4];
#pragma unroll
        for (int j = 0; j < NC; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) ie[j][i] = io[j][i] = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint2 q0 = *(const uint2 *)(r0 + 16 + c * 32 + t * 8), q1 = *(const uint2 *)(r1 + 16 + c * 32 + t * 8);
            const uint32_t ae[4] = {q0.x & 0x0f0f0f0fu, q1.x & 0x0f0f0f0fu, q0.y & 0x0f0f0f0fu, q1.y & 0x0f0f0f0fu};
            const uint32_t ao[4] = {q0.x & 0xf0f0f0f0u, q1.x & 0xf0f0f0f0u, q0.y & 0xf0f0f0f0u, q1.y & 0xf0f0f0f0u};
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                const uint2 be = *(const uint2 *)(xb + j * bstep + (2 * c) * 32);
                const uint2 bo = *(const uint2 *)(xb + j * bstep + (2 * c + 1) * 32);
                int ce[4], co[4];
                imma_u8(ce, ae, be.x, be.y);
                imma_u8(co, ao, bo.x, bo.y);
#pragma unroll
                for (int i = 0; i < 4; i += STEP) {
                    ie[j][i] += (i < 2 ? a.s[2 * c] : b.s[2 * c]) * ce[i];
                    io[j][i] += (i < 2 ? a.s[2 * c + 1] : b.s[2 * c + 1]) * co[i];
                }
            }
        }
        // the minima: sum_g m_g * (group sum of X * 2^-12), pieces hi + lo
        float cm[4] = {0.f, 0.f, 0.f, 0.f};
        hmma_k8(cm, a.mm, b.mm, *(const uint32_t *)gsb);
        if (WIDE) hmma_k8(cm, a.mm, b.mm, *(const uint32_t *)(gsb + gs_step));
        const float iv0 = iv[0], iv1 = NT == 1 ? 0.0f : iv[1];
        const float dm0 = -4096.0f * a.dmin, dm1 = -4096.0f * b.dmin;
#pragma unroll
        for (int i = 0; i < 4; i += STEP) {
            // 16 * sum_g s_g * sum(q * digit) per plane (below 2^29), each plane with the weight of its digits, met in F32
            float f = (float)((ie[0][i] << 4) + io[0][i]) * wl[0];
#pragma unroll
            for (int j = 1; j < NC; ++j) f = fmaf((float)((ie[j][i] << 4) + io[j][i]), wl[j], f);
            const float ivi = (i & 1) ? iv1 : iv0;
            acc[i] = fmaf(f, (i < 2 ? a.d : b.d) * ivi, acc[i]);
            acc[i] = fmaf(cm[i], (i < 2 ? dm0 : dm1) * ivi, acc[i]);
        }
    }
};

// One- and two-token jobs (plain or gate/up pairs) run 20 warps as 4 unit slots x 5 K parts; the wide form
// (three to eight tokens, 128 registers a thread) runs 15 warps as 3 x 5.
using Q4KPlain = Geometry<20, 5>;
using Q4KDense = Geometry<15, 5>;

}  // namespace i8
}  // namespace nu
