// The planar Q8_0 policy of the integer-path skeleton (i8_kernel.cuh): the bytes of a task, the copies that
// fetch a stage, and the mma loop over one task. gemv_q8_0_i8.cu has the scheme and the host side.
#pragma once
#include "i8_kernel.cuh"

namespace nu {
namespace i8 {

struct Q80 {
    static constexpr int ROW_BYTES = 256;                    // the 256 codes of one superblock of one row
    static constexpr int STAGE_SBS = 2;
    static constexpr int ROW_PITCH = STAGE_SBS * ROW_BYTES + 32;  // 544 bytes = 136 words: consecutive rows lie 8 banks apart, which the lanes'
                                                             // 8-byte loads need (rows of exactly 512 bytes would all start in bank 0). The
                                                             // 32 bytes past the stage's codes are the next codes of the row (zeros past it).
    static constexpr int MAIN_BYTES = 16 * ROW_PITCH;        // 8,704 = 68 x 128
    static constexpr int STAGE_BYTES = MAIN_BYTES + STAGE_SBS * 8 * 32;  // + 16 blocks x 16 rows of f16 scales = 9,216
    static constexpr int GROUP = 32;                         // one block
    static constexpr bool GROUP_SUMS = false;                // symmetric codes: nothing to fold into sums of X
    static constexpr int GS_BYTES = 16;                      // (room the skeleton keeps per superblock and column; unused)
    static constexpr float GS_SCALE = 1.0f;
    static constexpr int PLANE_SKEW = 32;                    // digit rows 32 bytes apart round the banks: 8-byte loads, 4 lanes a row
    static constexpr int LANE_BYTES = 8;                     // digits a lane supplies per mma: columns 8t..8t+7 of the block
    static constexpr float UNIT = 1.0f;

    __device__ static __forceinline__ uint32_t row(uint32_t g) { return g; }

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, STAGE_BYTES);
        tma_load_2d(dst, &p.map[seg], sb * (ROW_BYTES / 4), row0, bar, policy);
        tma_load_2d(dst + MAIN_BYTES, &p.map2[seg], row0 * 2, sb * 8, bar, policy);
    }

    // One task (superblock `part` of the stage): task rows gr and gr + 8 against every B column. A block of 32 codes is
    // one m16n8k32 step (signed bytes both sides); its f16 scale multiplies the int32 sums in F32.
    template <int NT>
    __device__ static __forceinline__ void task(const uint8_t *stage, uint32_t part, const uint8_t *xb, uint32_t bstep, const uint8_t *gsb, uint32_t gs_step, const float *iv,
                                                const float (&wl)[3], uint32_t gr, uint32_t t, float acc[4]) {
        constexpr int NC = mma_count<NT>();
        constexpr int STEP = NT == 1 ? 2 : 1;
        const uint8_t *r0 = stage + gr * ROW_PITCH + part * ROW_BYTES + t * 8, *r1 = r0 + 8 * ROW_PITCH;
        const __half *dsc = (const __half *)(stage + MAIN_BYTES) + part * 8 * 16 + gr;  // [block][16 rows]
        float f[NC][4];
#pragma unroll
        for (int j = 0; j < NC; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) f[j][i] = 0.0f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint2 q0 = *(const uint2 *)(r0 + c * 32), q1 = *(const uint2 *)(r1 + c * 32);
            const uint32_t a[4] = {q0.x, q1.x, q0.y, q1.y};
            const float d0 = __half2float(dsc[c * 16]), d1 = __half2float(dsc[c * 16 + 8]);
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                const uint2 b = *(const uint2 *)(xb + j * bstep + c * 32);
                int s[4];
                imma_s8(s, a, b.x, b.y);
#pragma unroll
                for (int i = 0; i < 4; i += STEP) f[j][i] = fmaf((float)s[i], i < 2 ? d0 : d1, f[j][i]);
            }
        }
        (void)gsb; (void)gs_step;
        const float iv0 = iv[0], iv1 = NT == 1 ? 0.0f : iv[1];
#pragma unroll
        for (int i = 0; i < 4; i += STEP) {
            float v = f[0][i] * wl[0];
#pragma unroll
            for (int j = 1; j < NC; ++j) v = fmaf(f[j][i], wl[j], v);
            acc[i] = fmaf(v, (i & 1) ? iv1 : iv0, acc[i]);
        }
    }
};

// 12 warps = 6 unit slots x 2 K parts (three stages of 9 KB a slot keep 110 KB in flight beside the digit rows); the same
// for the forms with more token rows.
using Q80Plain = Geometry<12, 2>;

}  // namespace i8
}  // namespace nu
