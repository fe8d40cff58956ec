// Q6_K GEMM for 2..8 token rows on the planar form (prepare.cu), on the shared skeleton
// (rows_kernel.cuh; the scheme is described in gemv_q4k_rows.cu). The reference's kernel for this
// is nu_matvec_rows_q6_k (inference/src/backends/metal/kernels/matvec.metal).
//
// A Q6_K scale is a signed byte per 16 columns and a code has six bits, so code * scale needs 14
// bits and cannot be folded into the fp16 A operand the way Q4_K's 6-bit scales are. Instead a k16
// step of the mma is made to cover exactly one scale group: in step (chunk c, quarter qr) lane t
// of a quad supplies columns 4t..4t+3 of the 16-column group, i.e. word t of the three 16-byte
// pieces of chunk c in the planar record. The step's sums start from zero and are added to the
// task's sums with the group's scale as an F32 factor (four FFMA per step). The bias of 32 goes
// through the tensor core: one m16n8k16 step whose A holds the 16 scales of a row (exact in fp16)
// and whose B holds the 16 group sums of x (times 2^-5 so that they fit fp16, split hi + lo).
// Per superblock and row: out += d * (2^24 * sum_g sc_g * C_g - 1024 * C_bias).
#include "rows_kernel.cuh"

namespace nu {
namespace rows {

struct Q6K {
    static constexpr int ROW_BYTES = 208;               // one planar record
    static constexpr int MAIN_BYTES = 16 * ROW_BYTES;   // 3328
    static constexpr int TASK_BYTES = MAIN_BYTES + 128; // + the 16 super-scales (32 bytes), padded to a multiple of 128
    static constexpr bool SWIZZLED = false;  // whether the task's TMA boxes use a shared-memory swizzle
    static constexpr int AUX_BYTES = 0;
    static constexpr int GS_BYTES = 32;                 // staged group sums per (B column, superblock): sixteen fp16

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, MAIN_BYTES + 32);
        tma_load_2d(dst, &p.map[seg], sb * ROW_BYTES, row0, bar, policy);
        tma_load_2d(dst + MAIN_BYTES, &p.map2[seg], row0 * 2, sb, bar, policy);
    }
    // Float4 ci of a superblock (columns 4ci..4ci+3): half hh, quarter qr, column half ch, word m.
    // Lane m of a quad keeps its 16 steps (chunk 2 hh + ch, quarter qr) as 8 bytes each, 128 bytes in all.
    __device__ static __forceinline__ uint32_t x_offset(uint32_t i) {
        const uint32_t sb = i >> 6, ci = i & 63u;
        const uint32_t hh = ci >> 5, qr = (ci >> 3) & 3u, ch = (ci >> 2) & 1u, m = ci & 3u;
        return (sb * 4 + m) * PITCH + ((hh * 2 + ch) * 4 + qr) * 8;
    }
    // Sum of a 16-column group (four consecutive lanes), times 2^-5, as fp16 pieces, at the place
    // of the group's scale byte (hh * 8 + qr * 2 + ch).
    __device__ static __forceinline__ void group_sum(uint8_t *gs_hi, uint8_t *gs_lo, uint32_t i, float sum, uint32_t lane) {
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((lane & 3) == 0) {
            sum *= 0.03125f;
            const __half sh = __float2half_rn(sum), sl = __float2half_rn(sum - __half2float(sh));
            const uint32_t sb = i >> 6, ci = i & 63u;
            const uint32_t gid = (ci >> 5) * 8 + ((ci >> 3) & 3u) * 2 + ((ci >> 2) & 1u);
            *(__half *)(gs_hi + (sb * 16 + gid) * 2) = sh;
            *(__half *)(gs_lo + (sb * 16 + gid) * 2) = sl;
        }
    }

    // One task: rows g and g+8 of the tile against every token column; see rows_kernel.cuh for the arguments.
    template <bool WIDE>
    __device__ static __forceinline__ void task(const uint8_t *task, const uint8_t *, const uint8_t *xb, uint32_t lo_off, const uint8_t *gsb, uint32_t gs_lo_off, uint32_t g,
                                                uint32_t t, float o[4]) {
        const uint8_t *row[2] = {task + g * ROW_BYTES, task + (g + 8) * ROW_BYTES};
        uint4 sc[2];
        float d[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            sc[h] = *(const uint4 *)(row[h] + 192);
            sc[h].x ^= 0x80808080u; sc[h].y ^= 0x80808080u; sc[h].z ^= 0x80808080u; sc[h].w ^= 0x80808080u;  // scale + 128
            d[h] = __half2float(*(const __half *)(task + MAIN_BYTES + (g + 8 * h) * 2));
        }
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // chunk: half c >> 1 of the superblock, column half c & 1
            uint32_t la[2], lb[2], hb[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                la[h] = *(const uint32_t *)(row[h] + c * 48 + t * 4);       // low nibbles: quarter 0, high nibbles: quarter 2
                lb[h] = *(const uint32_t *)(row[h] + c * 48 + 16 + t * 4);  // quarters 1 and 3
                hb[h] = *(const uint32_t *)(row[h] + c * 48 + 32 + t * 4);  // two high bits of all four quarters
            }
            // the eight steps' activations of this chunk: 32 bytes (two k16 steps per 16 bytes)
            const uint4 b01 = *(const uint4 *)(xb + c * 32), b23 = *(const uint4 *)(xb + c * 32 + 16);
            uint4 l01, l23;
            if (WIDE) {
                l01 = *(const uint4 *)(xb + lo_off + c * 32);
                l23 = *(const uint4 *)(xb + lo_off + c * 32 + 16);
            }
#pragma unroll
            for (int qr = 0; qr < 4; ++qr) {
                uint32_t a[4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t w = (qr & 1) ? lb[h] : la[h];
                    const uint32_t nib = (qr >> 1) ? (w >> 4) : w;
                    const uint32_t top = (qr == 0 ? (hb[h] << 4) : qr == 1 ? (hb[h] << 2) : qr == 2 ? hb[h] : (hb[h] >> 2)) & 0x30303030u;
                    const uint32_t v = (nib & 0x0f0f0f0fu) | top;  // four codes 0..63, one per byte
                    a[h] = __byte_perm(v, 0u, 0x4240);             // columns +0, +2 as fp16 subnormals
                    a[2 + h] = __byte_perm(v, 0u, 0x4341);         // columns +1, +3
                }
                float cs[4] = {0.f, 0.f, 0.f, 0.f};
                const uint4 &bq = qr < 2 ? b01 : b23;
                mma16816(cs, a, (qr & 1) ? bq.z : bq.x, (qr & 1) ? bq.w : bq.y);
                if (WIDE) {
                    const uint4 &lq = qr < 2 ? l01 : l23;
                    mma16816(cs, a, (qr & 1) ? lq.z : lq.x, (qr & 1) ? lq.w : lq.y);
                }
                // scale of group (c >> 1) * 8 + qr * 2 + (c & 1): that byte of the row's 16 scale bytes
                const int gid = (c >> 1) * 8 + qr * 2 + (c & 1);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t sw = (gid >> 2) == 0 ? sc[h].x : (gid >> 2) == 1 ? sc[h].y : (gid >> 2) == 2 ? sc[h].z : sc[h].w;
                    const float s = __uint_as_float(__byte_perm(sw, 0x4b000000u, 0x7650u + (gid & 3))) - 8388736.0f;  // 2^23 + scale + 128
                    acc[2 * h] = fmaf(s, cs[2 * h], acc[2 * h]);
                    acc[2 * h + 1] = fmaf(s, cs[2 * h + 1], acc[2 * h + 1]);
                }
            }
        }
        // the bias: A = the row's scales as fp16 (bytes 2t, 2t+1 and 2t+8, 2t+9), B = the group sums
        uint32_t am[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w_lo = (t >> 1) ? sc[h].y : sc[h].x, w_hi = (t >> 1) ? sc[h].w : sc[h].z;
            const uint32_t p_lo = (t & 1u) ? (w_lo >> 16) : w_lo, p_hi = (t & 1u) ? (w_hi >> 16) : w_hi;
            // a byte b under the exponent byte 0x64 is the fp16 1024 + b; b = scale + 128
            am[h] = hsub2(__byte_perm(p_lo, 0x64646464u, 0x4140), 0x64806480u);
            am[2 + h] = hsub2(__byte_perm(p_hi, 0x64646464u, 0x4140), 0x64806480u);
        }
        float cb[4] = {0.f, 0.f, 0.f, 0.f};
        mma16816(cb, am, *(const uint32_t *)(gsb + t * 4), *(const uint32_t *)(gsb + 16 + t * 4));
        if (WIDE) mma16816(cb, am, *(const uint32_t *)(gsb + gs_lo_off + t * 4), *(const uint32_t *)(gsb + gs_lo_off + 16 + t * 4));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float dq = d[h] * 16777216.0f, db = d[h] * 1024.0f;
#pragma unroll
            for (int cidx = 0; cidx < 2; ++cidx) {
                const int j = 2 * h + cidx;
                o[j] = fmaf(dq, acc[j], o[j]);
                o[j] = fmaf(-db, cb[j], o[j]);
            }
        }
    }
};

static bool fill_q6k(const FastJob &job, Params &p, Plan &plan, bool maps) {
    if (job.enc != Q6_K || job.layout != 1) return false;
    if (!fill_common<Q6K>(job, p, plan)) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows % 16 != 0) return false;
        const uint8_t *dplane = g.w + (size_t)g.rows * p.ksb * 208;
        if (maps && !encode_weight_map(&p.map[s], g.w, (uint64_t)p.ksb * 208, g.rows, (uint64_t)p.ksb * 208, 208, 16)) return false;
        if (maps && !encode_weight_map(&p.map2[s], dplane, (uint64_t)g.rows * 2, p.ksb, (uint64_t)g.rows * 2, 32, 1)) return false;
    }
    return true;
}

}  // namespace rows

bool q6k_rows_configure() { return rows::configure<rows::Q6K>(); }

bool q6k_rows_supported(const FastJob &job) {
    if (job.tokens < 2) return false;
    rows::Params p;
    rows::Plan plan;
    return rows::fill_q6k(job, p, plan, false);
}

int launch_q6k_rows(cudaStream_t s, const FastJob &job) {
    rows::Params p;
    rows::Plan plan;
    if (!rows::fill_q6k(job, p, plan, true)) return 0;
    return rows::launch<rows::Q6K>(s, job, p, plan);
}

}  // namespace nu
