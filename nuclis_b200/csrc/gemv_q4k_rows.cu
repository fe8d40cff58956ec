// Q4_K GEMM for 2..8 token rows (the speculative-verify batch) for sm_100a: the kernel behind
// Backend.matvecRows and small Backend.matmul on Q4_K weights
// (inference/src/backends/metal/ops/matvec.zig:119-188; the reference's kernel for this is
// nu_matvec_rows_q4_k, kernels/matvec.metal). Every weight byte is read once for all token rows.
//
// It shares the decode GEMV's machinery (decode_kernel.cuh: a task is 16 weight rows by one
// superblock, fetched by one TMA tensor copy into a per-warp ring of stages; the 4-bit codes are
// fp16 subnormals in place; activations are scaled by a power of two per token row and split into
// fp16 pieces hi + lo; products are exact and accumulate in F32 on the tensor cores). What differs:
//
//  * The 8 columns of the mma B operand are taken by the tokens (2..4 tokens: column 2*token + piece;
//    5..8 tokens: one mma with the hi pieces and one with the lo pieces), so a k16 step mixes the
//    codes of the four lanes of a quad, which belong to four different scale groups. The group
//    scale is therefore folded into the A operand: code * 2^-24 times the 6-bit scale is still an
//    exact fp16 value (at most 945 * 2^-24), one HMUL2 per register, and a single accumulator
//    serves the whole superblock. High nibbles, which sit at 2^-20, take scale / 16 (exact).
//  * The minima go through the tensor core too: an m16n8k8 step whose A holds the eight 6-bit minima
//    of a row and whose B holds the eight group sums of x (times 2^-6 so that they fit fp16, split
//    hi + lo like x). Per superblock and row: out += d * 2^24 * C_q - dmin * 2^6 * C_m.
//  * Eight token rows of staged activations take 32 bytes per column, so a block stages the window
//    of one K slice only, and no block spans two slices: each slice owns a range of blocks (sized
//    by the host so that all finish together) which split the slice's row tiles evenly.
//  * The four warps that share a unit (K parts) meet at a named barrier of their own and the first
//    of them adds the parts in order and writes the outputs, or, with several slices, the partial
//    sums; the last block to arrive for a row tile adds the slices in order. No block-wide barrier
//    in the main loop, no sum that depends on timing.
#include "rows_kernel.cuh"

namespace nu {
namespace rows {

// Scales of one row for this lane's group pair t, as fp16 pairs ready for the A operand:
// {s_even, s_even}, {s_odd / 16, s_odd / 16}, {m_even, m_odd}.
struct RowScales {
    uint32_t se2, so2, mm;
};
__device__ __forceinline__ RowScales row_scales(const uint4 &hdr, uint32_t t) {
    const uint32_t shift = (t & 1u) * 16;
    const uint32_t y = (hdr.y >> shift) & 0xffffu, z = (hdr.z >> shift) & 0xffffu, w = (hdr.w >> shift) & 0xffffu;
    // groups 0..3: low six bits of bytes 0..3 / 4..7; groups 4..7: nibbles of bytes 8..11 plus the top two bits of bytes 0..7
    const uint32_t s_lo = y & 0x3f3fu, m_lo = z & 0x3f3fu;
    const uint32_t s_hi = (w & 0x0f0fu) | ((y >> 2) & 0x3030u), m_hi = ((w >> 4) & 0x0f0fu) | ((z >> 2) & 0x3030u);
    const uint32_t s2 = t < 2 ? s_lo : s_hi, m2 = t < 2 ? m_lo : m_hi;
    RowScales r;
    // a byte b under the exponent byte 0x64 is the fp16 1024 + b; under 0x54 it is 64 + b / 16
    r.se2 = hsub2(__byte_perm(s2, 0x64646464u, 0x4040), 0x64006400u);
    r.so2 = hsub2(__byte_perm(s2, 0x54545454u, 0x4141), 0x54005400u);
    r.mm = hsub2(__byte_perm(m2, 0x64646464u, 0x4140), 0x64006400u);
    return r;
}

// One task: rows g and g+8 of the tile against every token column. xb: this lane's staged activations
// (B column g, group pair t of the task's superblock); WIDE: the lo pieces sit lo_off bytes further.
// gsb: the staged group sums of B column g, pair t. o[]: (row g, col 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1).
struct Q4K {
    static constexpr int ROW_BYTES = 144;
    static constexpr int TASK_BYTES = 16 * ROW_BYTES;
    static constexpr bool SWIZZLED = false;  // whether the task's TMA boxes use a shared-memory swizzle
    static constexpr int AUX_BYTES = 0;
    static constexpr int GS_BYTES = 16;  // staged group sums per (B column, superblock): eight fp16

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, TASK_BYTES);
        tma_load_2d(dst, &p.map[seg], sb * ROW_BYTES, row0, bar, policy);
    }
    // Float4 i of the window (columns 4i..4i+3): 16 of them per group pair, pairs PITCH apart.
    __device__ static __forceinline__ uint32_t x_offset(uint32_t i) { return (i >> 4) * PITCH + (i & 15u) * 8; }
    // Sum of a 32-column group (eight consecutive lanes), times 2^-6, as fp16 pieces.
    __device__ static __forceinline__ void group_sum(uint8_t *gs_hi, uint8_t *gs_lo, uint32_t i, float sum, uint32_t lane) {
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if ((lane & 7) == 0) {
            sum *= 0.015625f;
            const __half sh = __float2half_rn(sum), sl = __float2half_rn(sum - __half2float(sh));
            const uint32_t grp = i >> 3;  // group within the window
            *(__half *)(gs_hi + grp * 2) = sh;
            *(__half *)(gs_lo + grp * 2) = sl;
        }
    }

template <bool WIDE>
__device__ static __forceinline__ void task(const uint8_t *task, const uint8_t *, const uint8_t *xb, uint32_t lo_off, const uint8_t *gsb, uint32_t gs_lo_off, uint32_t g,
                                     uint32_t t, float o[4]) {
    uint4 hdr[2], q0[2], q1[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint8_t *row = task + (g + 8 * h) * ROW_BYTES;
        hdr[h] = *(const uint4 *)row;
        q0[h] = *(const uint4 *)(row + 16 + t * 32);
        q1[h] = *(const uint4 *)(row + 32 + t * 32);
    }
    const RowScales r0 = row_scales(hdr[0], t), r1 = row_scales(hdr[1], t);
    float ce[4] = {0.f, 0.f, 0.f, 0.f}, co[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i2 = 0; i2 < 4; ++i2) {
        // 16 bytes of staged activations hold two k16 steps: even group at +0, odd group at +64
        const uint4 be = *(const uint4 *)(xb + i2 * 16), bo = *(const uint4 *)(xb + 64 + i2 * 16);
        uint4 bel, bol;
        if (WIDE) {
            bel = *(const uint4 *)(xb + lo_off + i2 * 16);
            bol = *(const uint4 *)(xb + lo_off + 64 + i2 * 16);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int i = i2 * 2 + k;
            const uint32_t w0 = i < 4 ? word(q0[0], i) : word(q1[0], i - 4);
            const uint32_t w1 = i < 4 ? word(q0[1], i) : word(q1[1], i - 4);
            const uint32_t s0 = w0 >> 8, s1 = w1 >> 8;
            uint32_t ae[4], ao[4];
            ae[0] = hmul2(w0 & 0x000f000fu, r0.se2); ae[1] = hmul2(w1 & 0x000f000fu, r1.se2);
            ae[2] = hmul2(s0 & 0x000f000fu, r0.se2); ae[3] = hmul2(s1 & 0x000f000fu, r1.se2);
            ao[0] = hmul2(w0 & 0x00f000f0u, r0.so2); ao[1] = hmul2(w1 & 0x00f000f0u, r1.so2);
            ao[2] = hmul2(s0 & 0x00f000f0u, r0.so2); ao[3] = hmul2(s1 & 0x00f000f0u, r1.so2);
            mma16816(ce, ae, k ? be.z : be.x, k ? be.w : be.y);
            mma16816(co, ao, k ? bo.z : bo.x, k ? bo.w : bo.y);
            if (WIDE) {
                mma16816(ce, ae, k ? bel.z : bel.x, k ? bel.w : bel.y);
                mma16816(co, ao, k ? bol.z : bol.x, k ? bol.w : bol.y);
            }
        }
    }
    float cm[4] = {0.f, 0.f, 0.f, 0.f};
    mma1688(cm, r0.mm, r1.mm, *(const uint32_t *)(gsb + t * 4));
    if (WIDE) mma1688(cm, r0.mm, r1.mm, *(const uint32_t *)(gsb + gs_lo_off + t * 4));
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float d = __half2float(__ushort_as_half((unsigned short)(hdr[h].x & 0xffffu))) * 16777216.0f;
        const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr[h].x >> 16))) * 64.0f;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int j = 2 * h + c;
            o[j] = fmaf(d, ce[j] + co[j], o[j]);
            o[j] = fmaf(-dmin, cm[j], o[j]);
        }
    }
}
};

static bool fill(const FastJob &job, Params &p, Plan &plan, bool maps) {
    if (job.enc != Q4_K || job.layout != 0) return false;
    if (!fill_common<Q4K>(job, p, plan)) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.stride % 16 != 0) return false;
        if (maps && !encode_weight_map(&p.map[s], g.w, (uint64_t)p.ksb * 144, g.rows, g.stride, 144, 16)) return false;
    }
    return true;
}

}  // namespace rows

// NUCLIS_ROWS_ONE_TOKEN=1 sends one-token plain jobs through this kernel too (for measurements).
bool q4k_rows_one_token() {
    static const bool on = [] { const char *e = getenv("NUCLIS_ROWS_ONE_TOKEN"); return e && e[0] == '1'; }();
    return on;
}

bool q4k_rows_configure() { return rows::configure<rows::Q4K>(); }

bool q4k_rows_supported(const FastJob &job) {
    if (job.tokens < 2 && !q4k_rows_one_token()) return false;
    rows::Params p;
    rows::Plan plan;
    return rows::fill(job, p, plan, false);
}

int launch_q4k_rows(cudaStream_t s, const FastJob &job) {
    rows::Params p;
    rows::Plan plan;
    if (!rows::fill(job, p, plan, true)) return 0;
    return rows::launch<rows::Q4K>(s, job, p, plan);
}

}  // namespace nu
