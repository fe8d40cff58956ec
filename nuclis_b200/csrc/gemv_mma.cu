// Fused block-dequant GEMV / small-M GEMM for 1..8 activation rows (sm_100a).
//
// Serves Backend.matvec, matvecRows, the <= 8-token arm of matmul and
// matvecSegments (inference/src/backends/metal/ops/matvec.zig:85-116, 149-165,
// 268-343; ops/matmul.zig:134-159) for the block encodings with a packed
// unpacker below. One kernel covers every token count so that a verify batch
// reads each weight byte exactly once and costs what a single row costs.
//
// How the arithmetic is arranged
//   * Weight bytes stream HBM -> shared memory with TMA tensor copies
//     (cp.async.bulk.tensor.2d + mbarrier): one instruction moves a box of 16
//     weight rows by one superblock, whatever the row stride; several stages
//     deep per warp. Each warp owns its stages, so there is no block-wide
//     barrier on the weight path.
//   * The integer codes are exact in fp16. They go straight from the packed
//     bytes into the A operand of mma.sync.m16n8k16 (a 4-bit code masked in
//     place is the fp16 subnormal code * 2^-24, so no int->float conversion is
//     issued); 16 weight rows by 16 columns per instruction.
//   * Each activation x is scaled by a power of two per (token, K slice) and
//     split into two fp16 pieces hi + lo (22 significant bits); the pieces are
//     the B operand: for <= 4 tokens both pieces sit side by side in the 8 B
//     columns (one mma per 16 columns), for 5..8 tokens they take two mmas.
//     Products of fp16 values are exact and accumulate in F32.
//   * The per-group scales never touch the tensor core: after the two mmas of
//     a 32-value group the F32 result is multiplied by d*scale in an F32 FMA
//     (the factored form sum_g d*s_g*sum(q*x) - dmin*sum_g m_g*sum(x) of
//     kernels/matvec.metal:197). The min term is itself one small mma per
//     superblock over the eight group sums of x.
//   * K is cut into slices (as long as the staged activations allow: 32
//     superblocks for one token, 4 for eight); a work unit is 32 weight rows by
//     one slice, and units are dealt out statically, slice-major, to persistent
//     blocks (one per SM). Inside a block the unit's superblocks are tasks taken
//     round-robin by the warps; each task leaves its 32 x tokens sums in a
//     shared-memory slot and the last task of a unit adds the slots in
//     superblock order. With more than one slice those sums go to a global
//     scratch array and the last unit to arrive for a row block adds them in
//     slice order. Every sum has a fixed order: results do not depend on timing.
//
// Accuracy: each product carries a relative error <= 2^-22 from the hi/lo split
// (plus 2^-38 of the largest |x| of the slice); accumulation is F32. The
// reference's GPU kernels are held to 4e-6 * sum|w*x| + 1e-6 per element
// (inference/metal-check.zig:3976); this kernel is tested to the same formula.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstring>

#include "kernels.hpp"
#include "nu_device.cuh"

namespace nu {
namespace fast {

constexpr int UNIT_ROWS = 32;  // weight rows per work unit (two m16 tiles)
constexpr int RING = 8;        // units whose task slots a block keeps at once
constexpr int PENDING = 4;     // units whose arrival shares one memory fence
constexpr uint32_t SPIN_LIMIT = 1u << 22;  // polls of a bounded barrier wait

struct Params {
    CUtensorMap map[4];  // per segment: uint8 [rows][row bytes], box 16 rows x one superblock
    float *out[4];
    unsigned long long out_stride[4];
    uint32_t rows[4];
    uint32_t rb_begin[5];    // first row block of each segment in the unit list
    uint32_t prow_begin[4];  // first row of each segment in the partial array
    uint32_t total_prows;
    uint32_t count, mode, tokens;
    uint32_t ksb, ksl, nks, total_rb;  // superblocks per row, per slice; slices; row blocks
    uint32_t ksl_inv;                  // ceil(65536 / ksl)
    const float *in;
    unsigned long long in_stride;
    float *partials;
    uint32_t *counters;
    uint32_t *status;  // set to 1 if a bounded wait ran out
};

// ---- PTX wrappers ---------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait: false if the barrier did not complete within SPIN_LIMIT polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ uint64_t evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
// TMA box copy global -> shared: x is the byte offset in the row (a multiple of 16), y the first row;
// rows past the tensor are filled with zeros.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar), "l"(policy)
        : "memory");
}
// d = a * b (no accumulator input: the zero operands cost no register moves)
__device__ __forceinline__ void mma16816_first(float d[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma1688_first(float d[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "f"(0.0f));
}
__device__ __forceinline__ void mma1688(float c[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(b0));
}
// Shared-memory loads as plain C++ loads: the compiler may hoist and interleave them freely
// between the barriers that order them against the asynchronous copies.
__device__ __forceinline__ uint4 lds128(const uint8_t *p) { return *(const uint4 *)p; }
__device__ __forceinline__ uint2 lds64(const uint8_t *p) { return *(const uint2 *)p; }
__device__ __forceinline__ uint32_t lds32(const uint8_t *p) { return *(const uint32_t *)p; }

// ---- geometry -------------------------------------------------------------------------

template <int ENC> struct Geo;
template <> struct Geo<Q4_K> {
    static constexpr int UB = 144;  // bytes per 256 columns of one row
    // One pipeline stage: two boxes of 16 rows x one superblock, rows packed 144 B apart.
    // Lane group g of an mma reads row perm8(g) of each 8-row half (0,2,4,6,1,3,5,7): the four
    // rows a half-warp reads with one 64-bit load per lane (32 contiguous bytes per row) then
    // start 288 B apart, i.e. in four different groups of eight banks.
    static constexpr int ROW = 144;
    static constexpr int STAGE_BYTES = UNIT_ROWS * ROW;
    // Decoded scales of the stage: d*s pairs [4 p][32 rows][2] f32, minima [32 rows][4] u32, dmin [32] f32.
    static constexpr int SCALE_BYTES = 4 * UNIT_ROWS * 8 + UNIT_ROWS * 16 + UNIT_ROWS * 4;
};

// Token-slot geometry. TS is the number of token slots (1, 2, 4 or 8).
template <int TS> struct Cols {
    static constexpr int NP = TS == 8 ? 2 : 1;       // mmas per 16 columns
    static constexpr int NS = TS == 8 ? 8 : 2 * TS;  // stored B columns per piece array
    static constexpr int KSL_MAX = 32 / TS;          // longest slice whose activations fit the staging area
    static constexpr int X_BYTES = NP * KSL_MAX * 32 * NS * 16;   // 32 KiB
    static constexpr int S_BYTES = NP * KSL_MAX * 4 * NS * 4;     // 1 KiB
    static constexpr int SLOT_BYTES = UNIT_ROWS * TS * 4;         // one task's sums, [token][row]
    static constexpr int RING_BYTES = RING * KSL_MAX * SLOT_BYTES;  // 32 KiB
};

template <int ENC, int TS, int WARPS, int STAGES> constexpr int smem_bytes() {
    return Cols<TS>::X_BYTES + Cols<TS>::S_BYTES + 1024 /* inv scale, max scratch, ring counters */ + Cols<TS>::RING_BYTES +
           WARPS * (STAGES * Geo<ENC>::STAGE_BYTES + Geo<ENC>::SCALE_BYTES) + WARPS * STAGES * 8 + 128;
}

__device__ __forceinline__ uint32_t slice_sbs(const Params &p, uint32_t ks) { return min(p.ksl, p.ksb - ks * p.ksl); }

struct UnitRows {
    uint32_t seg, row0;
    uint32_t rows_left[2];  // valid rows from the first row of each 16-row tile (may exceed 16)
};

// Row block `rb` -> the two 16-row tiles it covers. Plain mode: 32 consecutive
// rows of one segment. Pair mode: rows [16 rb, 16 rb + 16) of segment 0 and of segment 1.
__device__ __forceinline__ UnitRows unit_rows(const Params &p, uint32_t rb) {
    UnitRows u;
    if (p.mode != ACT_NONE) {
        u.seg = 0;
        u.row0 = rb * 16;
        u.rows_left[0] = u.rows_left[1] = p.rows[0] - u.row0;
    } else {
        u.seg = 0;
#pragma unroll
        for (int s = 1; s < 4; ++s)
            if ((uint32_t)s < p.count && rb >= p.rb_begin[s]) u.seg = s;
        u.row0 = (rb - p.rb_begin[u.seg]) * UNIT_ROWS;
        u.rows_left[0] = p.rows[u.seg] - u.row0;
        u.rows_left[1] = u.rows_left[0] > 16 ? u.rows_left[0] - 16 : 0;
    }
    return u;
}

// Row of an mma fragment's lane group g within its 8-row half (see Geo::ROW).
__device__ __forceinline__ uint32_t perm8(uint32_t g) { return ((g & 3u) << 1) | (g >> 2); }

// ---- activation staging -------------------------------------------------------------
// Splits the slice's activations into scaled fp16 pieces laid out as mma B
// fragments, and the per-group sums of x (for the min term) likewise.
//
// B layout for Q4_K. An mma of group pair p (groups 2p low nibbles, 2p+1 high
// nibbles), half h, takes from lane (t = lane & 3) the four codes of quant word
// 8p + 2t + h, i.e. columns 8t + 4h + {0,1,2,3} of the group, with
// k index 2t <- +0, 2t+1 <- +2, 2t+8 <- +1, 2t+9 <- +3 (the order the byte
// masks below produce). So the 16 bytes stored per (column group of 8, B column)
// are x[+0], x[+2], x[+1], x[+3], x[+4], x[+6], x[+5], x[+7].
template <int TS>
__device__ __forceinline__ uint32_t b_slot(uint32_t n) {
    if (TS == 8) return n;
    // pieces side by side: columns 0..3 hi, 4..7 lo. A column whose token slot does not exist
    // reads slot 0: its products land in an output column that is never stored.
    const uint32_t tok = n & 3;
    return (n >> 2) * TS + (tok < (uint32_t)TS ? tok : 0);
}

template <int TS, int WARPS>
__device__ void stage_activations(const Params &p, uint32_t ks, uint8_t *xs, uint8_t *ss, float *inv_scale, float *red) {
    using C = Cols<TS>;
    constexpr int THREADS = WARPS * 32;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t nsb = slice_sbs(p, ks);
    const uint32_t groups = nsb * 32;  // column groups of 8 in the slice
    const uint32_t col_base = ks * p.ksl * 256;
    // Pass 1: largest |x| per token over the slice.
    float mx[TS];
#pragma unroll
    for (int t = 0; t < TS; ++t) mx[t] = 0.0f;
    for (uint32_t f = tid; f < groups * TS; f += THREADS) {
        const uint32_t tok = f / groups, cg = f % groups;
        if (tok < p.tokens) {
            const float4 *src = (const float4 *)(p.in + (size_t)tok * p.in_stride + col_base + cg * 8);
            const float4 a = src[0], b = src[1];
            const float m = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                                  fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
#pragma unroll
            for (int t = 0; t < TS; ++t)
                if ((uint32_t)t == tok) mx[t] = fmaxf(mx[t], m);
        }
    }
#pragma unroll
    for (int t = 0; t < TS; ++t) {
        float m = mx[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) red[warp * 8 + t] = m;
    }
    __syncthreads();
    // Scale 2^e puts the largest value in [2^13, 2^14): hi pieces cannot overflow
    // fp16 and lo pieces keep 11 bits down to 2^-25 of the largest value.
    float scale[TS];
#pragma unroll
    for (int t = 0; t < TS; ++t) {
        float m = red[t];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) m = fmaxf(m, red[w * 8 + t]);
        const uint32_t e = (__float_as_uint(m) >> 23) & 0xffu;
        const bool ok = e >= 40u && e < 255u;  // finite and not vanishingly small
        scale[t] = ok ? __uint_as_float((267u - e) << 23) : 1.0f;
        if (tid == 0) inv_scale[t] = ok ? __uint_as_float((e - 13u) << 23) : 1.0f;
    }
    // Pass 2: pieces and group sums.
    for (uint32_t f = tid; f < groups * TS; f += THREADS) {
        const uint32_t tok = f / groups, cg = f % groups;
        float v[8];
        if (tok < p.tokens) {
            const float4 *src = (const float4 *)(p.in + (size_t)tok * p.in_stride + col_base + cg * 8);
            const float4 a = src[0], b = src[1];
            float sc = 1.0f;
#pragma unroll
            for (int t = 0; t < TS; ++t)
                if ((uint32_t)t == tok) sc = scale[t];
            v[0] = a.x * sc; v[1] = a.y * sc; v[2] = a.z * sc; v[3] = a.w * sc;
            v[4] = b.x * sc; v[5] = b.y * sc; v[6] = b.z * sc; v[7] = b.w * sc;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        }
        __half hi[8], lo[8];
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            hi[i] = __float2half_rn(v[i]);
            lo[i] = __float2half_rn(v[i] - __half2float(hi[i]));
            sum += v[i];
        }
        // 32-column group sum: the four lanes of a quad hold its four column groups.
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float mean = sum * 0.03125f;  // /32 keeps the sum inside fp16 range
        const __half mhi = __float2half_rn(mean);
        const __half mlo = __float2half_rn(mean - __half2float(mhi));
        uint32_t whi[4], wlo[4];
        whi[0] = (uint32_t)__half_as_ushort(hi[0]) | ((uint32_t)__half_as_ushort(hi[2]) << 16);
        whi[1] = (uint32_t)__half_as_ushort(hi[1]) | ((uint32_t)__half_as_ushort(hi[3]) << 16);
        whi[2] = (uint32_t)__half_as_ushort(hi[4]) | ((uint32_t)__half_as_ushort(hi[6]) << 16);
        whi[3] = (uint32_t)__half_as_ushort(hi[5]) | ((uint32_t)__half_as_ushort(hi[7]) << 16);
        wlo[0] = (uint32_t)__half_as_ushort(lo[0]) | ((uint32_t)__half_as_ushort(lo[2]) << 16);
        wlo[1] = (uint32_t)__half_as_ushort(lo[1]) | ((uint32_t)__half_as_ushort(lo[3]) << 16);
        wlo[2] = (uint32_t)__half_as_ushort(lo[4]) | ((uint32_t)__half_as_ushort(lo[6]) << 16);
        wlo[3] = (uint32_t)__half_as_ushort(lo[5]) | ((uint32_t)__half_as_ushort(lo[7]) << 16);
        const uint32_t grp = cg >> 2;  // 32-column group within the slice
        const uint32_t lo_x = TS == 8 ? C::X_BYTES / 2 : TS * 16;
        const uint32_t lo_s = TS == 8 ? C::S_BYTES / 2 : TS * 4;
        uint8_t *xdst = xs + ((size_t)cg * C::NS + tok) * 16;
        *(uint4 *)xdst = make_uint4(whi[0], whi[1], whi[2], whi[3]);
        *(uint4 *)(xdst + lo_x) = make_uint4(wlo[0], wlo[1], wlo[2], wlo[3]);
        if ((lane & 3) == 0) {
            uint8_t *sdst = ss + ((size_t)(grp >> 1) * C::NS + tok) * 4 + (grp & 1) * 2;
            *(__half *)sdst = mhi;
            *(__half *)(sdst + lo_s) = mlo;
        }
    }
}

// ---- Q4_K: scale pre-pass and the mma loop over one pipeline stage -----------------------

// Decodes the packed 6-bit scales and minima of the stage once per warp, lane r
// taking row r: d*s as F32 with the 2^24 (low nibble) or 2^20 (high nibble) of
// the subnormal trick folded in, the minima as fp16 subnormals (m * 2^-24) in
// mma A order, and dmin * 2^29 (2^24 from the minima, 2^5 from the group sums
// being stored as means). Integer -> float goes through the 2^23 magic number
// (one byte permute and one FMA per value) instead of a conversion.
__device__ __forceinline__ void q4k_prepass(const uint8_t *stage, uint8_t *scales, uint32_t lane) {
    const uint4 hdr = lds128(stage + lane * Geo<Q4_K>::ROW);
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
    const float dm = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    const uint32_t s_lo = hdr.y & 0x3f3f3f3fu;
    const uint32_t m_lo = hdr.z & 0x3f3f3f3fu;
    const uint32_t s_hi = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
    const uint32_t m_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
    const float even = d * 16777216.0f, odd = d * 1048576.0f;
    const float even_bias = -8388608.0f * even, odd_bias = -8388608.0f * odd;
    // groups 2p (even: low nibbles) and 2p+1 (odd: high nibbles) of pair p are bytes 2p%4, 2p%4+1 of s_lo / s_hi
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const uint32_t src = p < 2 ? s_lo : s_hi;
        const float fe = __uint_as_float(__byte_perm(src, 0x4b000000u, 0x7650 + 2 * (p & 1)));
        const float fo = __uint_as_float(__byte_perm(src, 0x4b000000u, 0x7651 + 2 * (p & 1)));
        const float se = fmaf(fe, even, even_bias), so = fmaf(fo, odd, odd_bias);
        *(float2 *)(scales + (p * UNIT_ROWS + lane) * 8) = make_float2(se, so);
    }
    uint4 mm;
    mm.x = (m_lo & 0xffu) | ((m_lo & 0xff00u) << 8);
    mm.y = ((m_lo >> 16) & 0xffu) | ((m_lo >> 8) & 0xff0000u);
    mm.z = (m_hi & 0xffu) | ((m_hi & 0xff00u) << 8);
    mm.w = ((m_hi >> 16) & 0xffu) | ((m_hi >> 8) & 0xff0000u);
    *(uint4 *)(scales + 4 * UNIT_ROWS * 8 + lane * 16) = mm;
    *(float *)(scales + 4 * UNIT_ROWS * 8 + UNIT_ROWS * 16 + lane * 4) = dm * 536870912.0f;
}

// One stage: 32 rows x 256 columns against the slice's B fragments at superblock `sb` of the slice.
template <int TS>
__device__ __forceinline__ void q4k_stage(const uint8_t *stage, uint32_t sb, const uint8_t *scales, const uint8_t *xs, const uint8_t *ss, uint32_t lane, float acc[2][4]) {
    using C = Cols<TS>;
    const uint32_t g = lane >> 2, t = lane & 3, gp = perm8(g);
    const uint32_t slot = b_slot<TS>(g);
    const uint8_t *xsb = xs + sb * 32 * C::NS * 16 + (t * C::NS + slot) * 16;
    const uint8_t *ssb = ss + sb * 4 * C::NS * 4 + (t * C::NS + slot) * 4;
    const uint8_t *wrow = stage + gp * Geo<Q4_K>::ROW + 16 + t * 8;
    const uint8_t *srow = scales + gp * 8;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        uint2 wq[2][2];  // [tile][row g / g+8] -> words for h = 0, 1
        float2 ds[2][2];
#pragma unroll
        for (int rt = 0; rt < 2; ++rt)
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                wq[rt][hrow] = lds64(wrow + (rt * 16 + hrow * 8) * Geo<Q4_K>::ROW + p * 32);
                const uint2 s = lds64(srow + (p * UNIT_ROWS + rt * 16 + hrow * 8) * 8);
                ds[rt][hrow] = make_float2(__uint_as_float(s.x), __uint_as_float(s.y));
            }
#pragma unroll
        for (int odd = 0; odd < 2; ++odd) {
            const uint32_t mask = odd ? 0x00f000f0u : 0x000f000fu;
            uint4 bf[C::NP];
#pragma unroll
            for (int a = 0; a < C::NP; ++a) bf[a] = lds128(xsb + a * (C::X_BYTES / 2) + (p * 2 + odd) * 4 * C::NS * 16);
#pragma unroll
            for (int rt = 0; rt < 2; ++rt) {
                float c[4];
                uint32_t a0[4], a1[4];
                a0[0] = wq[rt][0].x & mask; a0[1] = wq[rt][1].x & mask;
                a0[2] = (wq[rt][0].x >> 8) & mask; a0[3] = (wq[rt][1].x >> 8) & mask;
                a1[0] = wq[rt][0].y & mask; a1[1] = wq[rt][1].y & mask;
                a1[2] = (wq[rt][0].y >> 8) & mask; a1[3] = (wq[rt][1].y >> 8) & mask;
                mma16816_first(c, a0, bf[0].x, bf[0].y);
                mma16816(c, a1, bf[0].z, bf[0].w);
                if (C::NP == 2) {
                    mma16816(c, a0, bf[C::NP - 1].x, bf[C::NP - 1].y);
                    mma16816(c, a1, bf[C::NP - 1].z, bf[C::NP - 1].w);
                }
                const float s0 = odd ? ds[rt][0].y : ds[rt][0].x, s1 = odd ? ds[rt][1].y : ds[rt][1].x;
                acc[rt][0] = fmaf(s0, c[0], acc[rt][0]);
                acc[rt][1] = fmaf(s0, c[1], acc[rt][1]);
                acc[rt][2] = fmaf(s1, c[2], acc[rt][2]);
                acc[rt][3] = fmaf(s1, c[3], acc[rt][3]);
            }
        }
    }
    // min term: one k8 mma per tile over the eight group means
    const uint8_t *mins = scales + 4 * UNIT_ROWS * 8, *dmin = mins + UNIT_ROWS * 16;
    uint32_t sfrag[C::NP];
#pragma unroll
    for (int a = 0; a < C::NP; ++a) sfrag[a] = lds32(ssb + a * (C::S_BYTES / 2));
#pragma unroll
    for (int rt = 0; rt < 2; ++rt) {
        const uint32_t r0 = rt * 16 + gp;
        const uint32_t m0 = lds32(mins + (r0 * 4 + t) * 4), m1 = lds32(mins + ((r0 + 8) * 4 + t) * 4);
        float c[4];
        mma1688_first(c, m0, m1, sfrag[0]);
        if (C::NP == 2) mma1688(c, m0, m1, sfrag[C::NP - 1]);
        const float d0 = __uint_as_float(lds32(dmin + r0 * 4)), d1 = __uint_as_float(lds32(dmin + (r0 + 8) * 4));
        acc[rt][0] = fmaf(-d0, c[0], acc[rt][0]);
        acc[rt][1] = fmaf(-d0, c[1], acc[rt][1]);
        acc[rt][2] = fmaf(-d1, c[2], acc[rt][2]);
        acc[rt][3] = fmaf(-d1, c[3], acc[rt][3]);
    }
}

// Adds the partial sums of row block `rb` in slice order and writes the outputs.
__device__ __forceinline__ void reduce_row_block(const Params &p, uint32_t rb, uint32_t lane) {
    const UnitRows u = unit_rows(p, rb);
    const bool pair = p.mode != ACT_NONE;
    const uint32_t rows = pair ? 16u : 32u;
    if (lane >= rows || lane >= u.rows_left[0]) return;
    for (uint32_t tok = 0; tok < p.tokens; ++tok) {
        const float *src = p.partials + ((size_t)p.prow_begin[u.seg] + u.row0 + lane) * p.tokens + tok;
        const size_t step = (size_t)p.total_prows * p.tokens;
        float sum = 0.0f, up = 0.0f;
        uint32_t k = 0;
        // four loads in flight at a time; the additions keep slice order
        for (; k + 4 <= p.nks; k += 4) {
            const float a0 = __ldcg(src + (k + 0) * step), a1 = __ldcg(src + (k + 1) * step);
            const float a2 = __ldcg(src + (k + 2) * step), a3 = __ldcg(src + (k + 3) * step);
            sum = ((sum + a0) + a1) + a2;
            sum += a3;
        }
        for (; k < p.nks; ++k) sum += __ldcg(src + k * step);
        if (pair) {
            const float *usrc = p.partials + ((size_t)p.prow_begin[1] + u.row0 + lane) * p.tokens + tok;
            for (k = 0; k < p.nks; ++k) up += __ldcg(usrc + k * step);
            const float a = p.mode == ACT_SILU ? silu_f32(sum) : gelu_f32(sum);
            sum = a * up;
        }
        p.out[u.seg][(size_t)tok * p.out_stride[u.seg] + u.row0 + lane] = sum;
    }
}

// Publishes the partial sums of the pending units with one fence, then counts
// this warp in for each; the last arrival for a row block reduces it.
__device__ __forceinline__ void flush_pending(const Params &p, uint32_t *pending, uint32_t &npending, uint32_t lane) {
    if (npending == 0) return;
    __syncwarp();
    __threadfence();
    uint32_t mine = pending[0];
#pragma unroll
    for (int i = 1; i < PENDING; ++i)
        if (lane == (uint32_t)i) mine = pending[i];
    uint32_t arrived = 0;
    if (lane < npending) arrived = atomicAdd(p.counters + mine, 1u);
    bool any_last = false;
#pragma unroll
    for (int i = 0; i < PENDING; ++i) {
        const uint32_t a = __shfl_sync(0xffffffffu, arrived, i);
        if ((uint32_t)i < npending && a == p.nks - 1) {
            if (!any_last) __threadfence();
            any_last = true;
            reduce_row_block(p, pending[i], lane);
            if (lane == 0) p.counters[pending[i]] = 0;  // leave the scratch as it was found
        }
    }
    npending = 0;
}

// A warp's position in the block's task list: unit (global index u = ks * total_rb + rb) and superblock in its slice.
struct Cursor {
    uint32_t u, ks, rb, sb;
};
__device__ __forceinline__ void normalize(const Params &p, Cursor &c) {
    uint32_t n = slice_sbs(p, c.ks);
    if (n == p.ksl) {
        // whole units skipped at once: sb / ksl by multiply-shift (exact for sb < 4096), while the slice does not change
        const uint32_t q = (c.sb * p.ksl_inv) >> 16;
        if (q != 0 && c.rb + q < p.total_rb) {
            c.sb -= q * n;
            c.u += q;
            c.rb += q;
            return;
        }
    }
    while (c.sb >= n) {
        c.sb -= n;
        ++c.u;
        if (++c.rb == p.total_rb) {
            c.rb = 0;
            ++c.ks;
            n = c.ks < p.nks ? slice_sbs(p, c.ks) : 1u;
        }
    }
}

// ---- the kernel -------------------------------------------------------------------------------

template <int ENC, int TS, int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, 1) fast_kernel(const __grid_constant__ Params p) {
    using C = Cols<TS>;
    using G = Geo<ENC>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *xs = smem;
    uint8_t *ss = xs + C::X_BYTES;
    float *inv_scale = (float *)(ss + C::S_BYTES);      // 16 floats
    float *red = inv_scale + 16;                        // WARPS * 8 floats (<= 128)
    volatile uint32_t *ring_cnt = (uint32_t *)(inv_scale + 160);  // RING arrival counters
    volatile uint32_t *ring_gen = ring_cnt + RING;      // RING generations: how often each entry was retired
    uint8_t *ring = ss + C::S_BYTES + 1024;
    uint8_t *warp_area = ring + C::RING_BYTES;
    constexpr int WARP_BYTES = STAGES * G::STAGE_BYTES + G::SCALE_BYTES;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint8_t *stage_ptr = warp_area + warp * WARP_BYTES;
    const uint32_t stage0 = smem_u32(stage_ptr);
    uint8_t *scales = stage_ptr + STAGES * G::STAGE_BYTES;
    uint64_t *bars = (uint64_t *)(warp_area + WARPS * WARP_BYTES);
    const uint32_t bar0 = smem_u32(bars + warp * STAGES);

    if (tid == 0) {
        for (int i = 0; i < WARPS * STAGES; ++i) mbar_init(smem_u32(bars + i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 2 * RING) ring_cnt[tid] = 0;
    __syncthreads();

    const uint32_t total_units = p.nks * p.total_rb;
    const uint32_t u_begin = (uint32_t)((unsigned long long)total_units * blockIdx.x / gridDim.x);
    const uint32_t u_end = (uint32_t)((unsigned long long)total_units * (blockIdx.x + 1) / gridDim.x);
    if (u_begin >= u_end) return;
    const uint64_t policy = evict_first_policy();
    const uint32_t ks_first = u_begin / p.total_rb, ks_last = (u_end - 1) / p.total_rb;

    // Producer and consumer walk the same task sequence: tasks warp, warp + WARPS, ... of the block's list.
    Cursor prod = {u_begin, ks_first, u_begin - ks_first * p.total_rb, warp};
    normalize(p, prod);
    Cursor cons = prod;
    uint32_t issued = 0, consumed = 0;

    // One lane issues the two box copies of a task: tile 0 and tile 1 of the unit, one superblock wide.
    auto issue = [&]() {
        const uint32_t st = issued % STAGES;
        if (lane == 0) {
            const UnitRows u = unit_rows(p, prod.rb);
            const uint32_t x = (prod.ks * p.ksl + prod.sb) * G::UB;
            const uint32_t dst = stage0 + st * G::STAGE_BYTES, bar = bar0 + st * 8;
            mbar_expect_tx(bar, UNIT_ROWS * G::UB);
            if (p.mode != ACT_NONE) {
                tma_load_2d(dst, &p.map[0], x, u.row0, bar, policy);
                tma_load_2d(dst + 16 * G::ROW, &p.map[1], x, u.row0, bar, policy);
            } else {
                tma_load_2d(dst, &p.map[u.seg], x, u.row0, bar, policy);
                tma_load_2d(dst + 16 * G::ROW, &p.map[u.seg], x, u.row0 + 16, bar, policy);
            }
        }
        ++issued;
        prod.sb += WARPS;
        normalize(p, prod);
    };
    for (int i = 0; i < STAGES - 1; ++i)
        if (prod.u < u_end) issue();

    uint32_t pending[PENDING], npending = 0;
    bool failed = false;
    const uint32_t g = perm8(lane >> 2), t = lane & 3;  // g: this lane group's weight row in each 8-row half
    const bool owner = TS == 8 || t < 2;                // for fewer than 8 slots only lanes t < 2 own tokens (2t, 2t+1)

    for (uint32_t ks = ks_first; ks <= ks_last && !failed; ++ks) {
        __syncthreads();  // every warp is done with the previous slice's activations
        stage_activations<TS, WARPS>(p, ks, xs, ss, inv_scale, red);
        __syncthreads();
        const uint32_t nsb = slice_sbs(p, ks);
        while (cons.u < u_end && cons.ks == ks) {
            if (prod.u < u_end) issue();  // keep STAGES - 1 tasks in flight
            const uint32_t st = consumed % STAGES;
            if (!mbar_wait(bar0 + st * 8, (consumed / STAGES) & 1u)) { failed = true; break; }
            const uint8_t *stage = stage_ptr + st * G::STAGE_BYTES;
            float acc[2][4];
#pragma unroll
            for (int rt = 0; rt < 2; ++rt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[rt][i] = 0.0f;
            q4k_prepass(stage, scales, lane);
            __syncwarp();
            q4k_stage<TS>(stage, cons.sb, scales, xs, ss, lane, acc);
            __syncwarp();  // all lanes are done reading this stage before it is refilled
            ++consumed;

            // ---- the task's sums go to its slot of the unit's ring entry ----
            const uint32_t ul = cons.u - u_begin, entry = ul % RING;
            if (ul >= RING) {  // the entry must have been retired by the unit RING places back
                uint32_t ok = 1;
                if (lane == 0) {
                    ok = 0;
                    for (uint32_t i = 0; i < SPIN_LIMIT; ++i)
                        if (ring_gen[entry] == ul / RING) { ok = 1; break; }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { failed = true; break; }
                __threadfence_block();
            }
            float *slot = (float *)(ring + ((size_t)entry * C::KSL_MAX + cons.sb) * C::SLOT_BYTES);
#pragma unroll
            for (int rt = 0; rt < 2; ++rt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float a = acc[rt][i];
                    if (TS != 8) a += __shfl_xor_sync(0xffffffffu, a, 2);  // hi columns + lo columns
                    const uint32_t tok = 2 * t + (i & 1);
                    if (owner && tok < (uint32_t)TS) slot[tok * UNIT_ROWS + rt * 16 + (i >> 1) * 8 + g] = a;
                }
            __syncwarp();
            uint32_t arrived = 0;
            if (lane == 0) {
                __threadfence_block();
                arrived = atomicAdd((uint32_t *)ring_cnt + entry, 1u);
            }
            arrived = __shfl_sync(0xffffffffu, arrived, 0);
            if (arrived == nsb - 1) {
                // ---- last task of the unit: add the slots in superblock order ----
                __threadfence_block();
                const UnitRows u = unit_rows(p, cons.rb);
                const float *base = (const float *)(ring + (size_t)entry * C::KSL_MAX * C::SLOT_BYTES) + lane;
                const bool pair = p.mode != ACT_NONE;
#pragma unroll
                for (int tok = 0; tok < TS; ++tok) {
                    if ((uint32_t)tok >= p.tokens) break;
                    float sum = 0.0f;
                    for (uint32_t sb = 0; sb < nsb; ++sb) sum += base[sb * (C::SLOT_BYTES / 4) + tok * UNIT_ROWS];
                    sum *= inv_scale[tok];
                    if (p.nks > 1) {
                        // rows past the matrix land in the padding of the partial array
                        const uint32_t prow = pair ? p.prow_begin[lane >> 4] + u.row0 + (lane & 15) : p.prow_begin[u.seg] + u.row0 + lane;
                        p.partials[((size_t)ks * p.total_prows + prow) * p.tokens + tok] = sum;
                    } else if (pair) {
                        const float up = __shfl_down_sync(0xffffffffu, sum, 16);
                        if (lane < 16 && lane < u.rows_left[0]) {
                            const float a = p.mode == ACT_SILU ? silu_f32(sum) : gelu_f32(sum);
                            p.out[0][(size_t)tok * p.out_stride[0] + u.row0 + lane] = a * up;
                        }
                    } else if (lane < u.rows_left[0]) {
                        p.out[u.seg][(size_t)tok * p.out_stride[u.seg] + u.row0 + lane] = sum;
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    ring_cnt[entry] = 0;
                    __threadfence_block();
                    ring_gen[entry] = ul / RING + 1;
                }
                if (p.nks > 1) {
#pragma unroll
                    for (int i = 0; i < PENDING; ++i)
                        if (npending == (uint32_t)i) pending[i] = cons.rb;
                    if (++npending == PENDING) flush_pending(p, pending, npending, lane);
                }
            }
            cons.sb += WARPS;
            normalize(p, cons);
        }
    }
    flush_pending(p, pending, npending, lane);
    if (failed) {
        if (lane == 0) atomicExch(p.status, 1u);
        // Let this warp's copies still in flight land before the block's shared memory is released.
        for (; consumed < issued; ++consumed) mbar_wait(bar0 + (consumed % STAGES) * 8, (consumed / STAGES) & 1u);
    }
}

}  // namespace fast

// ---- host side ------------------------------------------------------------------------------------

static uint32_t token_slots(uint32_t tokens) { return tokens <= 1 ? 1 : tokens <= 2 ? 2 : tokens <= 4 ? 4 : 8; }

#ifndef NU_FAST_WARPS
#define NU_FAST_WARPS 12
#endif
#ifndef NU_FAST_STAGES
#define NU_FAST_STAGES 2
#endif
constexpr int kWarps = NU_FAST_WARPS, kStages = NU_FAST_STAGES;

// cuTensorMapEncodeTiled through the runtime's driver entry point: no link against libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    }
    return fn;
}

// A two-dimensional tensor [outer][inner] of `elem_bytes`-wide elements, `stride_bytes` between rows.
bool encode_tiled_map(CUtensorMap *map, CUtensorMapDataType type, uint32_t elem_bytes, const void *base, uint64_t inner, uint64_t outer,
                      uint64_t stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    (void)elem_bytes;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, type, 2, (void *)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A uint8 tensor [rows][row_bytes] with `stride` bytes between rows, copied in boxes of box_rows x box_bytes.
bool encode_weight_map(CUtensorMap *map, const uint8_t *base, uint64_t row_bytes, uint64_t rows, uint64_t stride, uint32_t box_bytes, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {stride};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool fill_params(const FastJob &job, fast::Params &p) {
    if (job.enc != Q4_K || job.layout != 0) return false;
    if (job.tokens < 1 || job.tokens > 8 || job.count < 1 || job.count > 4) return false;
    if (job.columns == 0 || job.columns % 256 != 0) return false;
    if ((uintptr_t)job.in % 16 != 0 || (job.tokens > 1 && job.in_stride % 4 != 0)) return false;
    if (job.mode != ACT_NONE && (job.count != 2 || job.seg[0].rows != job.seg[1].rows)) return false;
    memset(&p, 0, sizeof p);
    p.count = job.count;
    p.mode = job.mode;
    p.tokens = job.tokens;
    p.ksb = job.columns / 256;
    p.in = job.in;
    p.in_stride = job.in_stride;
    uint32_t rb = 0, prow = 0;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows == 0 || (uintptr_t)g.w % 16 != 0 || g.stride % 16 != 0 || (uintptr_t)g.out % 4 != 0) return false;
        if (!encode_weight_map(&p.map[s], g.w, (uint64_t)p.ksb * 144, g.rows, g.stride, 144, 16)) return false;
        p.out[s] = g.out;
        p.out_stride[s] = g.out_stride;
        p.rows[s] = g.rows;
        p.rb_begin[s] = rb;
        p.prow_begin[s] = prow;
        if (job.mode == ACT_NONE) rb += (g.rows + fast::UNIT_ROWS - 1) / fast::UNIT_ROWS;
        else if (s == 0) rb += (g.rows + 15) / 16;
        prow += (g.rows + 31) / 32 * 32;
    }
    for (uint32_t s = job.count; s < 5; ++s) p.rb_begin[s] = rb;
    p.total_rb = rb;
    p.total_prows = prow;
    // Slice length: as few slices as the staging area allows, a few more when that fills the
    // machine more evenly (whole rounds of units per block) at little cost in partial sums.
    {
        const uint32_t ksl_max = 32u / token_slots(job.tokens);
        const uint32_t nks_min = (p.ksb + ksl_max - 1) / ksl_max;
        const double weight_bytes = (double)p.ksb * 144.0 * prow;
        double best = -1.0;
        for (uint32_t nks = nks_min; nks <= p.ksb && nks < nks_min + 12; ++nks) {
            const uint32_t ksl = (p.ksb + nks - 1) / nks;
            const uint32_t slices = (p.ksb + ksl - 1) / ksl;
            const double units = (double)slices * rb;
            const double blocks = units < job.sm_count ? units : job.sm_count;
            const double rounds = (double)(uint64_t)((units + blocks - 1) / blocks);
            double eff = units / (rounds * blocks);
            if (slices > 1) eff /= 1.03 + 2.0 * slices * prow * job.tokens * 4.0 / weight_bytes;
            if (eff > best) { best = eff; p.ksl = ksl; p.nks = slices; p.ksl_inv = (65536u + ksl - 1) / ksl; }
        }
    }
    p.partials = job.partials;
    p.counters = job.counters;
    if (p.nks > 1) {
        if ((size_t)p.nks * prow * job.tokens > job.partials_floats) return false;
        if (rb > job.counters_len) return false;
    }
    return true;
}

bool fast_supported(const FastJob &job) {
    if (q4k_decode_supported(job) || q6k_decode_supported(job) || q8_0_decode_supported(job) || q4k_rows_supported(job) || q6k_rows_supported(job) || q8_0_rows_supported(job)) return true;
    fast::Params p;
    return fill_params(job, p);
}

template <int ENC, int TS>
static bool configure_variant() {
    return cudaFuncSetAttribute(fast::fast_kernel<ENC, TS, kWarps, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                fast::smem_bytes<ENC, TS, kWarps, kStages>()) == cudaSuccess;
}

bool fast_configure() {
    return q4k_decode_configure() && q4k_rows_configure() && q6k_rows_configure() && q8_0_rows_configure() && q6k_decode_configure() && q8_0_decode_configure() && prefill_configure() && configure_variant<Q4_K, 1>() && configure_variant<Q4_K, 2>() && configure_variant<Q4_K, 4>() && configure_variant<Q4_K, 8>();
}

template <int ENC, int TS>
static int launch_variant(cudaStream_t s, const fast::Params &p, int sm_count) {
    constexpr int bytes = fast::smem_bytes<ENC, TS, kWarps, kStages>();
    const uint32_t units = p.nks * p.total_rb;
    const uint32_t grid = units < (uint32_t)sm_count ? units : (uint32_t)sm_count;
    fast::fast_kernel<ENC, TS, kWarps, kStages><<<grid, kWarps * 32, bytes, s>>>(p);
    return 1;
}

int launch_fast(cudaStream_t s, const FastJob &job) {
    if (job.tokens == 1 && q4k_rows_one_token() && q4k_rows_supported(job)) return launch_q4k_rows(s, job);
    if (q4k_decode_supported(job)) return launch_q4k_decode(s, job);
    if (q6k_decode_supported(job)) return launch_q6k_decode(s, job);
    if (q8_0_decode_supported(job)) return launch_q8_0_decode(s, job);
    if (q4k_rows_supported(job)) return launch_q4k_rows(s, job);
    if (q6k_rows_supported(job)) return launch_q6k_rows(s, job);
    if (q8_0_rows_supported(job)) return launch_q8_0_rows(s, job);
    fast::Params p;
    if (!fill_params(job, p)) return 0;
    // The status word lives at the end of the counters array.
    p.status = job.counters + job.counters_len;
    switch (token_slots(job.tokens)) {
    case 1: return launch_variant<Q4_K, 1>(s, p, job.sm_count);
    case 2: return launch_variant<Q4_K, 2>(s, p, job.sm_count);
    case 4: return launch_variant<Q4_K, 4>(s, p, job.sm_count);
    default: return launch_variant<Q4_K, 8>(s, p, job.sm_count);
    }
}

}  // namespace nu
