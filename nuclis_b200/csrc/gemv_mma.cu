// Fused block-dequant GEMV / small-M GEMM for 1..8 activation rows (sm_100a).
//
// Serves Backend.matvec, matvecRows, the <= 8-token arm of matmul and
// matvecSegments (inference/src/backends/metal/ops/matvec.zig:85-116, 149-165,
// 268-343; ops/matmul.zig:134-159) for the block encodings with a packed
// unpacker below. One kernel covers every token count so that a verify batch
// reads each weight byte exactly once and costs what a single row costs.
//
// How the arithmetic is arranged
//   * Weight bytes stream HBM -> shared memory with 1-D bulk async copies
//     (cp.async.bulk + mbarrier), one copy per weight row segment, several
//     stages deep per warp; each warp owns its stages, so there is no block-wide
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
//   * K is cut into slices of up to 4 superblocks; a work unit is 32 weight
//     rows by one slice. Units are dealt out statically, slice-major, to
//     persistent blocks (one per SM). With more than one slice the partial sums
//     go to a scratch array and the last unit to arrive for a row block adds
//     them in slice order, so the result does not depend on timing.
//
// Accuracy: each product carries a relative error <= 2^-22 from the hi/lo split
// (plus 2^-38 of the largest |x| of the slice); accumulation is F32. The
// reference's GPU kernels are held to 4e-6 * sum|w*x| + 1e-6 per element
// (inference/metal-check.zig:3976); this kernel is tested to the same formula.
#include <cuda_fp16.h>

#include "kernels.hpp"
#include "nu_device.cuh"

namespace nu {
namespace fast {

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int KSL = 4;        // superblocks (256 columns) per K slice
constexpr int STAGE_SB = 2;   // superblocks per pipeline stage
constexpr int STAGES = 4;     // stages per warp
constexpr int UNIT_ROWS = 32; // weight rows per work unit (two m16 tiles)
constexpr uint32_t SPIN_LIMIT = 1u << 22;  // polls of a bounded barrier wait

struct Params {
    const uint8_t *w[4];
    unsigned long long stride[4];
    float *out[4];
    unsigned long long out_stride[4];
    uint32_t rows[4];
    uint32_t rb_begin[5];    // first row block of each segment in the unit list
    uint32_t prow_begin[4];  // first row of each segment in the partial array
    uint32_t total_prows;
    uint32_t count, mode, tokens;
    uint32_t ksb, nks, total_rb;
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
// 1-D bulk copy global -> shared; both addresses and the size are multiples of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void mma16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma1688(float c[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// ---- per-encoding geometry --------------------------------------------------------

template <int ENC> struct Geo;
template <> struct Geo<Q4_K> {
    static constexpr int UB = 144;                         // bytes per 256 columns of one row
    static constexpr int SLOT = STAGE_SB * UB;             // shared bytes per row per stage; 288 % 128 == 32, so the four rows a
                                                           // half-warp reads with 64-bit loads fall in four different bank groups
    static constexpr int SCALE_BYTES = STAGE_SB * UNIT_ROWS * (32 + 16 + 4);  // d*s[8] f32, mins[4] u32, dmin f32
};

// Token-slot geometry. TS is the number of token slots (1, 2, 4 or 8).
template <int TS> struct Cols {
    static constexpr int NP = TS == 8 ? 2 : 1;       // mmas per 16 columns
    static constexpr int NS = TS == 8 ? 8 : 2 * TS;  // stored B columns per piece array
    static constexpr int X_BYTES = NP * KSL * 32 * NS * 16;
    static constexpr int S_BYTES = NP * KSL * 4 * NS * 4;
};

template <int ENC, int TS> constexpr int smem_bytes() {
    return Cols<TS>::X_BYTES + Cols<TS>::S_BYTES + 256 /* inv scale + max scratch */ +
           WARPS * (STAGES * UNIT_ROWS * Geo<ENC>::SLOT + Geo<ENC>::SCALE_BYTES) + WARPS * STAGES * 8 + 128;
}

// The warp's sequence of pipeline steps: its units in order, each cut into
// chunks of STAGE_SB superblocks.
struct Cursor {
    uint32_t unit;   // global unit index
    uint32_t chunk;  // chunk within the unit's slice
};

__device__ __forceinline__ uint32_t slice_sbs(const Params &p, uint32_t ks) { return min((uint32_t)KSL, p.ksb - ks * KSL); }

__device__ __forceinline__ void advance(const Params &p, Cursor &c) {
    const uint32_t ks = c.unit / p.total_rb;
    const uint32_t chunks = (slice_sbs(p, ks) + STAGE_SB - 1) / STAGE_SB;
    if (++c.chunk == chunks) {
        c.chunk = 0;
        c.unit += WARPS;
    }
}

struct UnitRows {
    const uint8_t *base[2];  // first row of each 16-row tile
    uint32_t rows_left[2];   // valid rows in each tile (may exceed 16)
    unsigned long long stride;
};

// Row block `rb` -> the two 16-row tiles it covers. Plain mode: 32 consecutive
// rows of one segment. Pair mode: rows [16 rb, 16 rb + 16) of segment 0 and of segment 1.
__device__ __forceinline__ void unit_rows(const Params &p, uint32_t rb, uint32_t &seg, uint32_t &row0, UnitRows &u) {
    if (p.mode != ACT_NONE) {
        seg = 0;
        row0 = rb * 16;
        u.stride = p.stride[0];
        u.base[0] = p.w[0] + (size_t)row0 * p.stride[0];
        u.base[1] = p.w[1] + (size_t)row0 * p.stride[1];
        u.rows_left[0] = u.rows_left[1] = p.rows[0] - row0;
    } else {
        seg = 0;
#pragma unroll
        for (int s = 1; s < 4; ++s)
            if ((uint32_t)s < p.count && rb >= p.rb_begin[s]) seg = s;
        row0 = (rb - p.rb_begin[seg]) * UNIT_ROWS;
        u.stride = p.stride[seg];
        u.base[0] = p.w[seg] + (size_t)row0 * u.stride;
        u.base[1] = u.base[0] + 16 * u.stride;
        u.rows_left[0] = p.rows[seg] - row0;
        u.rows_left[1] = u.rows_left[0] > 16 ? u.rows_left[0] - 16 : 0;
    }
}

// Issues the bulk copies of one pipeline step: lane r copies row r of the unit
// (rows past the matrix re-read its last row; their results are never stored).
template <int ENC>
__device__ __forceinline__ void issue_step(const Params &p, const Cursor &c, uint32_t stage_base, uint32_t bar, uint32_t lane, uint64_t policy) {
    const uint32_t ks = c.unit / p.total_rb, rb = c.unit % p.total_rb;
    uint32_t seg, row0;
    UnitRows u;
    unit_rows(p, rb, seg, row0, u);
    const uint32_t sb0 = ks * KSL + c.chunk * STAGE_SB;
    const uint32_t nsb = min((uint32_t)STAGE_SB, min((uint32_t)KSL, p.ksb - ks * KSL) - c.chunk * STAGE_SB);
    const uint32_t bytes = nsb * Geo<ENC>::UB;
    if (lane == 0) mbar_expect_tx(bar, bytes * UNIT_ROWS);
    __syncwarp();
    const uint32_t tile = lane >> 4, r = lane & 15;
    const uint32_t valid = u.rows_left[tile];
    // A tile wholly past the matrix (pair mode never has one) re-reads tile 0.
    const uint8_t *base = valid ? u.base[tile] : u.base[0];
    const uint32_t lim = valid ? valid : u.rows_left[0];
    const uint32_t rr = min(r, lim - 1);
    const unsigned long long stride = (p.mode != ACT_NONE) ? p.stride[tile] : u.stride;
    const uint8_t *src = base + (size_t)rr * stride + (size_t)sb0 * Geo<ENC>::UB;
    bulk_load(stage_base + lane * Geo<ENC>::SLOT, src, bytes, bar, policy);
}

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
    return (n >> 2) * TS + (n & 3);  // pieces side by side: columns 0..3 hi, 4..7 lo
}

template <int TS>
__device__ void stage_activations(const Params &p, uint32_t ks, uint8_t *xs, uint8_t *ss, float *inv_scale, float *red) {
    using C = Cols<TS>;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t nsb = slice_sbs(p, ks);
    const uint32_t groups = nsb * 32;  // column groups of 8 in the slice
    const uint32_t col_base = ks * KSL * 256;
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
        const float m = fmaxf(fmaxf(red[t], red[8 + t]), fmaxf(red[16 + t], red[24 + t]));
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
        const int order[8] = {0, 2, 1, 3, 4, 6, 5, 7};
        uint32_t whi[4], wlo[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            whi[i] = (uint32_t)__half_as_ushort(hi[order[2 * i]]) | ((uint32_t)__half_as_ushort(hi[order[2 * i + 1]]) << 16);
            wlo[i] = (uint32_t)__half_as_ushort(lo[order[2 * i]]) | ((uint32_t)__half_as_ushort(lo[order[2 * i + 1]]) << 16);
        }
        const uint32_t grp = cg >> 2;  // 32-column group within the slice
        if (TS == 8) {
            *(uint4 *)(xs + ((size_t)cg * C::NS + tok) * 16) = make_uint4(whi[0], whi[1], whi[2], whi[3]);
            *(uint4 *)(xs + C::X_BYTES / 2 + ((size_t)cg * C::NS + tok) * 16) = make_uint4(wlo[0], wlo[1], wlo[2], wlo[3]);
            if ((lane & 3) == 0) {
                *(__half *)(ss + ((size_t)(grp >> 1) * C::NS + tok) * 4 + (grp & 1) * 2) = mhi;
                *(__half *)(ss + C::S_BYTES / 2 + ((size_t)(grp >> 1) * C::NS + tok) * 4 + (grp & 1) * 2) = mlo;
            }
        } else {
            *(uint4 *)(xs + ((size_t)cg * C::NS + tok) * 16) = make_uint4(whi[0], whi[1], whi[2], whi[3]);
            *(uint4 *)(xs + ((size_t)cg * C::NS + TS + tok) * 16) = make_uint4(wlo[0], wlo[1], wlo[2], wlo[3]);
            if ((lane & 3) == 0) {
                *(__half *)(ss + ((size_t)(grp >> 1) * C::NS + tok) * 4 + (grp & 1) * 2) = mhi;
                *(__half *)(ss + ((size_t)(grp >> 1) * C::NS + TS + tok) * 4 + (grp & 1) * 2) = mlo;
            }
        }
    }
}

// ---- Q4_K: scale pre-pass and the mma loop over one pipeline step -----------------------

// Decodes the packed 6-bit scales and minima of the step's (row, superblock)
// pairs once per warp: d*s as F32 with the 2^24 (low nibble) or 2^20 (high
// nibble) of the subnormal trick folded in, the minima as fp16 subnormals
// (m * 2^-24) in mma A order, and dmin * 2^29 (2^24 from the minima, 2^5 from
// the group sums stored as means).
__device__ __forceinline__ void q4k_prepass(uint32_t stage, uint32_t nsb, uint8_t *scales, uint32_t lane) {
    float *dsf = (float *)scales;                                   // [sb][row][8]
    uint32_t *mins = (uint32_t *)(scales + STAGE_SB * UNIT_ROWS * 32);  // [sb][row][4]
    float *dmin = (float *)(scales + STAGE_SB * UNIT_ROWS * 48);        // [sb][row]
    for (uint32_t pi = lane; pi < nsb * UNIT_ROWS; pi += 32) {
        const uint32_t row = pi % UNIT_ROWS, sb = pi / UNIT_ROWS;
        const uint4 hdr = lds128(stage + row * Geo<Q4_K>::SLOT + sb * 144);
        const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
        const float dm = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
        // Packed bytes: s[0..3], m[0..3], then s[4..7] and m[4..7] from the split fields.
        const uint32_t s_lo = hdr.y & 0x3f3f3f3fu;
        const uint32_t m_lo = hdr.z & 0x3f3f3f3fu;
        const uint32_t s_hi = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
        const uint32_t m_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
        float out[8];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            out[g] = (float)((s_lo >> (8 * g)) & 0xffu);
            out[4 + g] = (float)((s_hi >> (8 * g)) & 0xffu);
        }
        const float even = d * 16777216.0f, odd = d * 1048576.0f;
#pragma unroll
        for (int g = 0; g < 8; ++g) out[g] *= (g & 1) ? odd : even;
        float4 *dst = (float4 *)(dsf + ((size_t)sb * UNIT_ROWS + row) * 8);
        dst[0] = make_float4(out[0], out[1], out[2], out[3]);
        dst[1] = make_float4(out[4], out[5], out[6], out[7]);
        // minima pairs (m[2t], m[2t+1]) as two 16-bit integers = fp16 subnormals
        uint4 mm;
        mm.x = (m_lo & 0xffu) | ((m_lo & 0xff00u) << 8);
        mm.y = ((m_lo >> 16) & 0xffu) | ((m_lo >> 8) & 0xff0000u);
        mm.z = (m_hi & 0xffu) | ((m_hi & 0xff00u) << 8);
        mm.w = ((m_hi >> 16) & 0xffu) | ((m_hi >> 8) & 0xff0000u);
        *(uint4 *)(mins + ((size_t)sb * UNIT_ROWS + row) * 4) = mm;
        dmin[sb * UNIT_ROWS + row] = dm * 536870912.0f;
    }
}

template <int TS>
__device__ __forceinline__ void q4k_step(uint32_t stage, uint32_t nsb, uint32_t sb_in_slice, uint32_t scales, uint32_t xs, uint32_t ss,
                                         uint32_t lane, float acc[2][4]) {
    using C = Cols<TS>;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t slot = b_slot<TS>(g);
    const bool b_valid = TS == 8 || (g & 3u) < (uint32_t)TS;
    const uint32_t dsf = scales, mins = scales + STAGE_SB * UNIT_ROWS * 32, dmin = scales + STAGE_SB * UNIT_ROWS * 48;
    for (uint32_t sb = 0; sb < nsb; ++sb) {
        const uint32_t xsb = xs + (sb_in_slice + sb) * 32 * C::NS * 16;
        const uint32_t ssb = ss + (sb_in_slice + sb) * 4 * C::NS * 4;
        // min term: one k8 mma per tile over the eight group means
        float cmin[2][4];
        uint32_t sfrag[C::NP];
#pragma unroll
        for (int a = 0; a < C::NP; ++a) sfrag[a] = b_valid ? lds32(ssb + a * (C::S_BYTES / 2) + (t * C::NS + slot) * 4) : 0u;
        float ds[2][2][8];  // [tile][row g / g+8][group]
#pragma unroll
        for (int rt = 0; rt < 2; ++rt) {
#pragma unroll
            for (int i = 0; i < 4; ++i) cmin[rt][i] = 0.0f;
            const uint32_t r0 = (sb * UNIT_ROWS + rt * 16 + g);
            const uint32_t m0 = lds32(mins + (r0 * 4 + t) * 4), m1 = lds32(mins + ((r0 + 8) * 4 + t) * 4);
#pragma unroll
            for (int a = 0; a < C::NP; ++a) mma1688(cmin[rt], m0, m1, sfrag[a]);
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const uint4 lo4 = lds128(dsf + (r0 + hrow * 8) * 32), hi4 = lds128(dsf + (r0 + hrow * 8) * 32 + 16);
                ds[rt][hrow][0] = __uint_as_float(lo4.x); ds[rt][hrow][1] = __uint_as_float(lo4.y);
                ds[rt][hrow][2] = __uint_as_float(lo4.z); ds[rt][hrow][3] = __uint_as_float(lo4.w);
                ds[rt][hrow][4] = __uint_as_float(hi4.x); ds[rt][hrow][5] = __uint_as_float(hi4.y);
                ds[rt][hrow][6] = __uint_as_float(hi4.z); ds[rt][hrow][7] = __uint_as_float(hi4.w);
            }
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            uint2 wq[2][2];  // [tile][row g / g+8] -> words for h = 0, 1
#pragma unroll
            for (int rt = 0; rt < 2; ++rt) {
                const uint32_t a = stage + (rt * 16 + g) * Geo<Q4_K>::SLOT + sb * 144 + 16 + p * 32 + t * 8;
                wq[rt][0] = lds64(a);
                wq[rt][1] = lds64(a + 8 * Geo<Q4_K>::SLOT);
            }
#pragma unroll
            for (int odd = 0; odd < 2; ++odd) {
                const uint32_t mask = odd ? 0x00f000f0u : 0x000f000fu;
                uint4 bf[C::NP];
#pragma unroll
                for (int a = 0; a < C::NP; ++a)
                    bf[a] = b_valid ? lds128(xsb + a * (C::X_BYTES / 2) + (((p * 2 + odd) * 4 + t) * C::NS + slot) * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int rt = 0; rt < 2; ++rt) {
                    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    uint32_t a0[4], a1[4];
                    a0[0] = wq[rt][0].x & mask; a0[1] = wq[rt][1].x & mask;
                    a0[2] = (wq[rt][0].x >> 8) & mask; a0[3] = (wq[rt][1].x >> 8) & mask;
                    a1[0] = wq[rt][0].y & mask; a1[1] = wq[rt][1].y & mask;
                    a1[2] = (wq[rt][0].y >> 8) & mask; a1[3] = (wq[rt][1].y >> 8) & mask;
#pragma unroll
                    for (int a = 0; a < C::NP; ++a) {
                        mma16816(c, a0, bf[a].x, bf[a].y);
                        mma16816(c, a1, bf[a].z, bf[a].w);
                    }
                    const float s0 = ds[rt][0][2 * p + odd], s1 = ds[rt][1][2 * p + odd];
                    acc[rt][0] = fmaf(s0, c[0], acc[rt][0]);
                    acc[rt][1] = fmaf(s0, c[1], acc[rt][1]);
                    acc[rt][2] = fmaf(s1, c[2], acc[rt][2]);
                    acc[rt][3] = fmaf(s1, c[3], acc[rt][3]);
                }
            }
        }
#pragma unroll
        for (int rt = 0; rt < 2; ++rt) {
            const uint32_t r0 = (sb * UNIT_ROWS + rt * 16 + g);
            const float d0 = __uint_as_float(lds32(dmin + r0 * 4)), d1 = __uint_as_float(lds32(dmin + (r0 + 8) * 4));
            acc[rt][0] = fmaf(-d0, cmin[rt][0], acc[rt][0]);
            acc[rt][1] = fmaf(-d0, cmin[rt][1], acc[rt][1]);
            acc[rt][2] = fmaf(-d1, cmin[rt][2], acc[rt][2]);
            acc[rt][3] = fmaf(-d1, cmin[rt][3], acc[rt][3]);
        }
    }
}

// ---- the kernel -------------------------------------------------------------------------------

template <int ENC, int TS>
__global__ void __launch_bounds__(THREADS, 1) fast_kernel(const Params p) {
    using C = Cols<TS>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *xs = smem;
    uint8_t *ss = xs + C::X_BYTES;
    float *inv_scale = (float *)(ss + C::S_BYTES);
    float *red = inv_scale + 8;  // 32 floats
    uint8_t *warp_area = ss + C::S_BYTES + 256;
    constexpr int WARP_BYTES = STAGES * UNIT_ROWS * Geo<ENC>::SLOT + Geo<ENC>::SCALE_BYTES;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint8_t *stages = warp_area + warp * WARP_BYTES;
    uint8_t *scales = stages + STAGES * UNIT_ROWS * Geo<ENC>::SLOT;
    uint64_t *bars = (uint64_t *)(warp_area + WARPS * WARP_BYTES);
    const uint32_t bar0 = smem_u32(bars + warp * STAGES);
    const uint32_t stage0 = smem_u32(stages);

    if (tid == 0) {
        for (int i = 0; i < WARPS * STAGES; ++i) mbar_init(smem_u32(bars + i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const uint32_t total_units = p.nks * p.total_rb;
    const uint32_t u_begin = (uint32_t)((unsigned long long)total_units * blockIdx.x / gridDim.x);
    const uint32_t u_end = (uint32_t)((unsigned long long)total_units * (blockIdx.x + 1) / gridDim.x);
    if (u_begin >= u_end) return;
    const uint64_t policy = evict_first_policy();

    // Producer side: this warp's steps, issued STAGES - 1 ahead of their use.
    Cursor prod = {u_begin + warp, 0};
    uint32_t issued = 0;
    for (; issued < STAGES - 1 && prod.unit < u_end; ++issued) {
        issue_step<ENC>(p, prod, stage0 + (issued % STAGES) * UNIT_ROWS * Geo<ENC>::SLOT, bar0 + (issued % STAGES) * 8, lane, policy);
        advance(p, prod);
    }
    Cursor cons = {u_begin + warp, 0};
    uint32_t consumed = 0;
    bool failed = false;

    const uint32_t ks_first = u_begin / p.total_rb, ks_last = (u_end - 1) / p.total_rb;
    for (uint32_t ks = ks_first; ks <= ks_last; ++ks) {
        __syncthreads();  // every warp is done with the previous slice's activations
        stage_activations<TS>(p, ks, xs, ss, inv_scale, red);
        __syncthreads();
        const uint32_t slice_end = min(u_end, (ks + 1) * p.total_rb);
        const uint32_t chunks = (slice_sbs(p, ks) + STAGE_SB - 1) / STAGE_SB;
        while (!failed && cons.unit < slice_end) {
            float acc[2][4];
#pragma unroll
            for (int rt = 0; rt < 2; ++rt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[rt][i] = 0.0f;
            for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
                // keep the pipeline full: issue the step STAGES - 1 ahead
                if (prod.unit < u_end) {
                    issue_step<ENC>(p, prod, stage0 + (issued % STAGES) * UNIT_ROWS * Geo<ENC>::SLOT, bar0 + (issued % STAGES) * 8, lane, policy);
                    advance(p, prod);
                    ++issued;
                }
                const uint32_t st = consumed % STAGES;
                if (!mbar_wait(bar0 + st * 8, (consumed / STAGES) & 1u)) {
                    failed = true;
                    break;
                }
                const uint32_t nsb = min((uint32_t)STAGE_SB, slice_sbs(p, ks) - chunk * STAGE_SB);
                const uint32_t stage = stage0 + st * UNIT_ROWS * Geo<ENC>::SLOT;
                q4k_prepass(stage, nsb, scales, lane);
                __syncwarp();
                q4k_step<TS>(stage, nsb, chunk * STAGE_SB, smem_u32(scales), smem_u32(xs), smem_u32(ss), lane, acc);
                __syncwarp();  // all lanes are done reading this stage before it is refilled
                ++consumed;
            }
            if (failed) break;
            // ---- unit epilogue ----
            const uint32_t rb = cons.unit % p.total_rb;
            uint32_t seg, row0;
            UnitRows u;
            unit_rows(p, rb, seg, row0, u);
            const uint32_t g = lane >> 2, t = lane & 3;
            float v[2][4];
#pragma unroll
            for (int rt = 0; rt < 2; ++rt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float a = acc[rt][i];
                    if (TS != 8) a += __shfl_xor_sync(0xffffffffu, a, 2);  // hi columns + lo columns
                    v[rt][i] = a;
                }
            const bool owner = TS == 8 || t < 2;
            const uint32_t tok0 = 2 * t;  // tokens tok0, tok0 + 1 (for TS < 8 only lanes t < 2 own tokens)
            if (p.nks == 1) {
                if (owner) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint32_t tok = tok0 + j;
                        if (tok >= p.tokens) continue;
                        const float is = inv_scale[tok];
#pragma unroll
                        for (int hrow = 0; hrow < 2; ++hrow) {
                            const uint32_t r = g + hrow * 8;
                            if (p.mode != ACT_NONE) {
                                if (r < u.rows_left[0]) {
                                    const float gate = v[0][hrow * 2 + j] * is, up = v[1][hrow * 2 + j] * is;
                                    const float a = p.mode == ACT_SILU ? silu_f32(gate) : gelu_f32(gate);
                                    p.out[0][(size_t)tok * p.out_stride[0] + row0 + r] = a * up;
                                }
                            } else {
#pragma unroll
                                for (int rt = 0; rt < 2; ++rt)
                                    if (r < u.rows_left[rt])
                                        p.out[seg][(size_t)tok * p.out_stride[seg] + row0 + rt * 16 + r] = v[rt][hrow * 2 + j] * is;
                            }
                        }
                    }
                }
            } else {
                // partial sums, then the last arrival for this row block adds them in slice order
                if (owner) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint32_t tok = tok0 + j;
                        if (tok >= p.tokens) continue;
                        const float is = inv_scale[tok];
#pragma unroll
                        for (int rt = 0; rt < 2; ++rt)
#pragma unroll
                            for (int hrow = 0; hrow < 2; ++hrow) {
                                const uint32_t r = g + hrow * 8;
                                uint32_t prow;
                                if (p.mode != ACT_NONE) prow = p.prow_begin[rt] + row0 + r;
                                else prow = p.prow_begin[seg] + row0 + rt * 16 + r;
                                p.partials[((size_t)ks * p.total_prows + prow) * p.tokens + tok] = v[rt][hrow * 2 + j] * is;
                            }
                    }
                }
                __threadfence();
                __syncwarp();
                uint32_t arrived = 0;
                if (lane == 0) arrived = atomicAdd(p.counters + rb, 1u);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (arrived == p.nks - 1) {
                    __threadfence();
                    const uint32_t per_tile = 16 * p.tokens;
                    if (p.mode != ACT_NONE) {
                        for (uint32_t e = lane; e < per_tile; e += 32) {
                            const uint32_t r = e / p.tokens, tok = e % p.tokens;
                            if (r >= u.rows_left[0]) continue;
                            float gate = 0.0f, up = 0.0f;
                            for (uint32_t k = 0; k < p.nks; ++k) {
                                gate += __ldcg(p.partials + ((size_t)k * p.total_prows + p.prow_begin[0] + row0 + r) * p.tokens + tok);
                                up += __ldcg(p.partials + ((size_t)k * p.total_prows + p.prow_begin[1] + row0 + r) * p.tokens + tok);
                            }
                            const float a = p.mode == ACT_SILU ? silu_f32(gate) : gelu_f32(gate);
                            p.out[0][(size_t)tok * p.out_stride[0] + row0 + r] = a * up;
                        }
                    } else {
                        for (uint32_t e = lane; e < 2 * per_tile; e += 32) {
                            const uint32_t r = e / p.tokens, tok = e % p.tokens;
                            if (r >= u.rows_left[0]) continue;
                            float sum = 0.0f;
                            for (uint32_t k = 0; k < p.nks; ++k)
                                sum += __ldcg(p.partials + ((size_t)k * p.total_prows + p.prow_begin[seg] + row0 + r) * p.tokens + tok);
                            p.out[seg][(size_t)tok * p.out_stride[seg] + row0 + r] = sum;
                        }
                    }
                    if (lane == 0) p.counters[rb] = 0;  // leave the scratch as it was found
                }
            }
            cons.unit += WARPS;
        }
    }
    if (failed) {
        if (lane == 0) atomicExch(p.status, 1u);
        // Let this warp's copies still in flight land before the block's shared memory is released.
        for (; consumed < issued; ++consumed) mbar_wait(bar0 + (consumed % STAGES) * 8, (consumed / STAGES) & 1u);
    }
}

}  // namespace fast

// ---- host side ------------------------------------------------------------------------------------

static uint32_t token_slots(uint32_t tokens) { return tokens <= 1 ? 1 : tokens <= 2 ? 2 : tokens <= 4 ? 4 : 8; }

static bool fill_params(const FastJob &job, fast::Params &p) {
    if (job.enc != Q4_K) return false;
    if (job.tokens < 1 || job.tokens > 8 || job.count < 1 || job.count > 4) return false;
    if (job.columns == 0 || job.columns % 256 != 0) return false;
    if ((uintptr_t)job.in % 16 != 0 || (job.tokens > 1 && job.in_stride % 4 != 0)) return false;
    if (job.mode != ACT_NONE && (job.count != 2 || job.seg[0].rows != job.seg[1].rows)) return false;
    p = fast::Params{};
    p.count = job.count;
    p.mode = job.mode;
    p.tokens = job.tokens;
    p.ksb = job.columns / 256;
    p.nks = (p.ksb + fast::KSL - 1) / fast::KSL;
    p.in = job.in;
    p.in_stride = job.in_stride;
    uint32_t rb = 0, prow = 0;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows == 0 || (uintptr_t)g.w % 16 != 0 || g.stride % 16 != 0 || (uintptr_t)g.out % 4 != 0) return false;
        p.w[s] = g.w;
        p.stride[s] = g.stride;
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
    p.partials = job.partials;
    p.counters = job.counters;
    if (p.nks > 1) {
        if ((size_t)p.nks * prow * job.tokens > job.partials_floats) return false;
        if (rb > job.counters_len) return false;
    }
    return true;
}

bool fast_supported(const FastJob &job) {
    fast::Params p;
    return fill_params(job, p);
}

template <int ENC, int TS>
static bool configure_variant() {
    return cudaFuncSetAttribute(fast::fast_kernel<ENC, TS>, cudaFuncAttributeMaxDynamicSharedMemorySize, fast::smem_bytes<ENC, TS>()) == cudaSuccess;
}

bool fast_configure() {
    return configure_variant<Q4_K, 1>() && configure_variant<Q4_K, 2>() && configure_variant<Q4_K, 4>() && configure_variant<Q4_K, 8>();
}

template <int ENC, int TS>
static int launch_variant(cudaStream_t s, const fast::Params &p, int sm_count) {
    constexpr int bytes = fast::smem_bytes<ENC, TS>();
    const uint32_t units = p.nks * p.total_rb;
    const uint32_t grid = units < (uint32_t)sm_count ? units : (uint32_t)sm_count;
    fast::fast_kernel<ENC, TS><<<grid, fast::THREADS, bytes, s>>>(p);
    return 1;
}

int launch_fast(cudaStream_t s, const FastJob &job) {
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
