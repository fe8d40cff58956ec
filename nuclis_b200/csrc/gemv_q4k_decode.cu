// Q4_K decode GEMV (one activation row) for sm_100a: the kernel behind
// Backend.matvec and single-row matvecSegments on Q4_K weights
// (inference/src/backends/metal/ops/matvec.zig:85-116, 268-343; the reference's
// kernel for this is nu_matvec_q4_k, kernels/matvec.metal:161-209).
//
// The HBM stream is the only large traffic: every weight byte is loaded once,
// straight from global memory into registers with 128-bit loads (a quad of
// lanes reads the 128 contiguous quant bytes of a superblock row), one task
// (16 rows x 256 columns) prefetched ahead of the one being computed, and 16
// warps per SM keep those loads in flight. Nothing but the activations is
// staged in shared memory.
//
// Arithmetic. The 4-bit codes are exact in fp16: a code masked in place in its
// 16-bit lane is the fp16 subnormal code * 2^-24 (or * 2^-20 for a high
// nibble), so it becomes an mma.sync.m16n8k16 A operand with no conversion.
// The activation row is scaled by a power of two and split into fp16 pieces
// hi + lo (22 significant bits); products of fp16 values are exact and are
// accumulated in F32 by the tensor core.
// With one token the 8 columns of the B operand are free, so B is made block
// diagonal: lane t of a quad owns group pair t of the superblock (groups 2t and
// 2t+1, its own 32 quant bytes), supplies that pair's codes as its four k
// indices, and columns 2t (hi) and 2t+1 (lo) of B hold x for those k only.
// Each lane thus receives the sums of its own group, needs only its own
// group's 6-bit scale and minimum, and applies d*scale once per group per
// superblock: sum_g d*s_g*sum(q*x) - dmin*sum_g m_g*sum(x), the factored form
// of kernels/matvec.metal:197.
//
// Work split. K is cut into `nks` slices; a unit is a 16-row tile by one slice,
// a task one superblock of a unit. Units are dealt to persistent blocks (one per
// SM) in contiguous, slice-major ranges; inside a block tasks go round-robin to
// the warps, each leaves its 16 row sums in a shared-memory slot, and after a
// block-wide barrier the slots of a unit are added in superblock order. With
// several slices those sums go to a global scratch array and the last block to
// arrive for a row tile adds them in slice order. No sum depends on timing.
#include <cuda_fp16.h>

#include "kernels.hpp"
#include "nu_device.cuh"

namespace nu {
namespace dec {

constexpr int WARPS = 16;
constexpr int THREADS = WARPS * 32;
constexpr int ROUND_TASKS = 512;  // task slots per round: 32 KiB of row sums

struct Params {
    const uint8_t *w[4];
    unsigned long long stride[4];
    float *out[4];
    uint32_t rows[4];
    uint32_t tile_begin[5];  // first 16-row tile of each segment in the tile list
    uint32_t count, mode;
    uint32_t ksb, ksl, nks;  // superblocks per row, per slice; slices
    uint32_t total_tiles;    // tiles per slice (pair mode: gate and up tiles interleaved)
    const float *in;
    float *partials;         // [slice][tile][16]
    uint32_t *counters;      // per output tile (pair mode: per gate/up tile pair)
};

__device__ __forceinline__ void mma16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16816_first(float d[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}
// Streaming 128-bit load: the weights are read once, keep them out of L1.
__device__ __forceinline__ uint4 ldg_stream(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t slice_sbs(const Params &p, uint32_t ks) { return min(p.ksl, p.ksb - ks * p.ksl); }

// Tile `tile` of the list -> segment and first row. Pair mode interleaves the
// tiles of the gate (even) and up (odd) segments.
__device__ __forceinline__ void tile_rows(const Params &p, uint32_t tile, uint32_t &seg, uint32_t &row0) {
    if (p.mode != ACT_NONE) {
        seg = tile & 1u;
        row0 = (tile >> 1) * 16;
    } else {
        seg = 0;
#pragma unroll
        for (int s = 1; s < 4; ++s)
            if ((uint32_t)s < p.count && tile >= p.tile_begin[s]) seg = s;
        row0 = (tile - p.tile_begin[seg]) * 16;
    }
}

struct TaskData {
    uint4 hdr[2], q0[2], q1[2];  // rows g and g+8: block header, quant bytes [32t, 32t+16) and [32t+16, 32t+32)
};
__device__ __forceinline__ uint32_t word(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// The six loads of a task for this lane.
__device__ __forceinline__ void load_task(const Params &p, uint32_t tile, uint32_t sb_abs, uint32_t lane, TaskData &d) {
    uint32_t seg, row0;
    tile_rows(p, tile, seg, row0);
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t last = p.rows[seg] - 1;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t row = min(row0 + g + h * 8, last);  // rows past the matrix re-read the last row; never stored
        const uint8_t *b = p.w[seg] + (size_t)row * p.stride[seg] + (size_t)sb_abs * 144;
        d.hdr[h] = ldg_stream(b);
        d.q0[h] = ldg_stream(b + 16 + t * 32);
        d.q1[h] = ldg_stream(b + 32 + t * 32);
    }
}

// d*s (with the 2^24 / 2^20 of the subnormal codes) and dmin*m of this lane's two groups, for one row.
struct RowScales {
    float ds_e, ds_o, dm_e, dm_o;
};
__device__ __forceinline__ RowScales row_scales(const uint4 &hdr, uint32_t t) {
    const uint32_t shift = (t & 1u) * 16;
    const uint32_t y = (hdr.y >> shift) & 0xffffu, z = (hdr.z >> shift) & 0xffffu, w = (hdr.w >> shift) & 0xffffu;
    // groups 0..3: low six bits of bytes 0..3 / 4..7; groups 4..7: nibbles of bytes 8..11 plus the top two bits of bytes 0..7
    const uint32_t s_lo = y & 0x3f3fu, m_lo = z & 0x3f3fu;
    const uint32_t s_hi = (w & 0x0f0fu) | ((y >> 2) & 0x3030u), m_hi = ((w >> 4) & 0x0f0fu) | ((z >> 2) & 0x3030u);
    const uint32_t s2 = t < 2 ? s_lo : s_hi, m2 = t < 2 ? m_lo : m_hi;
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    // byte -> float through the 2^23 magic number: one permute and one FMA each
    const float se = __uint_as_float(__byte_perm(s2, 0x4b000000u, 0x7650)), so = __uint_as_float(__byte_perm(s2, 0x4b000000u, 0x7651));
    const float me = __uint_as_float(__byte_perm(m2, 0x4b000000u, 0x7650)), mo = __uint_as_float(__byte_perm(m2, 0x4b000000u, 0x7651));
    const float de = d * 16777216.0f, d_odd = d * 1048576.0f;
    RowScales r;
    r.ds_e = fmaf(se, de, -8388608.0f * de);
    r.ds_o = fmaf(so, d_odd, -8388608.0f * d_odd);
    r.dm_e = fmaf(me, dmin, -8388608.0f * dmin);
    r.dm_o = fmaf(mo, dmin, -8388608.0f * dmin);
    return r;
}

template <bool UNUSED = false>
__global__ void __launch_bounds__(THREADS, 1) q4k_decode_kernel(const Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t K = p.ksb * 256;
    // [hi pieces K halves][lo pieces K halves][128 B of zeros][group sums K/32 floats][slots][scratch]
    uint8_t *xhi = smem;
    uint8_t *xlo = xhi + (size_t)K * 2;
    uint8_t *zero = xlo + (size_t)K * 2;
    float *gsum = (float *)(zero + 128);
    float *slots = gsum + K / 32;
    float *red = slots + ROUND_TASKS * 16;  // WARPS floats + inverse scale
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;

    // ---- stage the activation row: scale, split into fp16 pieces, group sums ----
    float mx = 0.0f;
    for (uint32_t i = tid; i < K / 4; i += THREADS) {
        const float4 v = ((const float4 *)p.in)[i];
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    if (tid < 32) ((uint32_t *)zero)[tid] = 0;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) mx = fmaxf(mx, red[w]);
    // 2^e puts the largest |x| in [2^13, 2^14): hi cannot overflow fp16, lo keeps 11 bits down to 2^-25 of the largest value
    const uint32_t e = (__float_as_uint(mx) >> 23) & 0xffu;
    const bool ok = e >= 40u && e < 255u;
    const float scale = ok ? __uint_as_float((267u - e) << 23) : 1.0f;
    const float inv_scale = ok ? __uint_as_float((e - 13u) << 23) : 1.0f;
    for (uint32_t i = tid; i < K / 4; i += THREADS) {
        const float4 v = ((const float4 *)p.in)[i];
        const float x0 = v.x * scale, x1 = v.y * scale, x2 = v.z * scale, x3 = v.w * scale;
        const __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1), h2 = __float2half_rn(x2), h3 = __float2half_rn(x3);
        const __half l0 = __float2half_rn(x0 - __half2float(h0)), l1 = __float2half_rn(x1 - __half2float(h1));
        const __half l2 = __float2half_rn(x2 - __half2float(h2)), l3 = __float2half_rn(x3 - __half2float(h3));
        // k order of the A operand built below: columns +0, +2 in the first register, +1, +3 in the second
        uint2 hi, lo;
        hi.x = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h2) << 16);
        hi.y = (uint32_t)__half_as_ushort(h1) | ((uint32_t)__half_as_ushort(h3) << 16);
        lo.x = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l2) << 16);
        lo.y = (uint32_t)__half_as_ushort(l1) | ((uint32_t)__half_as_ushort(l3) << 16);
        ((uint2 *)xhi)[i] = hi;
        ((uint2 *)xlo)[i] = lo;
        // 32-column group sum: eight consecutive threads hold a group
        float s = (x0 + x1) + (x2 + x3);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if ((lane & 7) == 0) gsum[i >> 3] = s;
    }
    __syncthreads();

    const uint32_t total_units = p.nks * p.total_tiles;
    // contiguous unit range of this block; pair mode keeps a gate tile and its up tile in one block
    uint32_t u_begin = (uint32_t)((unsigned long long)total_units * blockIdx.x / gridDim.x);
    uint32_t u_end = (uint32_t)((unsigned long long)total_units * (blockIdx.x + 1) / gridDim.x);
    if (p.mode != ACT_NONE) { u_begin &= ~1u; u_end &= ~1u; if (blockIdx.x + 1 == gridDim.x) u_end = total_units; }

    // Lanes whose B column is not theirs (column n = lane >> 2 belongs to quad lane n >> 1) read zeros.
    const bool mine = (g >> 1) == t;
    const uint8_t *piece = (g & 1u) ? xlo : xhi;

    uint32_t round_begin = u_begin;
    while (round_begin < u_end) {
        // a round: whole units, at most ROUND_TASKS tasks
        uint32_t round_end = round_begin, round_tasks = 0;
        while (round_end < u_end) {
            const uint32_t n = slice_sbs(p, round_end / p.total_tiles);
            if (round_tasks + n > ROUND_TASKS && round_end > round_begin) break;
            round_tasks += n;
            ++round_end;
        }
        if (p.mode != ACT_NONE && ((round_end - round_begin) & 1u)) --round_end;  // a gate tile and its up tile share a round
        // ---- tasks of the round, round-robin over the warps; one task of loads in flight ahead ----
        // cursor: unit cu, superblock csb in its slice, task index cj in the round
        uint32_t cu = round_begin, cks = cu / p.total_tiles, ctile = cu - cks * p.total_tiles, csb = warp, cj = warp;
        auto normalize = [&](uint32_t &u, uint32_t &ks, uint32_t &tile, uint32_t &sb) {
            uint32_t n = slice_sbs(p, ks);
            while (sb >= n && u < round_end) {
                sb -= n;
                ++u;
                if (++tile == p.total_tiles) { tile = 0; ++ks; n = ks < p.nks ? slice_sbs(p, ks) : 1u; }
            }
        };
        normalize(cu, cks, ctile, csb);
        auto compute = [&](const TaskData &cur, uint32_t sb_abs, uint32_t j) {
            const uint8_t *xb = mine ? piece + (size_t)sb_abs * 512 + t * 128 : zero;  // 64 columns of this pair: 128 B of halves
            float ce[4], co[4];  // even group / odd group: (hi, lo) sums of row g, (hi, lo) of row g+8
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t w0 = i < 4 ? word(cur.q0[0], i) : word(cur.q1[0], i - 4);
                const uint32_t w1 = i < 4 ? word(cur.q0[1], i) : word(cur.q1[1], i - 4);
                const uint32_t s0 = w0 >> 8, s1 = w1 >> 8;
                uint32_t ae[4], ao[4];
                ae[0] = w0 & 0x000f000fu; ae[1] = w1 & 0x000f000fu; ae[2] = s0 & 0x000f000fu; ae[3] = s1 & 0x000f000fu;
                ao[0] = w0 & 0x00f000f0u; ao[1] = w1 & 0x00f000f0u; ao[2] = s0 & 0x00f000f0u; ao[3] = s1 & 0x00f000f0u;
                const uint2 be = *(const uint2 *)(xb + i * 8);  // the zero block is as long as a pair's 128 bytes
                const uint2 bo = *(const uint2 *)(xb + 64 + i * 8);
                if (i == 0) {
                    mma16816_first(ce, ae, be.x, be.y);
                    mma16816_first(co, ao, bo.x, bo.y);
                } else {
                    mma16816(ce, ae, be.x, be.y);
                    mma16816(co, ao, bo.x, bo.y);
                }
            }
            const float2 gs = *(const float2 *)(gsum + sb_abs * 8 + t * 2);
            float acc[2];  // rows g, g+8
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const RowScales r = row_scales(cur.hdr[h], t);
                float a = r.ds_e * (ce[2 * h] + ce[2 * h + 1]);
                a = fmaf(r.ds_o, co[2 * h] + co[2 * h + 1], a);
                a = fmaf(-r.dm_e, gs.x, a);
                a = fmaf(-r.dm_o, gs.y, a);
                // the four lanes of a quad hold the four group pairs of the superblock
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                acc[h] = a;
            }
            if (t == 0) {
                slots[j * 16 + g] = acc[0];
                slots[j * 16 + g + 8] = acc[1];
            }
        };
        // two task buffers in turn: while one is computed the other's loads are in flight
        TaskData bufa, bufb;
        if (cu < round_end) load_task(p, ctile, cks * p.ksl + csb, lane, bufa);
        while (cu < round_end) {
            uint32_t nu = cu, nks_ = cks, ntile = ctile, nsb = csb + WARPS;
            normalize(nu, nks_, ntile, nsb);
            if (nu < round_end) load_task(p, ntile, nks_ * p.ksl + nsb, lane, bufb);
            compute(bufa, cks * p.ksl + csb, cj);
            cu = nu; cks = nks_; ctile = ntile; csb = nsb; cj += WARPS;
            if (cu >= round_end) break;
            nsb = csb + WARPS;
            normalize(nu, nks_, ntile, nsb);
            if (nu < round_end) load_task(p, ntile, nks_ * p.ksl + nsb, lane, bufa);
            compute(bufb, cks * p.ksl + csb, cj);
            cu = nu; cks = nks_; ctile = ntile; csb = nsb; cj += WARPS;
        }
        __syncthreads();
        // ---- add each unit's slots in superblock order; lanes 0..15 take one unit's rows, lanes 16..31 the next unit's ----
        {
            const uint32_t half = lane >> 4, r = lane & 15;
            // task index of a unit within the round: prefix over the round's units (slices change rarely: walk)
            for (uint32_t pair0 = round_begin + 2 * warp; pair0 < round_end; pair0 += 2 * WARPS) {
                const uint32_t u = pair0 + half;
                const bool live = u < round_end;
                float sum = 0.0f;
                uint32_t ks = 0, tile = 0, seg = 0, row0 = 0;
                if (live) {
                    ks = u / p.total_tiles;
                    tile = u - ks * p.total_tiles;
                    // first task of unit u in the round
                    uint32_t j0 = 0;
                    {
                        const uint32_t ks0 = round_begin / p.total_tiles;
                        if (ks == ks0) j0 = (u - round_begin) * slice_sbs(p, ks0);
                        else {
                            uint32_t uu = round_begin;
                            for (uint32_t k = ks0; k < ks; ++k) {
                                const uint32_t stop = (k + 1) * p.total_tiles;
                                j0 += (stop - uu) * slice_sbs(p, k);
                                uu = stop;
                            }
                            j0 += (u - uu) * slice_sbs(p, ks);
                        }
                    }
                    const uint32_t n = slice_sbs(p, ks);
                    for (uint32_t sb = 0; sb < n; ++sb) sum += slots[(j0 + sb) * 16 + r];
                    sum *= inv_scale;
                    tile_rows(p, tile, seg, row0);
                }
                const bool pair = p.mode != ACT_NONE;
                if (p.nks == 1) {
                    if (pair) {
                        const float up = __shfl_down_sync(0xffffffffu, sum, 16);
                        if (live && half == 0 && row0 + r < p.rows[0]) {
                            const float a = p.mode == ACT_SILU ? silu_f32(sum) : gelu_f32(sum);
                            p.out[0][row0 + r] = a * up;
                        }
                    } else if (live && row0 + r < p.rows[seg]) {
                        p.out[seg][row0 + r] = sum;
                    }
                } else {
                    // partial sums, then the last block to arrive for this output tile adds them in slice order
                    if (live) p.partials[((size_t)ks * p.total_tiles + tile) * 16 + r] = sum;
                    __threadfence();
                    __syncwarp();
                    const uint32_t ctr = pair ? (tile >> 1) : tile;
                    const uint32_t target = pair ? 2 * p.nks : p.nks;
                    uint32_t arrived = 0;
                    if (live && r == 0) arrived = atomicAdd(p.counters + ctr, 1u);
                    arrived = __shfl_sync(0xffffffffu, arrived, lane & 16);
                    // in pair mode both halves arrive for the same counter: the later of the two sees the larger count
                    const uint32_t other = __shfl_xor_sync(0xffffffffu, arrived, 16);
                    bool last = live && arrived == target - 1;
                    if (pair) last = (live && (arrived == target - 1 || other == target - 1));
                    if (last) {
                        __threadfence();
                        if (pair) {
                            // lanes 0..15: row r of the tile pair
                            if (half == 0) {
                                const uint32_t gate_tile = tile & ~1u;
                                float gate = 0.0f, up = 0.0f;
                                for (uint32_t k = 0; k < p.nks; ++k) {
                                    gate += __ldcg(p.partials + ((size_t)k * p.total_tiles + gate_tile) * 16 + r);
                                    up += __ldcg(p.partials + ((size_t)k * p.total_tiles + gate_tile + 1) * 16 + r);
                                }
                                if (row0 + r < p.rows[0]) {
                                    const float a = p.mode == ACT_SILU ? silu_f32(gate) : gelu_f32(gate);
                                    p.out[0][row0 + r] = a * up;
                                }
                            }
                        } else {
                            float total = 0.0f;
                            for (uint32_t k = 0; k < p.nks; ++k) total += __ldcg(p.partials + ((size_t)k * p.total_tiles + tile) * 16 + r);
                            if (row0 + r < p.rows[seg]) p.out[seg][row0 + r] = total;
                        }
                        if (r == 0 && (!pair || half == 0)) p.counters[ctr] = 0;  // leave the scratch as it was found
                    }
                }
            }
        }
        __syncthreads();
        round_begin = round_end;
    }
}

static size_t smem_bytes(uint32_t K) { return (size_t)K * 4 + 128 + (size_t)K / 32 * 4 + ROUND_TASKS * 64 + 256; }

}  // namespace dec

bool q4k_decode_configure() {
    return cudaFuncSetAttribute(dec::q4k_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess;
}

static bool fill(const FastJob &job, dec::Params &p) {
    if (job.enc != Q4_K || job.tokens != 1 || job.count < 1 || job.count > 4) return false;
    if (job.columns == 0 || job.columns % 256 != 0) return false;
    if (dec::smem_bytes(job.columns) > 200 * 1024) return false;
    if ((uintptr_t)job.in % 16 != 0) return false;
    if (job.mode != ACT_NONE && (job.count != 2 || job.seg[0].rows != job.seg[1].rows)) return false;
    p = dec::Params{};
    p.count = job.count;
    p.mode = job.mode;
    p.ksb = job.columns / 256;
    p.in = job.in;
    uint32_t tiles = 0;
    uint64_t rows_total = 0;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows == 0 || (uintptr_t)g.w % 16 != 0 || g.stride % 16 != 0 || (uintptr_t)g.out % 4 != 0) return false;
        p.w[s] = g.w;
        p.stride[s] = g.stride;
        p.out[s] = g.out;
        p.rows[s] = g.rows;
        p.tile_begin[s] = tiles;
        tiles += (g.rows + 15) / 16;
        rows_total += g.rows;
    }
    for (uint32_t s = job.count; s < 5; ++s) p.tile_begin[s] = tiles;
    p.total_tiles = tiles;  // pair mode: gate tile i and up tile i are tiles 2i and 2i+1
    // Slices: one if that fills the machine evenly, else the count that wastes least (whole rounds
    // of units per block against the partial-sum traffic and the fences of a split).
    double best = -1.0;
    const double weight_bytes = (double)p.ksb * 144.0 * rows_total;
    for (uint32_t nks = 1; nks <= p.ksb && nks <= 16; ++nks) {
        const uint32_t ksl = (p.ksb + nks - 1) / nks;
        const uint32_t slices = (p.ksb + ksl - 1) / ksl;
        const double units = (double)slices * tiles;
        const double blocks = units < job.sm_count ? units : job.sm_count;
        const double rounds = (double)(uint64_t)((units + blocks - 1) / blocks);
        double eff = units / (rounds * blocks);
        if (slices > 1) eff /= 1.02 + 2.0 * slices * tiles * 64.0 / weight_bytes;
        if (eff > best + 1e-9) { best = eff; p.ksl = ksl; p.nks = slices; }
    }
    p.partials = job.partials;
    p.counters = job.counters;
    if (p.nks > 1) {
        if ((size_t)p.nks * tiles * 16 > job.partials_floats) return false;
        if (tiles > job.counters_len) return false;
    }
    return true;
}

bool q4k_decode_supported(const FastJob &job) {
    dec::Params p;
    return fill(job, p);
}

int launch_q4k_decode(cudaStream_t s, const FastJob &job) {
    dec::Params p;
    if (!fill(job, p)) return 0;
    const uint32_t units = p.nks * p.total_tiles;
    const uint32_t grid = units < (uint32_t)job.sm_count ? units : (uint32_t)job.sm_count;
    dec::q4k_decode_kernel<false><<<grid, dec::THREADS, dec::smem_bytes(job.columns), s>>>(p);
    return 1;
}

}  // namespace nu
