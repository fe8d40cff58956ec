// Q4_K decode GEMV (one activation row) for sm_100a: the kernel behind
// Backend.matvec and single-row matvecSegments on Q4_K weights
// (inference/src/backends/metal/ops/matvec.zig:85-116, 268-343; the reference's
// kernel for this is nu_matvec_q4_k, kernels/matvec.metal:161-209).
//
// The HBM stream is the only large traffic: every weight byte is read once.
// A task is 16 weight rows by one superblock (2304 bytes); one TMA tensor copy
// (cp.async.bulk.tensor.2d + mbarrier) brings it to shared memory, each warp
// keeps its own ring of stages filled a few tasks ahead, and 16 warps per SM
// keep about 100 KB of copies in flight. The lanes then read their 16-byte
// pieces with 128-bit shared loads (a quad of lanes reads the 128 contiguous
// quant bytes of a superblock row).
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
// SM) in contiguous, slice-major ranges of equal task count. A block's 16 warps
// are 4 unit slots x 4 K parts: in each step four units are in work, warp
// (slot, part) takes superblocks part, part+4, ... of its unit, keeps the sums
// in registers and leaves 16 row sums in a shared-memory slot. After a
// block-wide barrier the four parts of a unit are added in part order. With
// several slices those sums go to a global scratch array and the last block to
// arrive for a row tile adds them in slice order. No sum depends on timing.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <cstring>

#include "kernels.hpp"
#include "nu_device.cuh"

namespace nu {
namespace dec {

#ifndef NU_DEC_WARPS
#define NU_DEC_WARPS 16
#endif
constexpr int WARPS = NU_DEC_WARPS;
constexpr int THREADS = WARPS * 32;
constexpr int SLOTS = WARPS / 4;   // units in work at once
constexpr int PARTS = 4;           // warps sharing a unit's superblocks
constexpr int TASK_BYTES = 16 * 144;
constexpr int PAIR_PITCH = 136;    // bytes per 64 staged activations (128 of halves + 8 of bank skew)
constexpr int ROUND_STEPS = 8;     // steps between two reductions: 32 units, 8 KiB of slots
constexpr uint32_t SPIN_LIMIT = 1u << 22;

struct Params {
    CUtensorMap map[4];  // per segment: uint8 [rows][row bytes], box 16 rows x 144 bytes
    float *out[4];
    uint32_t rows[4];
    uint32_t tile_begin[5];  // first 16-row tile of each segment in the tile list
    uint32_t count, mode;
    uint32_t ksb, ksl, nks;  // superblocks per row, per slice; slices
    uint32_t total_tiles;    // tiles per slice (pair mode: gate and up tiles interleaved)
    const float *in;
    float *partials;         // [slice][tile][16]
    uint32_t *counters;      // per output tile (pair mode: per gate/up tile pair)
    uint32_t *status;        // set to 1 if a bounded wait ran out
};

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

// First unit whose tasks start at or after `target` tasks into the slice-major unit list.
__device__ __forceinline__ uint32_t unit_at(const Params &p, unsigned long long target) {
    const unsigned long long full = (unsigned long long)p.total_tiles * p.ksl;  // tasks of a full slice
    uint32_t ks = (uint32_t)(target / full);
    if (ks >= p.nks) ks = p.nks - 1;
    const unsigned long long rem = target - (unsigned long long)ks * full;
    const uint32_t n = slice_sbs(p, ks);
    uint32_t tile = (uint32_t)((rem + n - 1) / n);
    if (tile > p.total_tiles) tile = p.total_tiles;
    return ks * p.total_tiles + tile;
}

__device__ __forceinline__ uint32_t word(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

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

// A warp's walk over its tasks: units u_begin + slot, + 4, ... and in each the superblocks part, part + 4, ...
struct Walk {
    uint32_t u;        // unit
    uint32_t sb;       // superblock within the unit's slice
    uint32_t n;        // superblocks of the unit's slice
    uint32_t x0;       // byte offset in the row of the slice's first superblock
    uint32_t seg, row0;
};
__device__ __forceinline__ void walk_enter(const Params &p, Walk &w, uint32_t u_end, uint32_t part) {
    // settle on the next unit (at or after w.u) that has a superblock for this part
    while (w.u < u_end) {
        const uint32_t ks = w.u / p.total_tiles;
        w.n = slice_sbs(p, ks);
        if (part < w.n) {
            w.sb = part;
            w.x0 = ks * p.ksl * 144;
            tile_rows(p, w.u - ks * p.total_tiles, w.seg, w.row0);
            return;
        }
        w.u += SLOTS;
    }
}
__device__ __forceinline__ void walk_next(const Params &p, Walk &w, uint32_t u_end, uint32_t part) {
    w.sb += PARTS;
    if (w.sb >= w.n) {
        w.u += SLOTS;
        walk_enter(p, w, u_end, part);
    }
}

template <int STAGES>
__global__ void __launch_bounds__(THREADS, 1) q4k_decode_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t K = p.ksb * 256;
    // [task stages][hi pieces][lo pieces][128 B of zeros][group sums K/32 floats][slots][flags, scratch][barriers]
    // A piece array holds K halves, the 128 bytes of each group pair (64 columns) padded to PAIR_PITCH = 136:
    // the four quad lanes then read four different pairs of banks, and the lo array starts 32 bytes
    // further round the banks than the hi array, so the eight loading lanes of a warp never collide.
    uint8_t *stages = smem;
    uint8_t *xhi = stages + WARPS * STAGES * TASK_BYTES;
    const uint32_t piece_bytes = (K / 64) * PAIR_PITCH;  // a multiple of 128 when K is a multiple of 1024; see lo_skew
    const uint32_t lo_skew = (128u - piece_bytes % 128u) % 128u + 32u;
    uint8_t *xlo = xhi + piece_bytes + lo_skew;
    uint8_t *zero = xlo + piece_bytes + (128u - (piece_bytes + lo_skew + piece_bytes) % 128u) % 128u;
    float *gsum = (float *)(zero + 128);
    float *slots = gsum + K / 32;
    uint32_t *last_flag = (uint32_t *)(slots + ROUND_STEPS * SLOTS * PARTS * 16);  // one per unit of the round
    float *red = (float *)(last_flag + ROUND_STEPS * SLOTS);
    uint64_t *bars = (uint64_t *)(red + 32);
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t slot = warp >> 2, part = warp & 3;
    static_assert(WARPS % 4 == 0 && WARPS <= 32, "warps are unit slots x four K parts");
    const uint8_t *my_stage = stages + warp * STAGES * TASK_BYTES;
    const uint32_t stage0 = smem_u32(my_stage), bar0 = smem_u32(bars + warp * STAGES);

#ifdef NU_DEC_TRACE
    unsigned long long t_start; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
    __shared__ unsigned long long trace_ns[8];
#define NU_TRACE(i) do { if (tid == 0) { unsigned long long tt; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tt)); trace_ns[(i)] = tt - t_start; } } while (0)
#else
#define NU_TRACE(i)
#endif
    if (tid == 0) {
        for (int i = 0; i < WARPS * STAGES; ++i) mbar_init(smem_u32(bars + i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // ---- this block's units: contiguous, equal task count; pair mode keeps a gate tile with its up tile ----
    const unsigned long long total_tasks = (unsigned long long)p.total_tiles * p.ksb;
    uint32_t u_begin = unit_at(p, total_tasks * blockIdx.x / gridDim.x);
    uint32_t u_end = blockIdx.x + 1 == gridDim.x ? p.nks * p.total_tiles : unit_at(p, total_tasks * (blockIdx.x + 1) / gridDim.x);
    if (p.mode != ACT_NONE) { u_begin &= ~1u; u_end &= ~1u; }
    const uint64_t policy = evict_first_policy();

    // ---- start the weight stream before anything else ----
    Walk prod;
    prod.u = u_begin + slot;
    walk_enter(p, prod, u_end, part);
    Walk cons = prod;
    uint32_t issued = 0, consumed = 0;
    auto issue = [&]() {
        if (lane == 0) {
            const uint32_t st = issued % STAGES;
            mbar_expect_tx(bar0 + st * 8, TASK_BYTES);
            tma_load_2d(stage0 + st * TASK_BYTES, &p.map[prod.seg], prod.x0 + prod.sb * 144, prod.row0, bar0 + st * 8, policy);
        }
        ++issued;
        walk_next(p, prod, u_end, part);
    };
    for (int i = 0; i < STAGES - 1; ++i)
        if (prod.u < u_end) issue();

    // ---- stage the activation row: scale, split into fp16 pieces, group sums ----
    // The row is read from global memory once and kept in registers between the two passes.
    constexpr int XV = (20480 / 4 + THREADS - 1) / THREADS;  // float4 per thread: rows of up to 20480 columns
    float4 xv[XV];
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < XV; ++j) {
        const uint32_t i = tid + j * THREADS;
        xv[j] = i < K / 4 ? ((const float4 *)p.in)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(xv[j].x), fabsf(xv[j].y)), fmaxf(fabsf(xv[j].z), fabsf(xv[j].w))));
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
#pragma unroll
    for (int j = 0; j < XV; ++j) {
        const uint32_t i = tid + j * THREADS;
        if (i < K / 4) {  // uniform per warp: K / 4 is a multiple of 32
            const float x0 = xv[j].x * scale, x1 = xv[j].y * scale, x2 = xv[j].z * scale, x3 = xv[j].w * scale;
            const __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1), h2 = __float2half_rn(x2), h3 = __float2half_rn(x3);
            const __half l0 = __float2half_rn(x0 - __half2float(h0)), l1 = __float2half_rn(x1 - __half2float(h1));
            const __half l2 = __float2half_rn(x2 - __half2float(h2)), l3 = __float2half_rn(x3 - __half2float(h3));
            // k order of the A operand built below: columns +0, +2 in the first register, +1, +3 in the second
            uint2 hi, lo;
            hi.x = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h2) << 16);
            hi.y = (uint32_t)__half_as_ushort(h1) | ((uint32_t)__half_as_ushort(h3) << 16);
            lo.x = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l2) << 16);
            lo.y = (uint32_t)__half_as_ushort(l1) | ((uint32_t)__half_as_ushort(l3) << 16);
            const uint32_t off = (i >> 4) * PAIR_PITCH + (i & 15u) * 8;  // 16 groups of 4 columns per pair
            *(uint2 *)(xhi + off) = hi;
            *(uint2 *)(xlo + off) = lo;
            // 32-column group sum: eight consecutive threads hold a group
            float sg = (x0 + x1) + (x2 + x3);
            sg += __shfl_xor_sync(0xffffffffu, sg, 1);
            sg += __shfl_xor_sync(0xffffffffu, sg, 2);
            sg += __shfl_xor_sync(0xffffffffu, sg, 4);
            if ((lane & 7) == 0) gsum[i >> 3] = sg;
        }
    }
    __syncthreads();

    // Lanes whose B column is not theirs (column n = lane >> 2 belongs to quad lane n >> 1) read zeros.
    const bool mine = (g >> 1) == t;
    const uint8_t *piece = (g & 1u) ? xlo : xhi;
    bool failed = false;

    for (uint32_t round_begin = u_begin; round_begin < u_end && !failed; round_begin += ROUND_STEPS * SLOTS) {
        const uint32_t round_end = min(u_end, round_begin + ROUND_STEPS * SLOTS);
        // ---- this warp's units of the round: round_begin + slot, + 4, ... ----
        while (cons.u < round_end && !failed) {
            const uint32_t unit = cons.u;
            float acc[2] = {0.0f, 0.0f};  // rows g, g+8: this lane's group pair, summed over the warp's superblocks
            while (cons.u == unit) {
                if (prod.u < u_end) issue();  // keep STAGES - 1 tasks in flight
                const uint32_t st = consumed % STAGES;
                if (!mbar_wait(bar0 + st * 8, (consumed / STAGES) & 1u)) { failed = true; break; }
                const uint8_t *task = my_stage + st * TASK_BYTES;
                const uint32_t sb_abs = cons.x0 / 144 + cons.sb;
                uint4 hdr[2], q0[2], q1[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint8_t *row = task + (g + 8 * h) * 144;
                    hdr[h] = *(const uint4 *)row;
                    q0[h] = *(const uint4 *)(row + 16 + t * 32);
                    q1[h] = *(const uint4 *)(row + 32 + t * 32);
                }
                const uint8_t *xb = mine ? piece + (sb_abs * 4 + t) * PAIR_PITCH : zero;  // the 64 columns of this pair: 128 B of halves
                float ce[4], co[4];  // even group / odd group: (hi, lo) sums of row g, (hi, lo) of row g+8
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t w0 = i < 4 ? word(q0[0], i) : word(q1[0], i - 4);
                    const uint32_t w1 = i < 4 ? word(q0[1], i) : word(q1[1], i - 4);
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
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const RowScales r = row_scales(hdr[h], t);
                    float a = fmaf(r.ds_e, ce[2 * h] + ce[2 * h + 1], acc[h]);
                    a = fmaf(r.ds_o, co[2 * h] + co[2 * h + 1], a);
                    a = fmaf(-r.dm_e, gs.x, a);
                    acc[h] = fmaf(-r.dm_o, gs.y, a);
                }
                __syncwarp();  // all lanes are done reading this stage before it is refilled
                ++consumed;
                walk_next(p, cons, u_end, part);
            }
            if (failed) break;
            // the four lanes of a quad hold the four group pairs of the superblock
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], 1);
                acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], 2);
            }
            if (t == 0) {
                float *dst = slots + ((unit - round_begin) * PARTS + part) * 16;
                dst[g] = acc[0];
                dst[g + 8] = acc[1];
            }
        }
        NU_TRACE(1);
        __syncthreads();
        NU_TRACE(2);
        // ---- add each unit's parts in part order: one thread per (unit, row); pair mode: per (gate unit, row) ----
        const bool pair = p.mode != ACT_NONE;
        for (uint32_t idx = tid; idx < (round_end - round_begin) * 16; idx += THREADS) {
            const uint32_t ul = idx >> 4, r = idx & 15, u = round_begin + ul;
            if (pair && (ul & 1u)) continue;
            const uint32_t ks = u / p.total_tiles, tile = u - ks * p.total_tiles;
            const uint32_t parts = min((uint32_t)PARTS, slice_sbs(p, ks));
            float sum = 0.0f, up = 0.0f;
            for (uint32_t k = 0; k < parts; ++k) sum += slots[(ul * PARTS + k) * 16 + r];
            sum *= inv_scale;
            if (pair) {
                for (uint32_t k = 0; k < parts; ++k) up += slots[((ul + 1) * PARTS + k) * 16 + r];
                up *= inv_scale;
            }
            uint32_t seg, row0;
            tile_rows(p, tile, seg, row0);
            if (p.nks == 1) {
                if (row0 + r < p.rows[seg]) {
                    if (pair) sum = (p.mode == ACT_SILU ? silu_f32(sum) : gelu_f32(sum)) * up;
                    p.out[seg][row0 + r] = sum;
                }
            } else {
                p.partials[((size_t)ks * p.total_tiles + tile) * 16 + r] = sum;
                if (pair) p.partials[((size_t)ks * p.total_tiles + tile + 1) * 16 + r] = up;
                __threadfence();
            }
        }
        if (p.nks > 1) {
            // the last block to arrive for an output tile adds its slices in order
            __syncthreads();
            for (uint32_t ul = tid; ul < round_end - round_begin; ul += THREADS) {
                uint32_t flag = 0;
                if (!(pair && (ul & 1u))) {
                    const uint32_t u = round_begin + ul, tile = u % p.total_tiles;
                    const uint32_t arrived = atomicAdd(p.counters + (pair ? tile >> 1 : tile), 1u);
                    flag = arrived == p.nks - 1;
                }
                last_flag[ul] = flag;
            }
            __syncthreads();
            for (uint32_t idx = tid; idx < (round_end - round_begin) * 16; idx += THREADS) {
                const uint32_t ul = idx >> 4, r = idx & 15;
                if (!last_flag[ul]) continue;
                __threadfence();
                const uint32_t tile = (round_begin + ul) % p.total_tiles;
                float sum = 0.0f, up = 0.0f;
                for (uint32_t k = 0; k < p.nks; ++k) sum += __ldcg(p.partials + ((size_t)k * p.total_tiles + tile) * 16 + r);
                if (pair)
                    for (uint32_t k = 0; k < p.nks; ++k) up += __ldcg(p.partials + ((size_t)k * p.total_tiles + tile + 1) * 16 + r);
                uint32_t seg, row0;
                tile_rows(p, tile, seg, row0);
                if (row0 + r < p.rows[seg]) {
                    if (pair) sum = (p.mode == ACT_SILU ? silu_f32(sum) : gelu_f32(sum)) * up;
                    p.out[seg][row0 + r] = sum;
                }
                if (r == 0) p.counters[pair ? tile >> 1 : tile] = 0;  // leave the scratch as it was found
            }
        }
        __syncthreads();  // slots and flags are free for the next round
        NU_TRACE(3);
    }
#ifdef NU_DEC_TRACE
    if (tid == 0 && (blockIdx.x == 0 || blockIdx.x == 77 || blockIdx.x == 147))
        printf("block %u: staged %llu ns, tasks done %llu, barrier %llu, reduced %llu; units %u..%u\n", blockIdx.x, trace_ns[0], trace_ns[1], trace_ns[2], trace_ns[3], u_begin, u_end);
#endif
    if (failed) {
        if (lane == 0) atomicExch(p.status, 1u);
        // let this warp's copies still in flight land before the block's shared memory is released
        for (; consumed < issued; ++consumed) mbar_wait(bar0 + (consumed % STAGES) * 8, (consumed / STAGES) & 1u);
    }
}

static size_t smem_bytes(uint32_t K, int stages) {
    return (size_t)WARPS * stages * TASK_BYTES + (size_t)(K / 64) * PAIR_PITCH * 2 + 512 + (size_t)K / 32 * 4 + ROUND_STEPS * SLOTS * PARTS * 64 +
           ROUND_STEPS * SLOTS * 4 + 128 + WARPS * stages * 8 + 128;
}

}  // namespace dec

#ifdef NU_DEC_TRACE
constexpr size_t kDecodeSmemMax = 226 * 1024;
#else
constexpr size_t kDecodeSmemMax = 227 * 1024;
#endif

constexpr int kDecodeMaxColumns = 20480;  // the staging pass keeps the activation row in registers

template <int STAGES>
static bool configure_stages() {
    return cudaFuncSetAttribute(dec::q4k_decode_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDecodeSmemMax) == cudaSuccess;
}
bool q4k_decode_configure() { return configure_stages<3>() && configure_stages<4>() && configure_stages<5>() && configure_stages<6>(); }

// Deepest ring of task stages that fits beside the staged activations: the copies in flight hide HBM latency.
static int pick_stages(uint32_t columns) {
    for (int st = 6; st >= 3; --st)
        if (dec::smem_bytes(columns, st) <= kDecodeSmemMax) return st;
    return 0;
}

bool encode_weight_map(CUtensorMap *map, const uint8_t *base, uint64_t row_bytes, uint64_t rows, uint64_t stride, uint32_t box_bytes, uint32_t box_rows);

static bool fill(const FastJob &job, dec::Params &p, bool maps) {
    if (job.enc != Q4_K || job.tokens != 1 || job.count < 1 || job.count > 4) return false;
    if (job.columns == 0 || job.columns % 256 != 0) return false;
    if (job.columns > kDecodeMaxColumns || pick_stages(job.columns) == 0) return false;
    if ((uintptr_t)job.in % 16 != 0) return false;
    if (job.mode != ACT_NONE && (job.count != 2 || job.seg[0].rows != job.seg[1].rows)) return false;
    memset(&p, 0, sizeof p);
    p.count = job.count;
    p.mode = job.mode;
    p.ksb = job.columns / 256;
    p.in = job.in;
    uint32_t tiles = 0;
    uint64_t rows_total = 0;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows == 0 || (uintptr_t)g.w % 16 != 0 || g.stride % 16 != 0 || (uintptr_t)g.out % 4 != 0) return false;
        if (maps && !encode_weight_map(&p.map[s], g.w, (uint64_t)p.ksb * 144, g.rows, g.stride, 144, 16)) return false;
        p.out[s] = g.out;
        p.rows[s] = g.rows;
        p.tile_begin[s] = tiles;
        tiles += (g.rows + 15) / 16;
        rows_total += g.rows;
    }
    for (uint32_t s = job.count; s < 5; ++s) p.tile_begin[s] = tiles;
    p.total_tiles = tiles;  // pair mode: gate tile i and up tile i are tiles 2i and 2i+1
    // Slices: one if that fills the machine evenly, else the count that wastes least: whole steps of
    // four units per block, four superblock parts per unit, against the partial sums and fences of a split.
    double best = -1.0;
    const double weight_bytes = (double)p.ksb * 144.0 * rows_total;
    for (uint32_t nks = 1; nks <= p.ksb && nks <= 32; ++nks) {
        const uint32_t ksl = (p.ksb + nks - 1) / nks;
        const uint32_t slices = (p.ksb + ksl - 1) / ksl;
        const double units = (double)slices * tiles;
        const double blocks = units < job.sm_count ? units : job.sm_count;
        const double per_block = units / blocks;
        const double steps = (double)(uint64_t)((per_block + dec::SLOTS - 1) / dec::SLOTS);
        double eff = per_block / (steps * dec::SLOTS);                                   // idle unit slots in the last step
        eff *= (double)ksl / ((double)((ksl + dec::PARTS - 1) / dec::PARTS) * dec::PARTS);  // idle parts
        if (slices > 1) eff /= 1.2 + 2.0 * slices * tiles * 64.0 / weight_bytes;  // partial sums, fences and a second reduction
        if (eff > best + 1e-9) { best = eff; p.ksl = ksl; p.nks = slices; }
    }
    p.partials = job.partials;
    p.counters = job.counters;
    p.status = job.counters + job.counters_len;
    if (p.nks > 1) {
        if ((size_t)p.nks * tiles * 16 > job.partials_floats) return false;
        if (tiles > job.counters_len) return false;
    }
    return true;
}

bool q4k_decode_supported(const FastJob &job) {
    dec::Params p;
    return fill(job, p, false);
}

int launch_q4k_decode(cudaStream_t s, const FastJob &job) {
    dec::Params p;
    if (!fill(job, p, true)) return 0;
    const uint32_t units = p.nks * p.total_tiles;
    const uint32_t grid = units < (uint32_t)job.sm_count ? units : (uint32_t)job.sm_count;
    const int stages = pick_stages(job.columns);
    const size_t bytes = dec::smem_bytes(job.columns, stages);
    switch (stages) {
    case 6: dec::q4k_decode_kernel<6><<<grid, dec::THREADS, bytes, s>>>(p); break;
    case 5: dec::q4k_decode_kernel<5><<<grid, dec::THREADS, bytes, s>>>(p); break;
    case 4: dec::q4k_decode_kernel<4><<<grid, dec::THREADS, bytes, s>>>(p); break;
    default: dec::q4k_decode_kernel<3><<<grid, dec::THREADS, bytes, s>>>(p); break;
    }
    return 1;
}

}  // namespace nu
