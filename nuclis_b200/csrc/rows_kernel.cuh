// Skeleton of the GEMM for 2..8 token rows over block-quantized weights (the speculative-verify
// batch): the work split, the TMA task ring, the staging of the token rows as fp16 pieces in mma B
// order, the sums across K parts and K slices. An encoding supplies a policy class E with the
// geometry of its task, the copy that fetches it, the place of each activation in the staged
// layout, its group sums, and the mma loop over one task. The scheme is described in
// gemv_q4k_rows.cu.
#pragma once
#include "decode_kernel.cuh"

#include "../../include/nuclis_cuda.h"

namespace nu {
namespace rows {

using dec::mbar_expect_tx;
using dec::mbar_init;
using dec::mbar_wait;
using dec::mma16816;
using dec::smem_u32;
using dec::tma_load_2d;

constexpr int WARPS = 16;
constexpr int THREADS = WARPS * 32;
constexpr int SLOTS = 4;
constexpr int PARTS = 4;
constexpr int PITCH = 144;          // bytes per 64 staged activations of one B column (128 + 16 of bank skew)
constexpr int MAX_SLICES = 32;
constexpr int PARTIAL_FLOATS = 128; // per (slice, row tile): 16 rows x 8 columns
constexpr int XV = 10;              // float4 of activations a thread stages: tokens x slice length <= 80 superblocks

struct Params {
    CUtensorMap map[4];
    CUtensorMap map2[4];  // a second plane of the encoding, if it has one
    float *out[4];
    uint32_t out_stride[4];
    uint32_t rows[4];
    uint32_t tile_begin[5];
    uint32_t count, tokens;
    uint32_t ksb, ksl, nks, total_tiles;
    uint32_t blk_first[MAX_SLICES + 1];  // blocks blk_first[s] .. blk_first[s+1]-1 work on slice s
    uint32_t arr_stride;                 // bytes between the staged activations of two B columns
    uint32_t gs_stride;                  // bytes between the staged group sums of two B columns
    const float *in;
    uint32_t in_stride;
    float *partials;
    uint32_t *counters;
    uint32_t *status;
};

__device__ __forceinline__ void mma1688(float c[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));  // no flush to zero: the codes are subnormals
    return d;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ uint32_t word(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

__device__ __forceinline__ void tile_rows(const Params &p, uint32_t tile, uint32_t &seg, uint32_t &row0) {
    seg = 0;
#pragma unroll
    for (int s = 1; s < 4; ++s)
        if ((uint32_t)s < p.count && tile >= p.tile_begin[s]) seg = s;
    row0 = (tile - p.tile_begin[seg]) * 16;
}

// Stores one lane's finished sums of a row tile: rows g, g+8; WIDE: tokens 2t, 2t+1 (val 0..3),
// else token t (val 0 and 2).
template <bool WIDE>
__device__ __forceinline__ void write_tile(const Params &p, uint32_t tile, uint32_t g, uint32_t t, const float val[4]) {
    uint32_t seg, row0;
    tile_rows(p, tile, seg, row0);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t row = row0 + g + 8 * h;
        if (row >= p.rows[seg]) continue;
#pragma unroll
        for (int c = 0; c < (WIDE ? 2 : 1); ++c) {
            const uint32_t tok = WIDE ? 2 * t + c : t;
            if (tok < p.tokens) p.out[seg][(size_t)tok * p.out_stride[seg] + row] = val[2 * h + c];
        }
    }
}

template <bool WIDE>
__host__ __device__ constexpr int columns() { return WIDE ? 16 : 8; }

// Shared memory: [task stages][staged activations: columns x arr_stride][group sums: columns x gs_stride]
// [per-token 1/scale: 8 floats][per-token max bits: 8 words][part sums: SLOTS x 2 x 3 x 512 B][barriers]
template <class E, bool WIDE>
static size_t smem_bytes(uint32_t arr_stride, uint32_t gs_stride, int stages) {
    // a swizzled TMA box needs the ring on a 1024-byte boundary: room to round the base up
    return (E::SWIZZLED ? 1024 : 0) + (size_t)WARPS * stages * (E::TASK_BYTES + E::AUX_BYTES) + (size_t)columns<WIDE>() * (arr_stride + gs_stride) + 64 + SLOTS * 2 * 3 * 512 + WARPS * stages * 8 + 128;
}

template <class E, bool WIDE, int STAGES>
__global__ void __launch_bounds__(THREADS, 1) rows_kernel(const __grid_constant__ Params p) {
    constexpr int NCOL = columns<WIDE>();
    constexpr int TASK_BYTES = E::TASK_BYTES;
    constexpr int AUX_BYTES = E::AUX_BYTES;  // a second, small part of a task kept apart so that TASK_BYTES can stay a multiple of 1024
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *smem = E::SWIZZLED ? (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023) : smem_raw;
    uint8_t *stages = smem;
    uint8_t *aux = stages + WARPS * STAGES * TASK_BYTES;
    uint8_t *xarr = aux + WARPS * STAGES * AUX_BYTES;
    uint8_t *gsarr = xarr + NCOL * p.arr_stride;
    float *inv = (float *)(gsarr + NCOL * p.gs_stride);
    uint32_t *maxbits = (uint32_t *)(inv + 8);
    float *parts = (float *)(maxbits + 8);
    uint64_t *bars = (uint64_t *)(parts + SLOTS * 2 * 3 * 128);
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t slot = warp >> 2, part = warp & 3;
    const uint8_t *my_stage = stages + warp * STAGES * TASK_BYTES;
    const uint8_t *my_aux = aux + warp * STAGES * AUX_BYTES;
    const uint32_t aux0 = smem_u32(my_aux);
    const uint32_t stage0 = smem_u32(my_stage), bar0 = smem_u32(bars + warp * STAGES);

    // See decode_kernel.cuh: dependents may start now; this kernel reads its activations and writes
    // global memory only after the wait below, its weights (constants) before it.
    asm volatile("griddepcontrol.launch_dependents;");
    // every warp owns its ring: it initialises its own barriers and nobody else touches them
    if (lane == 0) {
        for (int i = 0; i < STAGES; ++i) mbar_init(bar0 + i * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 8) maxbits[tid] = 0;
    __syncwarp();

    // ---- this block's slice and row tiles ----
    uint32_t ks = 0;
    while (ks + 1 < p.nks && blockIdx.x >= p.blk_first[ks + 1]) ++ks;
    const uint32_t sb0 = ks * p.ksl, n = min(p.ksl, p.ksb - sb0);
    const uint32_t nblk = p.blk_first[ks + 1] - p.blk_first[ks], jblk = blockIdx.x - p.blk_first[ks];
    // the first blocks of a slice take the tiles that do not divide evenly (see decode_kernel.cuh)
    const uint32_t per_blk = p.total_tiles / nblk, extra = p.total_tiles - per_blk * nblk;
    const uint32_t tile_lo = jblk * per_blk + min(jblk, extra);
    const uint32_t tile_hi = tile_lo + per_blk + (jblk < extra ? 1u : 0u);
    const uint32_t np = min((uint32_t)PARTS, n);                 // warps that share a unit
    const uint32_t m = part < n ? (n - part + PARTS - 1) / PARTS : 0;  // this warp's tasks per unit
    const uint32_t first_tile = tile_lo + slot;
    const uint32_t units = first_tile < tile_hi ? (tile_hi - first_tile + SLOTS - 1) / SLOTS : 0;
    const uint32_t total = units * m;
    const uint64_t policy = dec::evict_first_policy();

    // ---- the weight stream ----
    uint32_t issued = 0, p_stage = 0, p_tile = first_tile, p_j = 0, p_seg = 0, p_row0 = 0;
    if (total) tile_rows(p, p_tile, p_seg, p_row0);
    auto issue = [&]() {
        if (lane == 0) {
            E::issue(p, p_seg, sb0 + part + PARTS * p_j, p_row0, stage0 + p_stage * TASK_BYTES, aux0 + p_stage * AUX_BYTES, bar0 + p_stage * 8, policy);
        }
        ++issued;
        p_stage = p_stage + 1 == STAGES ? 0 : p_stage + 1;
        if (++p_j == m) {
            p_j = 0;
            p_tile += SLOTS;
            if (issued < total) tile_rows(p, p_tile, p_seg, p_row0);
        }
    };
    for (int i = 0; i < STAGES - 1; ++i)
        if (issued < total) issue();
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the previous kernel has ended; its writes are visible

    // ---- stage the token rows of this slice: per-token scale, fp16 pieces in mma B order, group sums ----
    // Every thread requests all its float4 at once (the window is read from global memory once and kept
    // in registers between the two passes); the flat index runs over [token][float4 of the window].
    const uint32_t row_f4 = n * 64;  // float4 per token row in the window
    const uint32_t all_f4 = p.tokens * row_f4;
    const uint32_t tok0 = tid / row_f4, i0 = tid - tok0 * row_f4;
    float4 xv[XV];
    {
        uint32_t tok = tok0, i = i0;
#pragma unroll
        for (int k = 0; k < XV; ++k) {
            xv[k] = tid + k * THREADS < all_f4 ? *(const float4 *)(p.in + (size_t)tok * p.in_stride + (size_t)sb0 * 256 + i * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            i += THREADS;
            while (i >= row_f4) { i -= row_f4; ++tok; }
        }
    }
    __syncthreads();  // the per-token maxima start at zero (written above by the first eight threads)
    {
        uint32_t tok = tok0, i = i0;
#pragma unroll
        for (int k = 0; k < XV; ++k) {
            if (tid + k * THREADS < all_f4) {  // uniform per warp: the window is a multiple of 64 float4
                float mx = fmaxf(fmaxf(fabsf(xv[k].x), fabsf(xv[k].y)), fmaxf(fabsf(xv[k].z), fabsf(xv[k].w)));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                if ((lane & 7) == 0) atomicMax(maxbits + tok, __float_as_uint(mx));  // non-negative floats order like their bits
            }
            i += THREADS;
            while (i >= row_f4) { i -= row_f4; ++tok; }
        }
    }
    __syncthreads();
    if (tid < 8) {
        // 2^e puts the token's largest |x| in [2^13, 2^14): hi cannot overflow fp16, lo keeps 11 more bits
        const uint32_t e = (maxbits[tid] >> 23) & 0xffu;
        const bool ok = e >= 40u && e < 255u;
        inv[tid] = ok ? __uint_as_float((e - 13u) << 23) : 1.0f;
    }
    {
        uint32_t tok = tok0, i = i0;
#pragma unroll
        for (int k = 0; k < XV; ++k) {
            if (tid + k * THREADS < all_f4) {
                const float4 v = xv[k];
                const uint32_t e = (maxbits[tok] >> 23) & 0xffu;
                const float scale = (e >= 40u && e < 255u) ? __uint_as_float((267u - e) << 23) : 1.0f;
                const float x0 = v.x * scale, x1 = v.y * scale, x2 = v.z * scale, x3 = v.w * scale;
                const __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1), h2 = __float2half_rn(x2), h3 = __float2half_rn(x3);
                const __half l0 = __float2half_rn(x0 - __half2float(h0)), l1 = __float2half_rn(x1 - __half2float(h1));
                const __half l2 = __float2half_rn(x2 - __half2float(h2)), l3 = __float2half_rn(x3 - __half2float(h3));
                // k order of the A operand: columns +0, +2 in the first register, +1, +3 in the second
                uint2 hi, lo;
                hi.x = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h2) << 16);
                hi.y = (uint32_t)__half_as_ushort(h1) | ((uint32_t)__half_as_ushort(h3) << 16);
                lo.x = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l2) << 16);
                lo.y = (uint32_t)__half_as_ushort(l1) | ((uint32_t)__half_as_ushort(l3) << 16);
                const uint32_t col_hi = WIDE ? tok : 2 * tok, col_lo = WIDE ? 8 + tok : 2 * tok + 1;
                const uint32_t off = E::x_offset(i);
                *(uint2 *)(xarr + col_hi * p.arr_stride + off) = hi;
                *(uint2 *)(xarr + col_lo * p.arr_stride + off) = lo;
                E::group_sum(gsarr + col_hi * p.gs_stride, gsarr + col_lo * p.gs_stride, i, (x0 + x1) + (x2 + x3), lane);
            }
            i += THREADS;
            while (i >= row_f4) { i -= row_f4; ++tok; }
        }
    }
    __syncthreads();

    // ---- the task loop ----
    const uint8_t *xlane = xarr + g * p.arr_stride + t * PITCH;  // B column g, pair t of superblock 0 of the window
    const uint8_t *gslane = gsarr + g * p.gs_stride;
    const uint32_t lo_off = 8 * p.arr_stride, gs_lo_off = 8 * p.gs_stride;
    uint32_t c_stage = 0, c_phase = 0, consumed = 0;
    bool failed = false;
    uint32_t unit = 0;
    for (uint32_t tile = first_tile; tile < tile_hi; tile += SLOTS, ++unit) {
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        // After a wait has run out the warp stops computing but still walks its units, so that the
        // warps it shares them with are not left at the barrier below.
        for (uint32_t j = 0; j < m && !failed; ++j) {
            if (issued < total) issue();  // keep STAGES - 1 tasks in flight
            if (!mbar_wait(bar0 + c_stage * 8, c_phase)) { failed = true; break; }
            const uint32_t sbw = part + PARTS * j;  // superblock within the window
            E::template task<WIDE>(my_stage + c_stage * TASK_BYTES, my_aux + c_stage * AUX_BYTES, xlane + sbw * 4 * PITCH, lo_off, gslane + sbw * E::GS_BYTES, gs_lo_off, g, t, o);
            __syncwarp();  // all lanes are done reading this stage before it is refilled
            ++consumed;
            if (++c_stage == STAGES) { c_stage = 0; c_phase ^= 1u; }
        }
        if (part >= np) continue;  // this warp has no superblocks in this slice
        // ---- the parts of the unit meet; part 0 adds them in order ----
        float4 *buf = (float4 *)(parts + ((slot * 2 + (unit & 1u)) * 3) * 128);
        if (part > 0) buf[(part - 1) * 32 + lane] = make_float4(o[0], o[1], o[2], o[3]);
        if (np > 1) named_barrier(1 + slot, 32 * np);
        if (part != 0) continue;
        for (uint32_t k = 1; k < np; ++k) {
            const float4 v = buf[(k - 1) * 32 + lane];
            o[0] += v.x; o[1] += v.y; o[2] += v.z; o[3] += v.w;
        }
        // this lane's outputs: rows g, g+8; WIDE: tokens 2t, 2t+1; else token t (hi + lo columns)
        float val[4];
        if (WIDE) {
            val[0] = o[0] * inv[2 * t]; val[1] = o[1] * inv[2 * t + 1]; val[2] = o[2] * inv[2 * t]; val[3] = o[3] * inv[2 * t + 1];
        } else {
            val[0] = (o[0] + o[1]) * inv[t]; val[1] = 0.0f; val[2] = (o[2] + o[3]) * inv[t]; val[3] = 0.0f;
        }
        if (p.nks > 1) {
            // several slices: leave the partial sums; they are published after the loop with one fence
            *(float4 *)(p.partials + ((size_t)ks * p.total_tiles + tile) * PARTIAL_FLOATS + lane * 4) = make_float4(val[0], val[1], val[2], val[3]);
        } else {
            write_tile<WIDE>(p, tile, g, t, val);
        }
    }
    if (p.nks > 1 && part == 0 && units) {
        // The last block to arrive for a row tile adds the slices in order. Lanes announce 32 tiles
        // at a time (one round trip for all of them), then the warp finishes those it was last for.
        __threadfence();
        __syncwarp();
        for (uint32_t base = 0; base < units; base += 32) {
            const uint32_t mine_u = base + lane;
            uint32_t last = 0;
            if (mine_u < units) last = atomicAdd(p.counters + first_tile + mine_u * SLOTS, 1u) == p.nks - 1;
            uint32_t mask = __ballot_sync(0xffffffffu, last != 0);
            if (mask) __threadfence();
            while (mask) {
                const uint32_t u = base + (uint32_t)__ffs((int)mask) - 1;
                mask &= mask - 1;
                const uint32_t tile = first_tile + u * SLOTS;
                // (four loads in flight at a time; added in slice order)
                float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
                const float *src = p.partials + (size_t)tile * PARTIAL_FLOATS + lane * 4;
                const size_t step = (size_t)p.total_tiles * PARTIAL_FLOATS;
                for (uint32_t k0 = 0; k0 < p.nks; k0 += 4) {
                    float4 v[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) v[k] = k0 + k < p.nks ? __ldcg((const float4 *)(src + (k0 + k) * step)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int k = 0; k < 4; ++k) { s.x += v[k].x; s.y += v[k].y; s.z += v[k].z; s.w += v[k].w; }
                }
                const float val[4] = {s.x, s.y, s.z, s.w};
                write_tile<WIDE>(p, tile, g, t, val);
                if (lane == 0) p.counters[tile] = 0;  // leave the scratch as it was found
            }
        }
    }
    if (failed) {
        if (lane == 0) atomicExch(p.status, 1u);
        // let this warp's copies still in flight land before the block's shared memory is released
        for (; consumed < issued; ++consumed) {
            mbar_wait(bar0 + c_stage * 8, c_phase);
            if (++c_stage == STAGES) { c_stage = 0; c_phase ^= 1u; }
        }
    }
}

constexpr size_t kSmemMax = 227 * 1024;
constexpr int kMaxStages = 5;

struct Plan {
    bool wide;
    int stages;
    uint32_t grid;
};

template <class E, bool WIDE>
static int fit_stages(uint32_t arr_stride, uint32_t gs_stride) {
    for (int st = kMaxStages; st >= 2; --st)
        if (smem_bytes<E, WIDE>(arr_stride, gs_stride, st) <= kSmemMax) return st;
    return 0;
}

// Picks the K slices and the blocks of each slice: every candidate slice length is costed in
// task steps of the slowest block (row tiles over unit slots, superblocks over K parts).
template <class E>
static bool fill_common(const FastJob &job, Params &p, Plan &plan) {
    if (job.tokens < 1 || job.tokens > 8 || job.count < 1 || job.count > 4 || job.mode != ACT_NONE) return false;
    if (job.columns == 0 || job.columns % 256 != 0) return false;
    if ((uintptr_t)job.in % 16 != 0 || job.in_stride % 4 != 0 || job.in_stride > 0xffffffffull) return false;
    memset(&p, 0, sizeof p);
    p.count = job.count;
    p.tokens = job.tokens;
    p.ksb = job.columns / 256;
    p.in = job.in;
    p.in_stride = (uint32_t)job.in_stride;
    uint32_t tiles = 0;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows == 0 || (uintptr_t)g.w % 16 != 0 || (uintptr_t)g.out % 4 != 0 || g.out_stride > 0xffffffffull) return false;
        p.out[s] = g.out;
        p.out_stride[s] = (uint32_t)g.out_stride;
        p.rows[s] = g.rows;
        p.tile_begin[s] = tiles;
        tiles += (g.rows + 15) / 16;
    }
    for (uint32_t s = job.count; s < 5; ++s) p.tile_begin[s] = tiles;
    p.total_tiles = tiles;
    plan.wide = job.tokens > 4;
    const uint32_t sms = (uint32_t)job.sm_count;
    double best = 1e30;
    uint32_t blocks[MAX_SLICES];
    for (uint32_t ksl = 1; ksl <= p.ksb; ++ksl) {
        const uint32_t nks = (p.ksb + ksl - 1) / ksl;
        if (nks > MAX_SLICES || nks > sms) continue;
        if (nks > 1 && ((size_t)nks * tiles * PARTIAL_FLOATS > job.partials_floats || tiles > job.counters_len)) continue;  // the scratch must hold it
        if ((size_t)job.tokens * ksl * 64 > (size_t)XV * THREADS) continue;  // the staging pass keeps the window in registers
        const uint32_t arr = ksl * 4 * PITCH + ((ksl * 4 * PITCH) % 128 == 64 ? 0 : 64);  // columns 64 bytes apart round the banks
        const uint32_t gs = ksl * E::GS_BYTES + (16 + 128 - (ksl * E::GS_BYTES) % 128) % 128;  // columns 16 bytes apart round the banks
        const int st = plan.wide ? fit_stages<E, true>(arr, gs) : fit_stages<E, false>(arr, gs);
        if (st < 2) continue;
        auto cost = [&](uint32_t s, uint32_t b) {
            const uint32_t n = s + 1 == nks ? p.ksb - s * ksl : ksl;
            const uint32_t tiles_blk = (tiles + b - 1) / b;
            return (double)((tiles_blk + SLOTS - 1) / SLOTS) * ((double)((n + PARTS - 1) / PARTS) + 0.35);
        };
        for (uint32_t s = 0; s < nks; ++s) blocks[s] = 1;
        for (uint32_t left = sms - nks; left > 0; --left) {
            uint32_t worst = 0;
            for (uint32_t s = 1; s < nks; ++s)
                if (cost(s, blocks[s]) > cost(worst, blocks[worst])) worst = s;
            if (blocks[worst] >= tiles) break;
            ++blocks[worst];
        }
        double est = 0;
        for (uint32_t s = 0; s < nks; ++s) est = cost(s, blocks[s]) > est ? cost(s, blocks[s]) : est;
        est *= st >= 4 ? 1.0 : st == 3 ? 1.06 : 1.2;            // a shallow ring hides less latency
        est += (nks > 1 ? 3.0 + 0.3 * nks : 0.0) + 0.005 * job.tokens * ksl;  // partial sums and the last arriver's pass; staging of the window
        if (est < best - 1e-9) {
            best = est;
            p.ksl = ksl;
            p.nks = nks;
            p.arr_stride = arr;
            p.gs_stride = gs;
            plan.stages = st;
            uint32_t first = 0;
            for (uint32_t s = 0; s < nks; ++s) { p.blk_first[s] = first; first += blocks[s]; }
            for (uint32_t s = nks; s <= MAX_SLICES; ++s) p.blk_first[s] = first;
            plan.grid = first;
        }
    }
    if (best >= 1e30) return false;
    p.partials = job.partials;
    p.counters = job.counters;
    p.status = job.counters + job.counters_len;
    return true;
}

template <class E, bool WIDE, int STAGES>
static bool configure_one() {
    return cudaFuncSetAttribute(rows_kernel<E, WIDE, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax) == cudaSuccess;
}

template <class E>
static bool configure() {
    return configure_one<E, false, 2>() && configure_one<E, false, 3>() && configure_one<E, false, 4>() && configure_one<E, false, 5>() &&
           configure_one<E, true, 2>() && configure_one<E, true, 3>() && configure_one<E, true, 4>() && configure_one<E, true, 5>();
}

template <class E, bool WIDE>
static void launch_wide(const cudaLaunchConfig_t &cfg, int stages, const Params &p) {
    switch (stages) {
    case 5: cudaLaunchKernelEx(&cfg, rows_kernel<E, WIDE, 5>, p); break;
    case 4: cudaLaunchKernelEx(&cfg, rows_kernel<E, WIDE, 4>, p); break;
    case 3: cudaLaunchKernelEx(&cfg, rows_kernel<E, WIDE, 3>, p); break;
    default: cudaLaunchKernelEx(&cfg, rows_kernel<E, WIDE, 2>, p); break;
    }
}

template <class E>
static int launch(cudaStream_t s, const FastJob &job, const Params &p, const Plan &plan) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = plan.wide ? smem_bytes<E, true>(p.arr_stride, p.gs_stride, plan.stages) : smem_bytes<E, false>(p.arr_stride, p.gs_stride, plan.stages);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = job.serial ? 0 : 1;
    if (plan.wide) launch_wide<E, true>(cfg, plan.stages, p);
    else launch_wide<E, false>(cfg, plan.stages, p);
    return 1;
}

}  // namespace rows
}  // namespace nu
