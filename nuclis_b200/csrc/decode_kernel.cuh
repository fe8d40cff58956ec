// Decode GEMV skeleton (one activation row) shared by the block encodings: the
// persistent-block work split, the TMA task ring, the staging of the activation
// row as fp16 hi/lo pieces in mma B order, the in-block and cross-block sums.
// An encoding supplies a policy class E with the geometry of its task, the copy
// that fetches it, the place of each activation in the staged layout, and the
// mma loop over one task. See gemv_q4k_decode.cu for the description of the scheme.
#pragma once
#include <cstdlib>
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
#ifndef NU_DEC_PRE
#define NU_DEC_PRE 1
#endif
constexpr int WARPS = NU_DEC_WARPS;
constexpr int THREADS = WARPS * 32;
constexpr int SLOTS = WARPS / 4;   // units in work at once
constexpr int PARTS = 4;           // warps sharing a unit's superblocks
constexpr int PAIR_PITCH = 136;    // bytes per 64 staged activations (128 of halves + 8 of bank skew)
constexpr int ROUND_STEPS = 8;     // steps between two reductions: 32 units, 8 KiB of slots
constexpr uint32_t SPIN_LIMIT = 1u << 22;

struct Params {
    CUtensorMap map[4];   // per segment: uint8 [rows][row bytes], box 16 rows x one superblock
    CUtensorMap map2[4];  // per segment: a second plane of the encoding, if it has one
    float *out[4];
    uint32_t rows[4];
    uint32_t tile_begin[5];  // first 16-row tile of each segment in the tile list
    uint32_t count, mode;
    uint32_t ksb, ksl, nks;  // superblocks per row, per slice; slices
    uint32_t total_tiles;    // tiles per slice (pair mode: gate and up tiles interleaved)
    uint32_t win_sb;         // superblocks of activations the widest block window holds
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

__host__ __device__ __forceinline__ uint32_t slice_sbs(const Params &p, uint32_t ks) { const uint32_t left = p.ksb - ks * p.ksl; return p.ksl < left ? p.ksl : left; }

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
__host__ __device__ __forceinline__ uint32_t unit_at(const Params &p, unsigned long long target) {
    const unsigned long long full = (unsigned long long)p.total_tiles * p.ksl;  // tasks of a full slice
    uint32_t ks = (uint32_t)(target / full);
    if (ks >= p.nks) ks = p.nks - 1;
    const unsigned long long rem = target - (unsigned long long)ks * full;
    const uint32_t n = slice_sbs(p, ks);
    uint32_t tile = (uint32_t)((rem + n - 1) / n);
    if (tile > p.total_tiles) tile = p.total_tiles;
    return ks * p.total_tiles + tile;
}

// A warp's walk over its tasks: units u_begin + slot, + 4, ... and in each the superblocks part, part + 4, ...
struct Walk {
    uint32_t u;        // unit
    uint32_t sb;       // superblock within the unit's slice
    uint32_t n;        // superblocks of the unit's slice
    uint32_t sb0;      // first superblock of the unit's slice
    uint32_t seg, row0;
};
__device__ __forceinline__ void walk_enter(const Params &p, Walk &w, uint32_t u_end, uint32_t part) {
    // settle on the next unit (at or after w.u) that has a superblock for this part
    while (w.u < u_end) {
        const uint32_t ks = w.u / p.total_tiles;
        w.n = slice_sbs(p, ks);
        if (part < w.n) {
            w.sb = part;
            w.sb0 = ks * p.ksl;
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

template <class E, int STAGES>
__global__ void __launch_bounds__(THREADS, 1) decode_kernel(const __grid_constant__ Params p) {
    constexpr int TASK_BYTES = E::TASK_BYTES;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t K = p.win_sb * 256;  // columns the staging area holds: the widest window of any block
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
    float *slots = gsum + p.win_sb * E::GSUMS;
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
#define NU_TRACE(i) do { if (tid == 0) { unsigned long long tt; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tt)); trace_ns[(i)] = tt; } } while (0)
#else
#define NU_TRACE(i)
#endif
    // Programmatic dependent launch: the next kernel of the stream may take an SM as soon as this
    // block leaves it, and this kernel starts its weight stream (weights are constant) while the
    // previous kernel is still finishing elsewhere. Everything that reads the previous kernel's
    // output or writes global memory comes after grid_dependency_wait() below.
    asm volatile("griddepcontrol.launch_dependents;");
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
    // The activations this block needs: the columns of the slices its units lie in.
    const uint32_t ks_first = u_begin < u_end ? u_begin / p.total_tiles : 0, ks_last = u_begin < u_end ? (u_end - 1) / p.total_tiles : 0;
    const uint32_t win0 = ks_first * p.ksl;                                                  // first superblock of the window
    const uint32_t win_n = u_begin < u_end ? min(p.ksb, (ks_last + 1) * p.ksl) - win0 : 0;   // superblocks in the window

    // ---- start the weight stream before anything else ----
    Walk prod;
    prod.u = u_begin + slot;
    walk_enter(p, prod, u_end, part);
    Walk cons = prod;
    uint32_t issued = 0, consumed = 0;
    auto issue = [&]() {
        if (lane == 0) {
            const uint32_t st = issued % STAGES;
            E::issue(p, prod.seg, prod.sb0 + prod.sb, prod.row0, stage0 + st * TASK_BYTES, bar0 + st * 8, policy);
        }
        ++issued;
        walk_next(p, prod, u_end, part);
    };
    // Only a part of the ring is requested before the activations: loads are served in order, and
    // the activation row queued behind a full ring of weights would arrive microseconds late.
    constexpr int PRE = NU_DEC_PRE < STAGES - 1 ? NU_DEC_PRE : STAGES - 1;
    for (int i = 0; i < PRE; ++i)
        if (prod.u < u_end) issue();
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the previous kernel has ended; its writes are visible
    NU_TRACE(4);

    // ---- stage the activation row: scale, split into fp16 pieces, group sums ----
    // The row is read from global memory once and kept in registers between the two passes.
    constexpr int XV = (20480 / 4 + THREADS - 1) / THREADS;  // float4 per thread: rows of up to 20480 columns
    float4 xv[XV];
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < XV; ++j) {
        const uint32_t i = tid + j * THREADS;
        xv[j] = i < win_n * 64 ? ((const float4 *)p.in)[win0 * 64 + i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int i = PRE; i < STAGES - 1; ++i)  // the loads above are in flight; the rest of the ring follows them
        if (prod.u < u_end) issue();
#pragma unroll
    for (int j = 0; j < XV; ++j) mx = fmaxf(mx, fmaxf(fmaxf(fabsf(xv[j].x), fabsf(xv[j].y)), fmaxf(fabsf(xv[j].z), fabsf(xv[j].w))));
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
        if (i < win_n * 64) {  // uniform per warp: a multiple of 32
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
            const uint32_t off = E::x_offset(i);
            *(uint2 *)(xhi + off) = hi;
            *(uint2 *)(xlo + off) = lo;
            E::group_sum(gsum, i, (x0 + x1) + (x2 + x3), lane);
        }
    }
    __syncthreads();
    NU_TRACE(0);

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
                const uint32_t sb_win = cons.sb0 + cons.sb - win0;
                const uint8_t *xb = mine ? piece + (sb_win * 4 + t) * PAIR_PITCH : zero;  // this lane's 64 columns: 128 B of halves
                E::task(task, xb, gsum + sb_win * E::GSUMS, g, t, acc);
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
        printf("TR tiles %u ksb %u block %u start %llu waited %llu staged %llu tasks %llu reduced %llu\n", p.total_tiles, p.ksb, blockIdx.x, t_start, trace_ns[4], trace_ns[0], trace_ns[1], trace_ns[3]);
#endif
    if (failed) {
        if (lane == 0) atomicExch(p.status, 1u);
        // let this warp's copies still in flight land before the block's shared memory is released
        for (; consumed < issued; ++consumed) mbar_wait(bar0 + (consumed % STAGES) * 8, (consumed / STAGES) & 1u);
    }
}

template <class E>
static size_t smem_bytes(uint32_t win_sb, int stages) {
    return (size_t)WARPS * stages * E::TASK_BYTES + (size_t)(win_sb * 4) * PAIR_PITCH * 2 + 512 + (size_t)win_sb * E::GSUMS * 4 + ROUND_STEPS * SLOTS * PARTS * 64 +
           ROUND_STEPS * SLOTS * 4 + 128 + WARPS * stages * 8 + 128;
}

#ifdef NU_DEC_TRACE
constexpr size_t kSmemMax = 226 * 1024;  // the trace keeps a few words of static shared memory
#else
constexpr size_t kSmemMax = 227 * 1024;
#endif
constexpr int kMaxColumns = 20480;  // the staging pass keeps the activation row in registers

// Deepest ring of task stages that fits beside the staged activations: the copies in flight hide HBM latency.
template <class E>
static int pick_stages(uint32_t win_sb) {
    for (int st = 6; st >= 2; --st)
        if (smem_bytes<E>(win_sb, st) <= kSmemMax) return st;
    return 0;
}

template <class E, int STAGES>
static bool configure_one() {
    return cudaFuncSetAttribute(decode_kernel<E, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax) == cudaSuccess;
}
template <class E>
static bool configure() { return configure_one<E, 2>() && configure_one<E, 3>() && configure_one<E, 4>() && configure_one<E, 5>() && configure_one<E, 6>(); }

// Fills everything of Params that does not depend on the encoding's planes; the caller adds the tensor maps.
template <class E>
static bool fill_common(const FastJob &job, Params &p) {
    if (job.tokens != 1 || job.count < 1 || job.count > 4) return false;
    if (job.columns == 0 || job.columns % 256 != 0) return false;
    if (job.columns > kMaxColumns) return false;
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
        if (g.rows == 0 || (uintptr_t)g.w % 16 != 0 || (uintptr_t)g.out % 4 != 0) return false;
        p.out[s] = g.out;
        p.rows[s] = g.rows;
        p.tile_begin[s] = tiles;
        tiles += (g.rows + 15) / 16;
        rows_total += g.rows;
    }
    for (uint32_t s = job.count; s < 5; ++s) p.tile_begin[s] = tiles;
    p.total_tiles = tiles;  // pair mode: gate tile i and up tile i are tiles 2i and 2i+1
    // Slices: one if that fills the machine evenly, else the count that wastes least: whole steps of
    // unit slots per block, four superblock parts per unit, against the partial sums and fences of a split.
    double best = -1.0;
    const double weight_bytes = (double)p.ksb * E::ROW_BYTES * rows_total;
    for (uint32_t nks = 1; nks <= p.ksb && nks <= 32; ++nks) {
        const uint32_t ksl = (p.ksb + nks - 1) / nks;
        const uint32_t slices = (p.ksb + ksl - 1) / ksl;
        const double units = (double)slices * tiles;
        const double blocks = units < job.sm_count ? units : job.sm_count;
        const double per_block = units / blocks;
        const double steps = (double)(uint64_t)((per_block + SLOTS - 1) / SLOTS);
        double eff = per_block / (steps * SLOTS);                                  // idle unit slots in the last step
        eff *= (double)ksl / ((double)((ksl + PARTS - 1) / PARTS) * PARTS);        // idle parts
        if (slices > 1) eff /= 1.2 + 2.0 * slices * tiles * 64.0 / weight_bytes;   // partial sums, fences and a second reduction
        if (eff > best + 1e-9) { best = eff; p.ksl = ksl; p.nks = slices; }
    }
    // The widest activation window of any block sizes the staging area (and so the depth of the task ring).
    {
        const uint32_t units = p.nks * tiles;
        const uint32_t grid = units < (uint32_t)job.sm_count ? units : (uint32_t)job.sm_count;
        const unsigned long long total_tasks = (unsigned long long)tiles * p.ksb;
        p.win_sb = 0;
        for (uint32_t b = 0; b < grid; ++b) {
            uint32_t ub = unit_at(p, total_tasks * b / grid);
            uint32_t ue = b + 1 == grid ? units : unit_at(p, total_tasks * (b + 1) / grid);
            if (job.mode != ACT_NONE) { ub &= ~1u; ue &= ~1u; }
            if (ub >= ue) continue;
            const uint32_t k0 = ub / tiles, k1 = (ue - 1) / tiles;
            const uint32_t hi = (k1 + 1) * p.ksl < p.ksb ? (k1 + 1) * p.ksl : p.ksb;
            if (hi - k0 * p.ksl > p.win_sb) p.win_sb = hi - k0 * p.ksl;
        }
        if (p.win_sb == 0 || pick_stages<E>(p.win_sb) == 0) return false;
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

// NUCLIS_NO_OVERLAP=1 in the environment launches every kernel fully serialised (for measurements).
inline bool overlap_launches() {
    static const bool on = [] { const char *e = getenv("NUCLIS_NO_OVERLAP"); return !(e && e[0] == '1'); }();
    return on;
}

template <class E>
static int launch(cudaStream_t s, const FastJob &job, const Params &p) {
    const uint32_t units = p.nks * p.total_tiles;
    const uint32_t grid = units < (uint32_t)job.sm_count ? units : (uint32_t)job.sm_count;
    const int stages = pick_stages<E>(p.win_sb);
    const size_t bytes = smem_bytes<E>(p.win_sb, stages);
    // launched so that it may overlap the tail of the kernel before it (see the kernel's prologue)
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = bytes;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_launches() && !job.serial ? 1 : 0;
    switch (stages) {
    case 6: cudaLaunchKernelEx(&cfg, decode_kernel<E, 6>, p); break;
    case 5: cudaLaunchKernelEx(&cfg, decode_kernel<E, 5>, p); break;
    case 4: cudaLaunchKernelEx(&cfg, decode_kernel<E, 4>, p); break;
    case 3: cudaLaunchKernelEx(&cfg, decode_kernel<E, 3>, p); break;
    default: cudaLaunchKernelEx(&cfg, decode_kernel<E, 2>, p); break;
    }
    return 1;
}

}  // namespace dec

bool encode_weight_map(CUtensorMap *map, const uint8_t *base, uint64_t row_bytes, uint64_t rows, uint64_t stride, uint32_t box_bytes, uint32_t box_rows);

}  // namespace nu
