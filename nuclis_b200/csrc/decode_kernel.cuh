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

#ifndef NU_DEC_PRE
#define NU_DEC_PRE 3
#endif
// A block's warps are unit slots x K parts. Plain GEMVs run 20 warps as 4 slots x 5 parts (a 20-superblock
// row is 4 tasks per warp and unit; measured 5 to 10 % faster alone than 16 warps); gate/up pairs measured
// better with 16 warps as 4 x 4 and a deeper ring.
template <int W, int P>
struct Geometry {
    static constexpr int WARPS = W, PARTS = P, SLOTS = W / P, THREADS = W * 32;
    static_assert(W % P == 0 && W <= 32 && W / P <= 8, "warps are unit slots x K parts; a named barrier per slot");
};
using Plain = Geometry<20, 5>;
using Pairs = Geometry<16, 4>;
constexpr int PAIR_PITCH = 136;    // bytes per 64 staged activations (128 of halves + 8 of bank skew)
constexpr int MAX_SLICES = 32;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

struct Params {
    CUtensorMap map[4];   // per segment: uint8 [rows][row bytes], box 16 rows x one superblock
    CUtensorMap map2[4];  // per segment: a second plane of the encoding, if it has one
    float *out[4];
    uint32_t rows[4];
    uint32_t tile_begin[5];  // first 16-row tile of each segment in the tile list
    uint32_t count, mode;
    uint32_t ksb, ksl, nks;  // superblocks per row, per slice; slices
    uint32_t units;          // units per slice: 16-row tiles (pair mode: a gate tile with its up tile)
    uint32_t blk_first[MAX_SLICES + 1];  // blocks blk_first[s] .. blk_first[s+1]-1 work on slice s
    const float *in;
    float *partials;         // [slice][unit][32]
    uint32_t *counters;      // per unit
    uint32_t *status;        // set to 1 if a bounded wait ran out
    PushTarget push;         // ranks > 0: output rows go to the ranks' inboxes instead of `out`
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

// Unit `unit` of a plain list -> segment and first row.
__device__ __forceinline__ void unit_rows(const Params &p, uint32_t unit, uint32_t &seg, uint32_t &row0) {
    seg = 0;
#pragma unroll
    for (int s = 1; s < 4; ++s)
        if ((uint32_t)s < p.count && unit >= p.tile_begin[s]) seg = s;
    row0 = (unit - p.tile_begin[seg]) * 16;
}
__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void push_word(uint2 *dst, float v, uint32_t tag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}

// Writes the finished sums of rows g and g+8 of a unit: v = plain sums (pair mode: gate), w = up sums.
__device__ __forceinline__ void write_unit(const Params &p, uint32_t unit, uint32_t g, float v0, float v1, float w0, float w1) {
    if (p.mode != ACT_NONE) {
        const uint32_t row = unit * 16 + g;
        if (row < p.rows[0]) p.out[0][row] = (p.mode == ACT_SILU ? silu_f32(v0) : gelu_f32(v0)) * w0;
        if (row + 8 < p.rows[0]) p.out[0][row + 8] = (p.mode == ACT_SILU ? silu_f32(v1) : gelu_f32(v1)) * w1;
    } else if (p.push.ranks) {
        // fused with the allreduce that follows: the rows travel to every rank's inbox as (value, tag)
        uint32_t seg, row0;
        unit_rows(p, unit, seg, row0);
        const uint32_t seq = *(volatile const uint32_t *)p.push.seq;
        const uint32_t tag = push_tag(seq);
        const size_t slot = ((size_t)(seq & 1u) * p.push.ranks + p.push.rank) * p.push.capacity;
#pragma unroll 1
        for (uint32_t r = 0; r < p.push.ranks; ++r) {
            uint2 *dst = p.push.inbox[r] + slot + row0 + g;
            if (row0 + g < p.rows[seg]) push_word(dst, v0, tag);
            if (row0 + g + 8 < p.rows[seg]) push_word(dst + 8, v1, tag);
        }
    } else {
        uint32_t seg, row0;
        unit_rows(p, unit, seg, row0);
        if (row0 + g < p.rows[seg]) p.out[seg][row0 + g] = v0;
        if (row0 + g + 8 < p.rows[seg]) p.out[seg][row0 + g + 8] = v1;
    }
}

// Work split. K is cut into `nks` slices and every slice owns a range of blocks (sized by the host
// so that all blocks finish together); the blocks of a slice split its units evenly, so a block
// stages the activations of one slice only. A block's warps are unit slots x K parts (4 x 4 or 4 x 5): warp
// (slot, part) takes units first + slot, + SLOTS, ... of the block and in each the superblocks part,
// part + PARTS, ... of the slice. The warps of a slot meet at a named barrier of their own after
// each unit and the first adds the parts in order; there is no block-wide barrier after staging.
template <class E, class G, int STAGES>
__global__ void __launch_bounds__(G::THREADS, 1) decode_kernel(const __grid_constant__ Params p) {
    constexpr int TASK_BYTES = E::TASK_BYTES;
    constexpr int WARPS = G::WARPS, THREADS = G::THREADS, SLOTS = G::SLOTS, PARTS = G::PARTS;
    extern __shared__ __align__(128) uint8_t smem[];
    // [task stages][hi pieces][lo pieces][128 B of zeros][group sums][per-superblock 1/scale][staged flags][part sums][barriers]
    // A piece array holds the slice's columns as halves, the 128 bytes of each group pair (64 columns) padded
    // to PAIR_PITCH = 136: the four quad lanes then read four different pairs of banks, and the lo array starts
    // 32 bytes further round the banks than the hi array, so the eight loading lanes of a warp never collide.
    uint8_t *stages = smem;
    uint8_t *xhi = stages + WARPS * STAGES * TASK_BYTES;
    const uint32_t piece_bytes = (p.ksl * 4) * PAIR_PITCH;
    const uint32_t lo_skew = (128u - piece_bytes % 128u) % 128u + 32u;
    uint8_t *xlo = xhi + piece_bytes + lo_skew;
    uint8_t *zero = xlo + piece_bytes + (128u - (piece_bytes + lo_skew + piece_bytes) % 128u) % 128u;
    float *gsum = (float *)(zero + 128);
    float *inv_sb = gsum + p.ksl * E::GSUMS;           // per superblock of the slice: 1 / its activation scale
    volatile uint32_t *ready = (volatile uint32_t *)(inv_sb + p.ksl);  // per superblock: staged
    float *parts = (float *)(ready + p.ksl);           // SLOTS x 2 x (PARTS - 1) x 32 floats
    uint64_t *bars = (uint64_t *)(parts + SLOTS * 2 * (PARTS - 1) * 32);
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t slot = warp / PARTS, part = warp % PARTS;
    const uint8_t *my_stage = stages + warp * STAGES * TASK_BYTES;
    const uint32_t stage0 = smem_u32(my_stage), bar0 = smem_u32(bars + warp * STAGES);

    // Programmatic dependent launch: the next kernel of the stream may take an SM as soon as this
    // block leaves it, and this kernel starts its weight stream (weights are constant) while the
    // previous kernel is still finishing elsewhere. Everything that reads the previous kernel's
    // output or writes global memory comes after the griddepcontrol.wait below.
    asm volatile("griddepcontrol.launch_dependents;");
    // every warp owns its ring: it initialises its own barriers and nobody else touches them
    if (lane == 0) {
        for (int i = 0; i < STAGES; ++i) mbar_init(bar0 + i * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // ---- this block's slice and units ----
    const bool pair = p.mode != ACT_NONE;
    uint32_t ks = 0;
    while (ks + 1 < p.nks && blockIdx.x >= p.blk_first[ks + 1]) ++ks;
    const uint32_t sb0 = ks * p.ksl, n = min(p.ksl, p.ksb - sb0);
    const uint32_t nblk = p.blk_first[ks + 1] - p.blk_first[ks], jblk = blockIdx.x - p.blk_first[ks];
    // The first blocks of a slice take the units that do not divide evenly: blocks are dispatched in index
    // order onto the SMs as the kernel before frees them, so the SMs that were done early (the light ones
    // of that kernel) get the heavy blocks of this one, and the block that starts last has the least to do.
    const uint32_t per_blk = p.units / nblk, extra = p.units - per_blk * nblk;
    const uint32_t u_lo = jblk * per_blk + min(jblk, extra);
    const uint32_t u_hi = u_lo + per_blk + (jblk < extra ? 1u : 0u);
    const uint32_t np = min((uint32_t)PARTS, n);                          // warps that share a unit
    const uint32_t m = part < n ? (n - part + PARTS - 1) / PARTS : 0;     // this warp's superblocks per unit
    const uint32_t first_unit = u_lo + slot;
    const uint32_t my_units = first_unit < u_hi ? (u_hi - first_unit + SLOTS - 1) / SLOTS : 0;
    const uint32_t total = my_units * m * (pair ? 2u : 1u);
    const uint64_t policy = evict_first_policy();

    // ---- the weight stream: this warp's tasks in order (pair mode: gate then up of each superblock) ----
    uint32_t issued = 0, p_stage = 0, p_unit = first_unit, p_j = 0, p_seg = 0, p_row0 = 0;
    if (total) {
        if (pair) p_row0 = p_unit * 16;
        else unit_rows(p, p_unit, p_seg, p_row0);
    }
    auto issue = [&]() {
        if (lane == 0) E::issue(p, p_seg, sb0 + part + PARTS * p_j, p_row0, stage0 + p_stage * TASK_BYTES, bar0 + p_stage * 8, policy);
        ++issued;
        p_stage = p_stage + 1 == STAGES ? 0 : p_stage + 1;
        if (pair && p_seg == 0) { p_seg = 1; return; }
        if (pair) p_seg = 0;
        if (++p_j == m) {
            p_j = 0;
            p_unit += SLOTS;
            if (pair) p_row0 = p_unit * 16;
            else if (issued < total) unit_rows(p, p_unit, p_seg, p_row0);
        }
    };
    // A part of the ring is requested before the wait (it streams under the tail of the kernel before),
    // the rest after the activation loads have left, so that those do not queue behind the whole ring.
    constexpr int PRE = NU_DEC_PRE < STAGES - 1 ? NU_DEC_PRE : STAGES - 1;
    for (int i = 0; i < PRE; ++i)
        if (issued < total) issue();
    for (uint32_t i = tid; i < p.ksl; i += THREADS) ready[i] = 0;
    if (tid < 32) ((uint32_t *)zero)[tid] = 0;
    __syncthreads();  // still under the tail of the previous kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the previous kernel has ended; its writes are visible

    // ---- stage the slice's activations, a superblock per warp at a time: scale, fp16 pieces, group sums ----
    // Warp w stages superblocks w, w + WARPS, ... of the slice (two float4 per lane each), with the
    // superblock's own power-of-two scale, and raises the superblock's flag; a task waits for the flag
    // of its superblock only, so the first tasks start while later superblocks are still being staged.
    {
        constexpr int SBW = (80 + WARPS - 1) / WARPS;  // superblocks per warp at most
        float4 xa[SBW], xb2[SBW];
#pragma unroll
        for (int j = 0; j < SBW; ++j) {
            const uint32_t sb = warp + j * WARPS;
            if (sb < n) {
                xa[j] = ((const float4 *)p.in)[(sb0 + sb) * 64 + lane];
                xb2[j] = ((const float4 *)p.in)[(sb0 + sb) * 64 + 32 + lane];
            }
        }
        for (int i = PRE; i < STAGES - 1; ++i)
            if (issued < total) issue();
#pragma unroll
        for (int j = 0; j < SBW; ++j) {
            const uint32_t sb = warp + j * WARPS;
            if (sb < n) {  // uniform per warp
                float mx = fmaxf(fmaxf(fmaxf(fabsf(xa[j].x), fabsf(xa[j].y)), fmaxf(fabsf(xa[j].z), fabsf(xa[j].w))),
                                 fmaxf(fmaxf(fabsf(xb2[j].x), fabsf(xb2[j].y)), fmaxf(fabsf(xb2[j].z), fabsf(xb2[j].w))));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                // 2^e puts the largest |x| in [2^13, 2^14): hi cannot overflow fp16, lo keeps 11 bits down to 2^-25 of the largest value
                const uint32_t e = (__float_as_uint(mx) >> 23) & 0xffu;
                const bool ok = e >= 40u && e < 255u;
                const float scale = ok ? __uint_as_float((267u - e) << 23) : 1.0f;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const float4 v = hf ? xb2[j] : xa[j];
                    const uint32_t i = sb * 64 + hf * 32 + lane;  // float4 index within the slice
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
                    const uint32_t off = E::x_offset(i);
                    *(uint2 *)(xhi + off) = hi;
                    *(uint2 *)(xlo + off) = lo;
                    E::group_sum(gsum, i, (x0 + x1) + (x2 + x3), lane);
                }
                if (lane == 0) inv_sb[sb] = ok ? __uint_as_float((e - 13u) << 23) : 1.0f;
                __threadfence_block();
                __syncwarp();
                if (lane == 0) ready[sb] = 1;
            }
        }
    }

    // ---- the task loop ----
    // Lanes whose B column is not theirs (column n = lane >> 2 belongs to quad lane n >> 1) read zeros.
    const bool mine = (g >> 1) == t;
    const uint8_t *piece = (g & 1u) ? xlo : xhi;
    const uint8_t *xlane = mine ? piece + t * PAIR_PITCH : zero;  // this lane's 64 columns of superblock 0: 128 B of halves
    const uint32_t xstep = mine ? 4 * PAIR_PITCH : 0;
    uint32_t c_stage = 0, c_phase = 0, consumed = 0;
    bool failed = false;
    uint32_t uidx = 0;
    for (uint32_t unit = first_unit; unit < u_hi; unit += SLOTS, ++uidx) {
        float acc[2] = {0.0f, 0.0f}, acc2[2] = {0.0f, 0.0f};  // rows g, g+8: this lane's groups, summed over the warp's superblocks
        // After a wait has run out the warp stops computing but still walks its units, so that the
        // warps it shares them with are not left at the barrier below.
        for (uint32_t j = 0; j < m && !failed; ++j) {
            const uint32_t sbw = part + PARTS * j;  // superblock within the slice
            if (issued < total) issue();  // keep STAGES - 1 tasks in flight
            if (uidx == 0) {
                // the first unit may run ahead of the staging of its superblocks
                uint32_t spins = 0;
                while (ready[sbw] == 0 && ++spins < SPIN_LIMIT) {}
                if (ready[sbw] == 0) { failed = true; break; }
                __threadfence_block();
            }
            if (!mbar_wait(bar0 + c_stage * 8, c_phase)) { failed = true; break; }
            const float inv = inv_sb[sbw];
            float tmp[2] = {0.0f, 0.0f};
            E::task(my_stage + c_stage * TASK_BYTES, xlane + sbw * xstep, gsum + sbw * E::GSUMS, g, t, tmp);
            acc[0] = fmaf(inv, tmp[0], acc[0]);
            acc[1] = fmaf(inv, tmp[1], acc[1]);
            __syncwarp();  // all lanes are done reading this stage before it is refilled
            ++consumed;
            if (++c_stage == STAGES) { c_stage = 0; c_phase ^= 1u; }
            if (pair) {
                if (issued < total) issue();
                if (!mbar_wait(bar0 + c_stage * 8, c_phase)) { failed = true; break; }
                float tmp2[2] = {0.0f, 0.0f};
                E::task(my_stage + c_stage * TASK_BYTES, xlane + sbw * xstep, gsum + sbw * E::GSUMS, g, t, tmp2);
                acc2[0] = fmaf(inv, tmp2[0], acc2[0]);
                acc2[1] = fmaf(inv, tmp2[1], acc2[1]);
                __syncwarp();
                ++consumed;
                if (++c_stage == STAGES) { c_stage = 0; c_phase ^= 1u; }
            }
        }
        if (part >= np) continue;  // this warp has no superblocks in this slice
        // the four lanes of a quad hold the four group pairs of the superblock
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], 1);
            acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], 2);
            if (pair) {
                acc2[h] += __shfl_xor_sync(0xffffffffu, acc2[h], 1);
                acc2[h] += __shfl_xor_sync(0xffffffffu, acc2[h], 2);
            }
        }
        // ---- the parts of the unit meet; part 0 adds them in part order ----
        float *buf = parts + ((slot * 2 + (uidx & 1u)) * (PARTS - 1)) * 32;
        if (part > 0 && t == 0) {
            float *dst = buf + (part - 1) * 32;
            dst[g] = acc[0];
            dst[g + 8] = acc[1];
            if (pair) { dst[16 + g] = acc2[0]; dst[24 + g] = acc2[1]; }
        }
        if (np > 1) named_barrier(1 + slot, 32 * np);
        if (part != 0 || t != 0) continue;
        for (uint32_t k = 1; k < np; ++k) {
            const float *src = buf + (k - 1) * 32;
            acc[0] += src[g];
            acc[1] += src[g + 8];
            if (pair) { acc2[0] += src[16 + g]; acc2[1] += src[24 + g]; }
        }
        if (p.nks > 1) {
            // several slices: leave the partial sums; they are published after the loop with one fence
            float *dst = p.partials + ((size_t)ks * p.units + unit) * 32;
            dst[g] = acc[0];
            dst[g + 8] = acc[1];
            if (pair) { dst[16 + g] = acc2[0]; dst[24 + g] = acc2[1]; }
        } else {
            write_unit(p, unit, g, acc[0], acc[1], acc2[0], acc2[1]);
        }
    }
    if (p.nks > 1 && part == 0 && my_units) {
        // The last block to arrive for a unit adds the slices in order. Lanes announce 32 units at a
        // time (one round trip for all of them), then the warp finishes those it was last for.
        __threadfence();
        __syncwarp();
        for (uint32_t base = 0; base < my_units; base += 32) {
            const uint32_t mine_u = base + lane;
            uint32_t last = 0;
            if (mine_u < my_units) last = atomicAdd(p.counters + first_unit + mine_u * SLOTS, 1u) == p.nks - 1;
            uint32_t mask = __ballot_sync(0xffffffffu, last != 0);
            if (mask) __threadfence();
            while (mask) {
                const uint32_t u = base + (uint32_t)__ffs((int)mask) - 1;
                mask &= mask - 1;
                const uint32_t unit = first_unit + u * SLOTS;
                // lane = row of the unit's 32 partial sums (pair mode: 16 gate, 16 up)
                // (eight loads in flight at a time; added in slice order)
                float sum = 0.0f;
                if (lane < 16 || pair) {
                    const float *src = p.partials + (size_t)unit * 32 + lane;
                    const size_t step = (size_t)p.units * 32;
                    for (uint32_t k0 = 0; k0 < p.nks; k0 += 8) {
                        float v[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) v[k] = k0 + k < p.nks ? __ldcg(src + (k0 + k) * step) : 0.0f;
#pragma unroll
                        for (int k = 0; k < 8; ++k) sum += v[k];
                    }
                }
                const float up = __shfl_down_sync(0xffffffffu, sum, 16);
                if (lane < 16) {
                    if (pair) {
                        const uint32_t row = unit * 16 + lane;
                        if (row < p.rows[0]) p.out[0][row] = (p.mode == ACT_SILU ? silu_f32(sum) : gelu_f32(sum)) * up;
                    } else {
                        uint32_t seg, row0;
                        unit_rows(p, unit, seg, row0);
                        if (row0 + lane < p.rows[seg]) {
                            if (p.push.ranks) {
                                const uint32_t seq = *(volatile const uint32_t *)p.push.seq;
                                const size_t slot = ((size_t)(seq & 1u) * p.push.ranks + p.push.rank) * p.push.capacity;
                                for (uint32_t r = 0; r < p.push.ranks; ++r) push_word(p.push.inbox[r] + slot + row0 + lane, sum, push_tag(seq));
                            } else {
                                p.out[seg][row0 + lane] = sum;
                            }
                        }
                    }
                }
                if (lane == 0) p.counters[unit] = 0;  // leave the scratch as it was found
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

template <class E, class G>
static size_t smem_bytes(uint32_t ksl, int stages) {
    constexpr int WARPS = G::WARPS, SLOTS = G::SLOTS, PARTS = G::PARTS;
    return (size_t)WARPS * stages * E::TASK_BYTES + (size_t)(ksl * 4) * PAIR_PITCH * 2 + 512 + (size_t)ksl * E::GSUMS * 4 + (size_t)ksl * 8 + SLOTS * 2 * (PARTS - 1) * 32 * 4 + 128 +
           WARPS * stages * 8 + 128;
}

constexpr size_t kSmemMax = 227 * 1024;
constexpr uint32_t kMaxSliceSbs = 80;  // the staging pass keeps a slice of up to 20480 columns in registers

// Deepest ring of task stages that fits beside the staged activations: the copies in flight hide HBM latency.
template <class E, class G>
static int pick_stages(uint32_t ksl) {
    for (int st = 6; st >= 2; --st)
        if (smem_bytes<E, G>(ksl, st) <= kSmemMax) return st;
    return 0;
}

template <class E, class G, int STAGES>
static bool configure_one() {
    return cudaFuncSetAttribute(decode_kernel<E, G, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax) == cudaSuccess;
}
template <class E, class G>
static bool configure_geometry() {
    return configure_one<E, G, 2>() && configure_one<E, G, 3>() && configure_one<E, G, 4>() && configure_one<E, G, 5>() && configure_one<E, G, 6>();
}
template <class E>
static bool configure() { return configure_geometry<E, Plain>() && configure_geometry<E, Pairs>(); }

// Fills everything of Params that does not depend on the encoding's planes; the caller adds the tensor maps.
// Picks the K slices and the blocks of each slice: every candidate slice length is costed in task
// steps of the slowest block (units over unit slots, superblocks over K parts).
template <class E, class G>
static bool fill_geometry(const FastJob &job, Params &p) {
    constexpr int SLOTS = G::SLOTS, PARTS = G::PARTS;
    if (job.tokens != 1 || job.count < 1 || job.count > 4) return false;
    if (job.columns == 0 || job.columns % 256 != 0) return false;
    if ((uintptr_t)job.in % 16 != 0) return false;
    if (job.mode != ACT_NONE && (job.count != 2 || job.seg[0].rows != job.seg[1].rows)) return false;
    memset(&p, 0, sizeof p);
    p.count = job.count;
    p.mode = job.mode;
    p.ksb = job.columns / 256;
    p.in = job.in;
    uint32_t tiles = 0;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows == 0 || (uintptr_t)g.w % 16 != 0 || (uintptr_t)g.out % 4 != 0) return false;
        p.out[s] = g.out;
        p.rows[s] = g.rows;
        p.tile_begin[s] = tiles;
        tiles += (g.rows + 15) / 16;
    }
    for (uint32_t s = job.count; s < 5; ++s) p.tile_begin[s] = tiles;
    const bool pair = job.mode != ACT_NONE;
    const uint32_t units = pair ? tiles / 2 : tiles;
    const double per_sb = pair ? 2.0 : 1.0;  // tasks per superblock of a unit
    p.units = units;
    const uint32_t sms = (uint32_t)job.sm_count;
    double best = 1e30;
    uint32_t blocks[MAX_SLICES];
    for (uint32_t ksl = 1; ksl <= p.ksb && ksl <= kMaxSliceSbs; ++ksl) {
        const uint32_t nks = (p.ksb + ksl - 1) / ksl;
        if (nks > MAX_SLICES || nks > sms) continue;
        // a slicing whose partial sums or arrival counters do not fit the caller's scratch is no candidate
        if (nks > 1 && ((size_t)nks * units * 32 > job.partials_floats || units > job.counters_len)) continue;
        const int st = pick_stages<E, G>(ksl);
        if (st < 2) continue;
        auto cost = [&](uint32_t s, uint32_t b) {
            const uint32_t n = s + 1 == nks ? p.ksb - s * ksl : ksl;
            const uint32_t units_blk = (units + b - 1) / b;
            return (double)((units_blk + SLOTS - 1) / SLOTS) * ((double)((n + PARTS - 1) / PARTS) * per_sb + 0.35);
        };
        for (uint32_t s = 0; s < nks; ++s) blocks[s] = 1;
        for (uint32_t left = sms - nks; left > 0; --left) {
            uint32_t worst = 0;
            for (uint32_t s = 1; s < nks; ++s)
                if (cost(s, blocks[s]) > cost(worst, blocks[worst])) worst = s;
            if (blocks[worst] >= units) break;
            ++blocks[worst];
        }
        double est = 0;
        for (uint32_t s = 0; s < nks; ++s) est = cost(s, blocks[s]) > est ? cost(s, blocks[s]) : est;
        est *= st >= 4 ? 1.0 : st == 3 ? 1.06 : 1.2;  // a shallow ring hides less latency
        est += (nks > 1 ? 5.0 + 0.3 * nks : 0.0) + 0.01 * ksl;  // partial sums, their fence and the last arriver's pass (measured: 4-6 us); staging of the slice
        if (est < best - 1e-9) {
            best = est;
            p.ksl = ksl;
            p.nks = nks;
            uint32_t first = 0;
            for (uint32_t s = 0; s < nks; ++s) { p.blk_first[s] = first; first += blocks[s]; }
            for (uint32_t s = nks; s <= MAX_SLICES; ++s) p.blk_first[s] = first;
        }
    }
    if (best >= 1e30) return false;
    p.partials = job.partials;
    p.counters = job.counters;
    p.status = job.counters + job.counters_len;
    p.push = job.push;
    if (p.push.ranks && (job.mode != ACT_NONE || job.count != 1)) return false;  // one plain matrix only
    return true;
}

template <class E, class G>
static int launch_geometry(cudaStream_t s, const FastJob &job, const Params &p) {
    const uint32_t grid = p.blk_first[p.nks];
    const int stages = pick_stages<E, G>(p.ksl);
    const size_t bytes = smem_bytes<E, G>(p.ksl, stages);
    // launched so that it may overlap the tail of the kernel before it (see the kernel's prologue)
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(G::THREADS);
    cfg.dynamicSmemBytes = bytes;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = job.serial ? 0 : 1;
    switch (stages) {
    case 6: cudaLaunchKernelEx(&cfg, decode_kernel<E, G, 6>, p); break;
    case 5: cudaLaunchKernelEx(&cfg, decode_kernel<E, G, 5>, p); break;
    case 4: cudaLaunchKernelEx(&cfg, decode_kernel<E, G, 4>, p); break;
    case 3: cudaLaunchKernelEx(&cfg, decode_kernel<E, G, 3>, p); break;
    default: cudaLaunchKernelEx(&cfg, decode_kernel<E, G, 2>, p); break;
    }
    return 1;
}

// The geometry follows the job: gate/up pairs on Pairs, everything else on Plain.
inline bool on_pairs(const FastJob &job) { return job.mode != ACT_NONE; }
template <class E>
static bool fill_common(const FastJob &job, Params &p) {
    return on_pairs(job) ? fill_geometry<E, Pairs>(job, p) : fill_geometry<E, Plain>(job, p);
}
template <class E>
static int launch(cudaStream_t s, const FastJob &job, const Params &p) {
    return on_pairs(job) ? launch_geometry<E, Pairs>(s, job, p) : launch_geometry<E, Plain>(s, job, p);
}

}  // namespace dec

bool encode_weight_map(CUtensorMap *map, const uint8_t *base, uint64_t row_bytes, uint64_t rows, uint64_t stride, uint32_t box_bytes, uint32_t box_rows);

}  // namespace nu
