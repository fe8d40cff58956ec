// GEMV / small-batch GEMM skeleton on the integer tensor path (1..8 activation rows) shared by the
// block encodings. The activation rows are turned into fixed point once per block: per token row and
// superblock a power of two puts the largest |x| in [2^21, 2^22), X = round(x * 2^k), and X is cut into
// three balanced base-256 digits X = d2*2^16 + d1*2^8 + d0, each in [-128, 127], kept as three planes of
// bytes in shared memory. The weight codes stay what they are, bytes, so
// mma.sync.m16n8k32.s32.u8.s8 gives sum(code * digit) exactly, 512 weights per instruction, and the
// products need no conversion at all: one mask per four codes. The three digit sums are recombined
// once per superblock (exactly in F32 up to the last bit), scaled by the superblock's F32 factors and
// accumulated in F32. An element of x is off by at most 2^-22 of its superblock's largest value.
//
// The B operand's 8 columns hold (digit plane, token): with one or two tokens one mma serves all
// three planes (column = plane * 2 + token); with three or four tokens two mmas do (planes 0 and 1 in
// the first, plane 2 in half of the second); with five to eight tokens each plane takes an mma of its
// own (column = token). The k index of an mma is a column within one scale group, so the group's
// scale multiplies the int32 sums after the mma (an integer scale by one IMAD per accumulator
// register, Q8_0's f16 scale in F32).
//
// An encoding supplies a policy class E: the bytes of a task (16 weight rows x one superblock), the
// copy that fetches it, and the mma loop over one task. Work split, task ring, programmatic dependent
// launch and the sums across K parts and K slices are described at run_op below; the small device helpers
// (barriers, copies) are in gemv_common.cuh.
#pragma once
#include "gemv_common.cuh"

namespace nu {
namespace i8 {

using dec::evict_first_policy;
using dec::mbar_expect_tx;
using dec::mbar_init;
using dec::mbar_wait;
using dec::named_barrier;
using dec::push_word;
using dec::smem_u32;
using dec::tma_load_2d;

constexpr int MAX_SLICES = 32;
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int SBW = 4;  // (token, superblock) pairs a warp stages per pass: a pass keeps them in registers

template <int W, int P>
struct Geometry {
    static constexpr int WARPS = W, PARTS = P, SLOTS = W / P, THREADS = W * 32;
    static_assert(W % P == 0 && W <= 32 && W / P <= 8, "warps are unit slots x K parts; a named barrier per slot");
};

struct Params {
    CUtensorMap map[4];   // per segment: uint8 [rows][row bytes], box 16 rows x one superblock
    CUtensorMap map2[4];  // per segment: a second plane of the encoding, if it has one
    float *out[4];
    uint32_t out_stride[4];
    uint32_t rows[4];
    uint32_t tile_begin[5];  // first 16-row tile of each segment in the tile list
    uint32_t count, mode, tokens;
    uint32_t ksb, ksl, nks;  // superblocks per row, per slice; slices
    uint32_t units;          // units per slice: 16-row tiles (pair mode: a gate tile with its up tile)
    uint32_t blk_first[MAX_SLICES + 1];  // blocks blk_first[s] .. blk_first[s+1]-1 work on slice s
    uint32_t plane_pitch;    // bytes between the digit rows of two B columns (32 or 16 mod 128: the eight rows a warp reads hit different banks)
    uint32_t gs_pitch;       // bytes between the group-sum rows of two B columns (16 mod 128)
    const float *in;
    uint32_t in_stride;
    float *partials;         // [slice][unit][pair half][record]
    uint32_t *counters;      // per unit
    uint32_t *status;        // set to 1 if a bounded wait ran out
    PushTarget push;         // ranks > 0: output rows go to the ranks' inboxes instead of `out`
    // The add + RMS norm ahead of the projections, folded into the staging pass when norm_weight is set: the rows the
    // kernel multiplies are (in + norm_input) * rsqrt(mean((in + norm_input)^2) + norm_eps) * norm_weight; block 0 writes
    // in + norm_input to residual_out. norm_input and residual_out may be null; all three row sets share in_stride.
    const float *norm_weight;
    const float *norm_input;
    float *residual_out;
    float norm_eps;
    const float *add0;       // not null: segment 0's output rows are add0[token * out_stride + row] + the products (may be `out` itself)
};

// C = A(16 x 32, unsigned bytes) x B(32 x 8, signed bytes), int32, starting from zero.
__device__ __forceinline__ void imma_u8(int c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
// The same with signed codes.
__device__ __forceinline__ void imma_s8(int c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
// C += A(16 x 8, f16) x B(8 x 8, f16): the minima (or biases) of a row against the group sums of x.
__device__ __forceinline__ void hmma_k8(float c[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Row of the task a lane's mma row g (0..7) stands for. Task rows are 144 bytes = 36 words apart, so the
// eight-byte pieces the lanes of a half-warp (g = 0..3 or 4..7) read hit distinct banks only when their
// rows are two apart: 0, 2, 4, 6 and 1, 3, 5, 7. Row g + 8 of the mma is task row row_of(g) + 8.
__device__ __forceinline__ uint32_t row_of(uint32_t g) { return g < 4 ? 2 * g : 2 * g - 7; }

// NT is the number of token columns a kernel instance is built for: 1, 2 (narrow: one mma serves the three
// digit planes), 4 (three or four tokens: two mmas, planes 0 and 1 in the first, plane 2 in half of the second) or
// 8 (wide: five to eight tokens, an mma per plane).
template <int NT>
__host__ __device__ constexpr int token_stride() { return NT == 8 ? 8 : NT == 4 ? 4 : 2; }  // rows between two digit planes (and between the hi and lo group sums)
template <int NT>
__host__ __device__ constexpr int plane_columns() { return 3 * token_stride<NT>(); }  // digit rows staged: planes x tokens
template <int NT>
__host__ __device__ constexpr int gs_columns() { return 2 * token_stride<NT>(); }     // group-sum rows staged: (hi, lo) x tokens
template <int NT>
__host__ __device__ constexpr int record_lanes() { return NT == 8 ? 32 : NT == 4 ? 16 : 8; }  // float4 a unit's sums take (the lanes that hold sums)
template <int NT>
__host__ __device__ constexpr int mma_count() { return NT == 8 ? 3 : NT == 4 ? 2 : 1; }  // integer mmas per scale group

__device__ __forceinline__ void unit_rows(const Params &p, uint32_t unit, uint32_t &seg, uint32_t &row0) {
    seg = 0;
#pragma unroll
    for (int s = 1; s < 4; ++s)
        if ((uint32_t)s < p.count && unit >= p.tile_begin[s]) seg = s;
    row0 = (unit - p.tile_begin[seg]) * 16;
}

// Writes the finished sums a lane holds for a unit. v: (row r, token a), (row r, token a + 1), (row r + 8, a), (row r + 8, a + 1)
// with r the task row of the lane's mma row (E::row); narrow: a = 0 and only quad lane 0 holds sums; four tokens: a = 2t in quad lanes 0 and 1; wide: a = 2t.
// w: the up sums in pair mode.
template <int NT, bool FOLD>
__device__ __forceinline__ void write_unit(const Params &p, uint32_t unit, uint32_t r, uint32_t t, const float v[4], const float w[4]) {
    constexpr bool WIDE = NT == 8, QUAD = NT == 4;
    if (QUAD ? t >= 2 : (!WIDE && t != 0)) return;
    const uint32_t tok0 = (WIDE || QUAD) ? 2 * t : 0;
    if (p.mode != ACT_NONE) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t row = unit * 16 + r + 8 * h;
            if (row >= p.rows[0]) continue;
#pragma unroll
            for (int c = 0; c < 2; ++c)
                if (tok0 + c < p.tokens) {
                    const float gate = v[2 * h + c];
                    p.out[0][(size_t)(tok0 + c) * p.out_stride[0] + row] = (p.mode == ACT_SILU ? silu_f32(gate) : gelu_f32(gate)) * w[2 * h + c];
                }
        }
        return;
    }
    uint32_t seg, row0;
    unit_rows(p, unit, seg, row0);
    if (p.push.ranks) {
        // fused with the allreduce that follows (one token): the rows travel to every rank's inbox as (value, tag)
        const uint32_t seq = *(volatile const uint32_t *)p.push.seq;
        const uint32_t tag = push_tag(seq);
        const size_t slot = ((size_t)(seq & 1u) * p.push.ranks + p.push.rank) * p.push.capacity;
#pragma unroll 1
        for (uint32_t k = 0; k < p.push.ranks; ++k) {
            uint2 *dst = p.push.inbox[k] + slot + row0 + r;
            if (row0 + r < p.rows[seg]) push_word(dst, v[0], tag);
            if (row0 + r + 8 < p.rows[seg]) push_word(dst + 8, v[2], tag);
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t row = row0 + r + 8 * h;
        if (row >= p.rows[seg]) continue;
#pragma unroll
        for (int c = 0; c < 2; ++c)
            if (tok0 + c < p.tokens) {
                const size_t at = (size_t)(tok0 + c) * p.out_stride[seg] + row;
                // the residual add behind a projection, folded into its write: the thread that writes a row is the only one that reads it
                p.out[seg][at] = (FOLD && p.add0 && seg == 0) ? p.add0[at] + v[2 * h + c] : v[2 * h + c];
            }
    }
}


// Shared memory: [barriers and parameter copies][stages][digit rows][group-sum rows][128 zero bytes][1/scale per (superblock, token)][part sums][slot sums]
// The barriers sit at a fixed place, a fixed distance apart per unit slot, so that the operators of a chain
// (gemv_chain.cu), whose geometries differ, find the barriers the operator before them left.
constexpr int kMaxStages = 5;
constexpr int kBarBytes = 3712;               // 8 unit slots x (kMaxStages full + kMaxStages empty) x 8 bytes = 640, then room for two
                                              // copies of an operator's Params (a chain keeps the current and the next one there)
constexpr int kParamsAt = 768;                // the first copy; the second follows it
static_assert(kParamsAt + 2 * sizeof(Params) <= kBarBytes && sizeof(Params) % 16 == 0, "the head of shared memory holds two Params");
constexpr int kSlotBarBytes = 2 * kMaxStages * 8;
template <class E, class G, int NT>
static size_t smem_bytes(uint32_t ksl, bool pair, int stages) {
    const size_t plane_pitch = (size_t)ksl * 256 + E::PLANE_SKEW;
    const size_t gs_pitch = (size_t)ksl * E::GS_BYTES + (16 + 128 - ((size_t)ksl * E::GS_BYTES) % 128) % 128;
    const size_t parts = (size_t)G::SLOTS * (2 * (G::PARTS - 1) + 1) * (pair ? 2 : 1) * record_lanes<NT>() * 16;  // part sums (two sets) and slot sums
    return kBarBytes + (size_t)G::SLOTS * stages * E::STAGE_BYTES + plane_columns<NT>() * plane_pitch + gs_columns<NT>() * gs_pitch + 128 + (size_t)ksl * 8 * 4 + parts + 256;
}

// How an operator of a chain follows the one before it in the same launch. A kernel of its own has target 0.
struct ChainLink {
    uint32_t *arrivals;    // blocks that have finished an operator of the chain, counted over the whole launch
    uint32_t target;       // the count at which every block has finished the operator before this one
    uint32_t prev_slots;   // unit slots and stages of the operator before: its barriers are invalidated before this one's are made
    uint32_t prev_stages;
};
constexpr uint32_t CHAIN_SPIN_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) { asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory"); }

// One operator: 16-row units of the matrices of p against the staged activation rows. Every thread of the
// first G::THREADS of the block calls it; STAGES is the depth of a slot's ring.
// p: the operator's parameters where they are cheapest to read (the kernel's own parameter, or a copy in shared memory);
// pm: where its tensor maps may be handed to the copy engine (the kernel's parameter space).
// SHARE: the instance whose slots share the units of a block's last round (below); the host picks it per geometry
// (fill_geometry).
// FOLD: the instance that can fold the add + RMS norm ahead of the projections into its staging pass and a residual add
// into its write (Params::norm_weight, add0); the plain instance carries none of that code.
template <class E, class G, int NT, bool SHARE, bool FOLD = false>
__device__ __forceinline__ void run_op(const Params &p, const Params &pm, const int STAGES, uint8_t *smem, const ChainLink link) {
    constexpr bool WIDE = NT == 8, QUAD = NT == 4;
    constexpr uint32_t TS = token_stride<NT>();
    constexpr int STAGE_BYTES = E::STAGE_BYTES;  // 16 weight rows x PARTS superblocks (one TMA box, one task per warp of the slot),
                                                 // then whatever second plane the encoding's records need
    constexpr int WARPS = G::WARPS, SLOTS = G::SLOTS, PARTS = G::PARTS;
    static_assert(PARTS == E::STAGE_SBS, "a stage holds one superblock per K part");
    constexpr int REC = record_lanes<NT>();
    const bool pair = p.mode != ACT_NONE;
    uint8_t *stages = smem + kBarBytes;
    uint8_t *planes = stages + SLOTS * STAGES * STAGE_BYTES;
    uint8_t *gs = planes + plane_columns<NT>() * p.plane_pitch;
    uint8_t *zero = gs + gs_columns<NT>() * p.gs_pitch;        // 128 bytes of zeros (group sums of the B columns no token uses)
    zero += (128u - (uint32_t)(zero - smem) % 128u) % 128u;
    float *inv = (float *)(zero + 128);                        // [superblock of the slice][8 tokens]: 1 / the activation scale
    float4 *parts = (float4 *)(((uintptr_t)(inv + p.ksl * 8) + 15) & ~(uintptr_t)15);
    float4 *coopbuf = parts + SLOTS * 2 * (PARTS - 1) * (pair ? 2 : 1) * REC;  // sums of the slots that share a unit
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t slot = warp / PARTS, part = warp % PARTS;
    // A slot's warps share one ring of stages. full[i]: the copy into stage i has landed (all of them wait on it);
    // empty[i]: all of them have read stage i (the slot's first warp waits on it before it refills the stage).
    const uint8_t *my_stage = stages + slot * STAGES * STAGE_BYTES;
    const uint32_t stage0 = smem_u32(my_stage), full0 = smem_u32(smem) + slot * kSlotBarBytes, empty0 = full0 + kMaxStages * 8;

    // Programmatic dependent launch: the next kernel of the stream may take an SM as soon as this
    // block leaves it, and this kernel starts its weight stream (weights are constant) while the
    // previous kernel is still finishing elsewhere. Everything that reads the previous kernel's
    // output or writes global memory comes after the griddepcontrol.wait below. In a chain the
    // same holds between operators: the weight stream of this one starts while other blocks are
    // still in the one before, and the wait is for the chain's arrival count.
    if (!link.target) asm volatile("griddepcontrol.launch_dependents;");
    if (part == 0 && lane == 0) {
        if (link.target) {
            // the barriers the operator before left (this slot's; the last slot also takes those of slots this operator has not)
            const uint32_t upto = slot == SLOTS - 1 ? max((uint32_t)SLOTS, link.prev_slots) : slot + 1;
            for (uint32_t s2 = slot; s2 < upto && s2 < link.prev_slots; ++s2)
                for (uint32_t i = 0; i < link.prev_stages; ++i) {
                    mbar_inval(smem_u32(smem) + s2 * kSlotBarBytes + i * 8);
                    mbar_inval(smem_u32(smem) + s2 * kSlotBarBytes + (kMaxStages + i) * 8);
                }
        }
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(full0 + i * 8, 1);
            mbar_init(empty0 + i * 8, PARTS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // shared memory the operator before wrote through the generic proxy is about to be written by copies
        if (link.target) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }

    // ---- this block's slice and units ----
    uint32_t ks = 0;
    while (ks + 1 < p.nks && blockIdx.x >= p.blk_first[ks + 1]) ++ks;
    const uint32_t sb0 = ks * p.ksl, n = min(p.ksl, p.ksb - sb0);
    const uint32_t nblk = p.blk_first[ks + 1] - p.blk_first[ks], jblk = blockIdx.x - p.blk_first[ks];
    // The first blocks of a slice take the units that do not divide evenly: blocks are dispatched in index
    // order onto the SMs as the kernel before frees them, so the block that starts last has the least to do.
    const uint32_t per_blk = p.units / nblk, extra = p.units - per_blk * nblk;
    const uint32_t u_lo = jblk * per_blk + min(jblk, extra);
    const uint32_t u_hi = u_lo + per_blk + (jblk < extra ? 1u : 0u);
    const uint32_t np = min((uint32_t)PARTS, n);   // warps of a slot that have superblocks in this slice
    const uint32_t m = (n + PARTS - 1) / PARTS;    // stages per unit (pair mode: per matrix of the unit)
    // The block's units go to its slots in rounds of SLOTS. When the last round has units for at most half of the
    // slots, `coop` slots share each of its units: slot i of a group streams the i-th part of the unit's stages, and
    // the groups' first slots add the others' sums (in slot order) from shared memory. Otherwise a small matrix would
    // leave most slots of every block idle for a whole unit.
    const uint32_t nunits = u_hi - u_lo, full = nunits / SLOTS, rem = nunits - full * SLOTS;
    const uint32_t coop = (SHARE && rem && 2 * rem <= (uint32_t)SLOTS) ? min((uint32_t)SLOTS / rem, m) : 1u;
    const bool in_last = slot < rem * coop;
    const uint32_t ci = slot % coop, group = slot / coop;           // place in the group; the group's unit of the last round
    const uint32_t last_unit = u_lo + full * SLOTS + group;
    const uint32_t jb = in_last ? ci * m / coop : 0u, je = in_last ? (ci + 1) * m / coop : 0u;  // its stages of that unit
    const uint32_t my_items = full + (in_last ? 1u : 0u);           // units (or shares of one) this slot works on
    const uint32_t my_units = full + (in_last && ci == 0 ? 1u : 0u);  // units whose sums this slot finishes and writes
    const uint32_t total = (full * m + (je - jb)) * (pair ? 2u : 1u);  // stages the slot streams
    auto item_unit = [&](uint32_t i) { return i < full ? u_lo + i * SLOTS + slot : last_unit; };

    // ---- the weight stream: the slot's stages in order (pair mode: gate then up of each group of superblocks). Only
    // the slot's first warp keeps this state; it refills a stage once all warps of the slot have left it.
    uint32_t issued = 0, p_stage = 0, p_phase = 0, p_item = 0, p_unit = item_unit(0), p_j = full ? 0u : jb, p_seg = 0, p_row0 = 0;
    bool stuck = false;
    const uint64_t policy = evict_first_policy();
    if (total) {
        if (pair) p_row0 = p_unit * 16;
        else unit_rows(p, p_unit, p_seg, p_row0);
    }
    auto issue = [&]() {
        if (lane == 0 && !stuck) {
            if (issued >= (uint32_t)STAGES && !mbar_wait(empty0 + p_stage * 8, p_phase ^ 1u)) stuck = true;
            else E::issue(pm, p_seg, sb0 + PARTS * p_j, p_row0, stage0 + p_stage * STAGE_BYTES, full0 + p_stage * 8, policy);
        }
        ++issued;
        if (++p_stage == STAGES) { p_stage = 0; p_phase ^= 1u; }
        if (pair && p_seg == 0) { p_seg = 1; return; }
        if (pair) p_seg = 0;
        if (++p_j == (p_item < full ? m : je)) {
            ++p_item;
            p_j = p_item < full ? 0u : jb;
            p_unit = item_unit(p_item);
            if (pair) p_row0 = p_unit * 16;
            else if (issued < total) unit_rows(p, p_unit, p_seg, p_row0);
        }
    };
    if (part == 0) {
        __syncwarp();
        for (int i = 0; i < STAGES - 1; ++i)
            if (issued < total) issue();
    }
    if (tid < 32) ((uint32_t *)zero)[tid] = 0;
    if (link.target) {
        // every block has finished the operator before (bounded: a block that never arrives raises the status word)
        if (tid == 0) {
            bool there = false;
            for (uint32_t i = 0; i < CHAIN_SPIN_LIMIT && !there; ++i) {
                there = ld_acquire_u32(link.arrivals) >= link.target;
                if (!there) __nanosleep(64);
            }
            if (!there) atomicExch(p.status, 1u);
        }
        named_barrier(15, G::THREADS);
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");  // the previous kernel has ended; its writes are visible
    }

    // ---- stage the slice's activations: a warp takes one (superblock, token) pair at a time ----
    // A pass keeps up to SBW pairs of a warp in registers between the loads and the conversion.
    // (token count: a constant of the one- and two-token instances; else a division by it is a multiplication by its
    // 16-bit reciprocal, exact for the few hundred pairs of a slice)
    const uint32_t ntok = NT <= 2 ? (uint32_t)NT : p.tokens, rtok = (65536u + ntok - 1u) / ntok;
    const uint32_t pairs = n * ntok;
    // The fused add + RMS norm: every block reads the whole rows once for their mean squares (the slice it stages is
    // not enough), block 0 also writes the sums of the add. The scratch is the part sums' memory, not in use yet:
    // [0, 32) the warps' sums, [32, 40) 1 / rms of the tokens.
    const bool normed = FOLD && p.norm_weight != nullptr;
    // One token, the whole row staged by this block, a superblock per warp at most (the gate/up pair and QKV of a 5120-wide
    // layer): the mean square comes from the values the staging pass holds in registers anyway, and the pass above it
    // over the rows is not needed.
    const bool merged = normed && NT == 1 && p.nks == 1 && pairs <= (uint32_t)WARPS;
    float *nscratch = (float *)parts;
    if (normed && !merged) {
        const uint32_t pieces = p.ksb * 64;
        for (uint32_t tok = 0; tok < ntok; ++tok) {
            const float4 *r4 = (const float4 *)(p.in + (size_t)tok * p.in_stride);
            const float4 *a4 = p.norm_input ? (const float4 *)(p.norm_input + (size_t)tok * p.in_stride) : nullptr;
            float4 *o4 = (p.residual_out && blockIdx.x == 0) ? (float4 *)(p.residual_out + (size_t)tok * p.in_stride) : nullptr;
            float sum = 0.0f;
            for (uint32_t i = tid; i < pieces; i += G::THREADS) {
                float4 v = __ldcg(r4 + i);
                if (a4) {
                    const float4 a = __ldcg(a4 + i);
                    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                }
                if (o4) o4[i] = v;
                sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) nscratch[warp] = sum;
            named_barrier(15, G::THREADS);
            if (tid == 0) {
                float total = 0.0f;
                for (int w2 = 0; w2 < WARPS; ++w2) total += nscratch[w2];
                nscratch[32 + tok] = rsqrtf(total / (float)(p.ksb * 256u) + p.norm_eps);
            }
            named_barrier(15, G::THREADS);
        }
    }
    for (uint32_t pass0 = 0; pass0 < pairs; pass0 += SBW * WARPS) {
        float4 xa[SBW], xb2[SBW];
#pragma unroll
        for (int j = 0; j < SBW; ++j) {
            const uint32_t q = pass0 + warp + j * WARPS;
            if (q < pairs) {
                const uint32_t sb = NT <= 2 ? q / ntok : (q * rtok) >> 16, tok = q - sb * ntok;
                const float4 *src = (const float4 *)(p.in + (size_t)tok * p.in_stride) + (size_t)(sb0 + sb) * 64;
                xa[j] = __ldcg(src + lane);  // L2: in a chain another block wrote them during this launch
                xb2[j] = __ldcg(src + 32 + lane);
                if (normed) {
                    const size_t col4 = (size_t)(sb0 + sb) * 64;
                    if (p.norm_input) {
                        const float4 *s2 = (const float4 *)(p.norm_input + (size_t)tok * p.in_stride) + col4;
                        const float4 a = __ldcg(s2 + lane), b = __ldcg(s2 + 32 + lane);
                        xa[j].x += a.x; xa[j].y += a.y; xa[j].z += a.z; xa[j].w += a.w;
                        xb2[j].x += b.x; xb2[j].y += b.y; xb2[j].z += b.z; xb2[j].w += b.w;
                    }
                    const float4 *wv = (const float4 *)p.norm_weight + col4;
                    const float4 wa = __ldg(wv + lane), wb = __ldg(wv + 32 + lane);
                    float r;
                    if (merged) {
                        // (one pair per warp: j == 0) the sums of the add leave from block 0, the squares meet across the warps
                        if (p.residual_out && blockIdx.x == 0) {
                            float4 *o4 = (float4 *)p.residual_out + col4;
                            o4[lane] = xa[j];
                            o4[32 + lane] = xb2[j];
                        }
                        float sum = (xa[j].x * xa[j].x + xa[j].y * xa[j].y + xa[j].z * xa[j].z + xa[j].w * xa[j].w) +
                                    (xb2[j].x * xb2[j].x + xb2[j].y * xb2[j].y + xb2[j].z * xb2[j].z + xb2[j].w * xb2[j].w);
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                        if (lane == 0) nscratch[warp] = sum;
                    }
                    if (merged) {
                        named_barrier(14, G::THREADS);  // every warp arrives here: those without a pair in the else branch below
                        float total = 0.0f;
                        for (uint32_t w2 = 0; w2 < pairs; ++w2) total += nscratch[w2];
                        r = rsqrtf(total / (float)(p.ksb * 256u) + p.norm_eps);
                    } else {
                        r = nscratch[32 + tok];
                    }
                    xa[j] = make_float4(xa[j].x * r * wa.x, xa[j].y * r * wa.y, xa[j].z * r * wa.z, xa[j].w * r * wa.w);
                    xb2[j] = make_float4(xb2[j].x * r * wb.x, xb2[j].y * r * wb.y, xb2[j].z * r * wb.z, xb2[j].w * r * wb.w);
                }
            } else if (merged && j == 0) {
                named_barrier(14, G::THREADS);  // a warp without a superblock still meets the others
            }
        }
#pragma unroll
        for (int j = 0; j < SBW; ++j) {
            const uint32_t q = pass0 + warp + j * WARPS;
            if (q < pairs) {  // uniform per warp
                const uint32_t sb = NT <= 2 ? q / ntok : (q * rtok) >> 16, tok = q - sb * ntok;
                float mx = fmaxf(fmaxf(fmaxf(fabsf(xa[j].x), fabsf(xa[j].y)), fmaxf(fabsf(xa[j].z), fabsf(xa[j].w))),
                                 fmaxf(fmaxf(fabsf(xb2[j].x), fabsf(xb2[j].y)), fmaxf(fabsf(xb2[j].z), fabsf(xb2[j].w))));
                mx = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mx)));  // (not negative: its bits order as it does)
                // 2^k puts the largest |x| in [2^21, 2^22). A row of zeros or of values below 2^-105 is staged as
                // zeros; an infinity or a NaN makes the superblock's factor a NaN, as F32 arithmetic would the sums.
                const uint32_t e = (__float_as_uint(mx) >> 23) & 0xffu;
                const bool ok = e >= 22u && e < 255u;
                const float scale = ok ? __uint_as_float((275u - e) << 23) : 0.0f;
                // the digit rows of this token: plane d is row d * TS + token (TS = 2, 4 or 8 tokens a plane)
                uint8_t *row0 = planes + (size_t)tok * p.plane_pitch + sb * 256 + lane * 4;  // byte c of a superblock's 256 is column c
                const uint32_t plane_step = TS * p.plane_pitch;
                int gsum[2];
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const float4 v = hf ? xb2[j] : xa[j];
                    // (scale is 0 when the row is not to be staged: the products are 0 or NaN, which converts to 0)
                    const int x0 = __float2int_rn(v.x * scale), x1 = __float2int_rn(v.y * scale), x2 = __float2int_rn(v.z * scale), x3 = __float2int_rn(v.w * scale);
                    gsum[hf] = (x0 + x1) + (x2 + x3);
                    // The balanced digits of x are the bytes of x + 0x808080, each less 128: with u_i those bytes,
                    // sum (u_i - 128) 256^i = x. As signed bytes, u - 128 is u ^ 0x80.
                    const uint32_t y0 = (uint32_t)x0 + 0x808080u, y1 = (uint32_t)x1 + 0x808080u, y2 = (uint32_t)x2 + 0x808080u, y3 = (uint32_t)x3 + 0x808080u;
#pragma unroll
                    for (int d = 0; d < 3; ++d) {
                        const uint32_t lo = __byte_perm(y0, y1, 0x0040 + 0x11 * d), hi = __byte_perm(y2, y3, 0x0040 + 0x11 * d);
                        *(uint32_t *)(row0 + d * plane_step + hf * 128) = __byte_perm(lo, hi, 0x5410) ^ 0x80808080u;
                    }
                }
                // group sums of X over the encoding's scale groups (exact integers below 2^27; 32 columns: eight lanes,
                // 16 columns: four), scaled to fit fp16, as pieces hi + lo
                constexpr uint32_t GLANES = E::GROUP / 4, GPER = 128 / E::GROUP;  // lanes and groups per 128 columns
#pragma unroll
                for (int hf = 0; hf < 2 && E::GROUP_SUMS; ++hf) {
                    int s = gsum[hf];
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    if (GLANES == 8) s += __shfl_xor_sync(0xffffffffu, s, 4);
                    if ((lane & (GLANES - 1)) == 0) {
                        const float f = (float)s * E::GS_SCALE;
                        const __half sh = __float2half_rn(f), sl = __float2half_rn(f - __half2float(sh));
                        const uint32_t grp = sb * (2 * GPER) + hf * GPER + lane / GLANES;
                        *(__half *)(gs + (size_t)tok * p.gs_pitch + grp * 2) = sh;
                        *(__half *)(gs + (size_t)(TS + tok) * p.gs_pitch + grp * 2) = sl;
                    }
                }
                if (lane == 0) inv[sb * 8 + tok] = ok ? __uint_as_float((e - 21u) << 23) : (e == 255u ? __uint_as_float(0x7fc00000u) : 0.0f);
            }
        }
    }
    named_barrier(15, G::THREADS);  // the staged rows, the zero block and the slots' barriers are visible to every warp

    // ---- the task loop ----
    // This lane's B column n = g. Narrow: column = plane * 2 + token, columns 6 and 7 and the columns of a
    // token that is not there read column 0 (finite integers; their sums are never used). Wide: plane d is
    // the mma d, column = token.
    const uint32_t gr = E::row(g);  // the task row this lane's mma row stands for (the encoding's shared-memory pitch decides)
    const uint8_t *xlane;
    const uint8_t *gslane;
    uint32_t gs_step;   // bytes from a lane's hi group sums to its lo group sums (wide)
    uint32_t bstep = 0; // bytes from a lane's digit row of one mma to that of the next
    if (WIDE) {
        xlane = planes + (size_t)(g < p.tokens ? g : 0u) * p.plane_pitch + t * E::LANE_BYTES;
        bstep = 8u * p.plane_pitch;
        gslane = g < p.tokens ? gs + (size_t)g * p.gs_pitch + t * 4 : zero;
        gs_step = g < p.tokens ? 8u * p.gs_pitch : 0u;
    } else if (QUAD) {
        // first mma: column g = (plane g >> 2, token g & 3); second: columns 0..3 = (plane 2, token), 4..7 unused. The
        // mma of the minima has columns (piece g >> 2, token g & 3). Columns of tokens that are not there read row 0.
        const bool there = (g & 3u) < p.tokens;
        const uint32_t row_a = there ? g : 0u, row_b = (there && g < 4) ? 8u + g : 0u;
        xlane = planes + (size_t)row_a * p.plane_pitch + t * E::LANE_BYTES;
        bstep = (row_b - row_a) * p.plane_pitch;  // (modulo 2^32: added to a pointer)
        gslane = there ? gs + (size_t)g * p.gs_pitch + t * 4 : zero;
        gs_step = 0;
    } else {
        const bool used = g < 6 && (g & 1u) < (uint32_t)NT;
        xlane = planes + (size_t)(used ? g : 0u) * p.plane_pitch + t * E::LANE_BYTES;
        // the mma of the minima has columns (piece, token): 0, 1 hi; 2, 3 lo
        const bool gs_used = g < 4 && (g & 1u) < (uint32_t)NT;
        gslane = gs_used ? gs + (size_t)g * p.gs_pitch + t * 4 : zero;
        gs_step = 0;
    }
    const uint32_t gs_sb = (gslane == zero) ? 0u : (uint32_t)E::GS_BYTES;
    // narrow: lane t holds the sums of digit plane t (weights 1, 2^8, 2^16; quad lane 3 holds nothing); E::UNIT undoes
    // a factor the encoding's integer sums carry (Q4_K: 16, the high nibbles left in place)
    // The weight of the digit plane each of the lane's mmas holds. Four tokens: quad lanes 0, 1 hold plane 0 (first mma)
    // and plane 2 (second), lanes 2, 3 plane 1 and nothing; lanes t and t ^ 2 hold the same two tokens.
    const float wl[3] = {E::UNIT * (WIDE ? 1.0f : QUAD ? (t < 2 ? 1.0f : 256.0f) : (t == 0 ? 1.0f : t == 1 ? 256.0f : t == 2 ? 65536.0f : 0.0f)),
                         E::UNIT * (WIDE ? 256.0f : (QUAD && t < 2) ? 65536.0f : 0.0f), E::UNIT * (WIDE ? 65536.0f : 0.0f)};
    const float *ivlane = inv + (WIDE ? 2 * t : QUAD ? 2 * (t & 1u) : 0);  // 1 / scale of the lane's token(s), per superblock
    uint32_t c_stage = 0, c_phase = 0, consumed = 0;
    bool failed = false;
    for (uint32_t uidx = 0; uidx < my_items; ++uidx) {
        const uint32_t unit = item_unit(uidx);
        const bool shared_unit = SHARE && uidx == full && coop > 1;  // this slot streams a share of the unit's stages
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
        // After a wait has run out the warp stops computing but still walks its units, so that the
        // warps it shares them with are not left at the barrier below.
        for (uint32_t j = uidx < full ? 0u : jb; j < (uidx < full ? m : je) && !failed; ++j) {
            const uint32_t sbw = part + PARTS * j;  // superblock within the slice: this warp's task of the stage
            const bool live = sbw < n;              // the last stage of a row may reach past the slice
            if (part == 0 && issued < total) issue();  // keep STAGES - 1 stages in flight
            if (!mbar_wait(full0 + c_stage * 8, c_phase)) { failed = true; break; }
            if (live)
                E::template task<NT>(my_stage + c_stage * STAGE_BYTES, part, xlane + sbw * 256, bstep, gslane + sbw * gs_sb, gs_step, ivlane + sbw * 8, wl, gr, t, acc);
            __syncwarp();  // all lanes are done reading this stage
            if (lane == 0) mbar_arrive(empty0 + c_stage * 8);
            ++consumed;
            if (++c_stage == STAGES) { c_stage = 0; c_phase ^= 1u; }
            if (pair) {
                if (part == 0 && issued < total) issue();
                if (!mbar_wait(full0 + c_stage * 8, c_phase)) { failed = true; break; }
                if (live)
                    E::template task<NT>(my_stage + c_stage * STAGE_BYTES, part, xlane + sbw * 256, bstep, gslane + sbw * gs_sb, gs_step, ivlane + sbw * 8, wl, gr, t, acc2);
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + c_stage * 8);
                ++consumed;
                if (++c_stage == STAGES) { c_stage = 0; c_phase ^= 1u; }
            }
        }
        // (a warp without superblocks in this slice, part >= np, holds zeros; it still meets the others below, so that
        // the warps of a slot leave the unit together: the pass after the loop counts on that)
        if (!WIDE) {
            // the quad's lanes hold the three digit planes (and the two pieces of the minima): add them
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (NT == 1 && (i & 1)) continue;
                if (!QUAD) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 1);
                acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 2);
                if (pair) {
                    if (!QUAD) acc2[i] += __shfl_xor_sync(0xffffffffu, acc2[i], 1);
                    acc2[i] += __shfl_xor_sync(0xffffffffu, acc2[i], 2);
                }
            }
        }
        // ---- the parts of the unit meet; part 0 adds them in part order ----
        const bool holds = WIDE || (QUAD ? t < 2 : t == 0);
        const uint32_t rec = WIDE ? lane : QUAD ? g * 2 + t : g;
        float4 *buf = parts + (size_t)((slot * 2 + (uidx & 1u)) * (PARTS - 1)) * (pair ? 2 : 1) * REC;
        if (part > 0 && part < np && holds) {
            float4 *dst = buf + (size_t)(part - 1) * (pair ? 2 : 1) * REC;
            dst[rec] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            if (pair) dst[REC + rec] = make_float4(acc2[0], acc2[1], acc2[2], acc2[3]);
        }
        named_barrier(1 + slot, 32 * PARTS);
        if (part != 0) continue;
        if (holds)
            for (uint32_t k = 1; k < np; ++k) {
                const float4 *src = buf + (size_t)(k - 1) * (pair ? 2 : 1) * REC;
                const float4 v = src[rec];
                acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
                if (pair) {
                    const float4 w = src[REC + rec];
                    acc2[0] += w.x; acc2[1] += w.y; acc2[2] += w.z; acc2[3] += w.w;
                }
            }
        if (shared_unit) {
            // ---- the slots that shared the unit meet (their first warps); the group's first slot adds them in slot order ----
            float4 *mine = coopbuf + (size_t)slot * (pair ? 2 : 1) * REC;
            if (ci > 0 && holds) {
                mine[rec] = make_float4(acc[0], acc[1], acc[2], acc[3]);
                if (pair) mine[REC + rec] = make_float4(acc2[0], acc2[1], acc2[2], acc2[3]);
            }
            named_barrier(9 + group, 32 * coop);
            if (ci > 0) continue;
            if (holds)
                for (uint32_t k = 1; k < coop; ++k) {
                    const float4 *src = mine + (size_t)k * (pair ? 2 : 1) * REC;
                    const float4 v = src[rec];
                    acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
                    if (pair) {
                        const float4 w = src[REC + rec];
                        acc2[0] += w.x; acc2[1] += w.y; acc2[2] += w.z; acc2[3] += w.w;
                    }
                }
        }
        if (!holds) continue;
        if (p.nks > 1) {
            // several slices: leave the partial sums; they are published after the loop with one fence
            float4 *dst = (float4 *)p.partials + ((size_t)ks * p.units + unit) * (pair ? 2 : 1) * REC;
            dst[rec] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            if (pair) dst[REC + rec] = make_float4(acc2[0], acc2[1], acc2[2], acc2[3]);
        } else {
            write_unit<NT, FOLD>(p, unit, gr, t, acc, acc2);
        }
    }
    if (p.nks > 1 && my_units) {
        // The last block to arrive for a unit adds the slices in order. The slot's first warp announces 32 units at a
        // time (one round trip for all of them); the units it was last for are then finished by all the warps of the
        // slot, one unit a warp at a time: each is a chain of dependent loads, and with eight token rows a slot has
        // several of them (one warp alone: 4.8 us for 15 units; measured).
        uint32_t *slot_mask = (uint32_t *)(smem + 640) + slot;  // (a free word behind the barriers)
        if (part == 0) {
            __threadfence();
            __syncwarp();
        }
        const bool holds = WIDE || (QUAD ? t < 2 : t == 0);
        const uint32_t rec = WIDE ? lane : QUAD ? g * 2 + t : g;
        for (uint32_t base = 0; base < my_units; base += 32) {
            if (part == 0) {
                const uint32_t mine_u = base + lane;
                uint32_t last = 0;
                if (mine_u < my_units) last = atomicAdd(p.counters + item_unit(mine_u), 1u) == p.nks - 1;
                const uint32_t found = __ballot_sync(0xffffffffu, last != 0);
                if (found) __threadfence();
                if (lane == 0) *slot_mask = found;
            }
            named_barrier(1 + slot, 32 * PARTS);
            uint32_t mask = *slot_mask;
            for (uint32_t turn = 0; mask; ++turn) {
                const uint32_t u = base + (uint32_t)__ffs((int)mask) - 1;
                mask &= mask - 1;
                if (turn % PARTS != part) continue;
                const uint32_t unit = item_unit(u);
                if (holds) {
                    const size_t per = (size_t)(pair ? 2 : 1) * REC;
                    const float4 *src = (const float4 *)p.partials + (size_t)unit * per + rec;
                    const size_t step = (size_t)p.units * per;
                    float4 s = make_float4(0.f, 0.f, 0.f, 0.f), s2 = make_float4(0.f, 0.f, 0.f, 0.f);
                    // (four loads in flight at a time; added in slice order)
                    for (uint32_t k0 = 0; k0 < p.nks; k0 += 4) {
                        float4 v[4], w[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            v[k] = k0 + k < p.nks ? __ldcg(src + (k0 + k) * step) : make_float4(0.f, 0.f, 0.f, 0.f);
                            w[k] = pair && k0 + k < p.nks ? __ldcg(src + (k0 + k) * step + REC) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            s.x += v[k].x; s.y += v[k].y; s.z += v[k].z; s.w += v[k].w;
                            s2.x += w[k].x; s2.y += w[k].y; s2.z += w[k].z; s2.w += w[k].w;
                        }
                    }
                    const float v4[4] = {s.x, s.y, s.z, s.w}, w4[4] = {s2.x, s2.y, s2.z, s2.w};
                    write_unit<NT, FOLD>(p, unit, gr, t, v4, w4);
                }
                if (lane == 0) p.counters[unit] = 0;  // leave the scratch as it was found
            }
            if (base + 32 < my_units) named_barrier(1 + slot, 32 * PARTS);  // the word is written again
        }
    }
    if (__any_sync(0xffffffffu, failed || stuck)) {
        if (lane == 0) atomicExch(p.status, 1u);
        // the slot's first warp lets the copies still in flight land before the block's shared memory is released
        if (part == 0)
            for (; consumed < issued; ++consumed) {
                mbar_wait(full0 + c_stage * 8, c_phase);
                if (++c_stage == STAGES) { c_stage = 0; c_phase ^= 1u; }
            }
    }
}

// The operator as a kernel of its own.
template <class E, class G, int NT, int STAGES, bool SHARE>
__global__ void __launch_bounds__(G::THREADS, 1) i8_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    run_op<E, G, NT, SHARE>(p, p, STAGES, smem, ChainLink{nullptr, 0u, 0u, 0u});
}

// The one-token instance with the folds.
template <class E, class G, int STAGES, bool SHARE>
__global__ void __launch_bounds__(G::THREADS, 1) i8_fold_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    run_op<E, G, 1, SHARE, true>(p, p, STAGES, smem, ChainLink{nullptr, 0u, 0u, 0u});
}

constexpr size_t kSmemMax = 227 * 1024;

struct Plan {
    int nt;       // the kernel instance: 1, 2 or 8 token columns
    int stages;
    bool share;   // the instance whose slots share the units of a block's last round
    uint32_t grid;
    size_t smem;
};

template <class E, class G, int NT>
static int pick_stages(uint32_t ksl, bool pair) {
    for (int st = kMaxStages; st >= 2; --st)
        if (smem_bytes<E, G, NT>(ksl, pair, st) <= kSmemMax) return st;
    return 0;
}

// Fills everything of Params that does not depend on the encoding's planes; the caller adds the tensor maps.
// Picks the K slices and the blocks of each slice: every candidate slice length is costed in stage
// steps of the slowest block (units over unit slots, superblocks over K parts).
template <class E, class G, int NT>
static bool fill_geometry(const FastJob &job, Params &p, Plan &plan) {
    constexpr int SLOTS = G::SLOTS, PARTS = G::PARTS;
    if (job.tokens < 1 || job.tokens > 8 || job.count < 1 || job.count > 4) return false;
    if (NT == 8 ? job.tokens < 3 : NT == 4 ? (job.tokens < 3 || job.tokens > 4) : job.tokens != (uint32_t)NT) return false;
    if (job.columns == 0 || job.columns % 256 != 0) return false;
    if ((uintptr_t)job.in % 16 != 0 || job.in_stride % 4 != 0 || job.in_stride > 0xffffffffull) return false;
    if (job.mode != ACT_NONE && (job.count != 2 || job.seg[0].rows != job.seg[1].rows)) return false;
    memset(&p, 0, sizeof p);
    p.count = job.count;
    p.mode = job.mode;
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
    const bool pair = job.mode != ACT_NONE;
    const uint32_t units = pair ? tiles / 2 : tiles;
    const double per_sb = pair ? 2.0 : 1.0;  // stages per group of superblocks of a unit
    p.units = units;
    plan.nt = NT;
    plan.share = false;
    const size_t rec_floats = (size_t)(pair ? 2 : 1) * record_lanes<NT>() * 4;  // partial sums a (slice, unit) leaves
    const uint32_t sms = (uint32_t)job.sm_count;
    double best = 1e30;
    uint32_t blocks[MAX_SLICES];
    // Measured: with six slots a block (Q6_K) sharing takes 17408 x 5120 from 19.8 to 17.4 us and the 64-layer stack from 289
    // to 297 tok/s; with four (Q4_K) it never shortened a launch (small matrices are bound by the launch, not by stage
    // steps) and its extra code cost the large ones 3 %.
    constexpr bool sharing = SLOTS >= 5;
    plan.share = sharing;
    for (uint32_t ksl = 1; ksl <= p.ksb; ++ksl) {
        const uint32_t nks = (p.ksb + ksl - 1) / ksl;
        if (nks > MAX_SLICES || nks > sms) continue;
        if (nks > 1 && ksl % PARTS != 0) continue;                        // a stage never spans two slices
        // a slicing whose partial sums or arrival counters do not fit the caller's scratch is no candidate
        if (nks > 1 && ((size_t)nks * units * rec_floats > job.partials_floats || units > job.counters_len)) continue;
        const int st = pick_stages<E, G, NT>(ksl, pair);
        if (st < 2) continue;
        // stage steps of a block with `ub` units of `st` stages each: whole rounds of SLOTS units, then a last round whose
        // units are shared by several slots each when there are few of them (the kernel's `coop`)
        auto steps = [&](uint32_t ub, uint32_t st) {
            const uint32_t whole = ub / SLOTS, rest = ub % SLOTS;
            double c = whole * (st * per_sb + 0.35);
            if (rest) {
                const uint32_t share = sharing && 2 * rest <= (uint32_t)SLOTS ? ((uint32_t)SLOTS / rest < st ? (uint32_t)SLOTS / rest : st) : 1u;
                c += (double)((st + share - 1) / share) * per_sb + 0.35 + (share > 1 ? 0.3 : 0.0);
            }
            return c;
        };
        auto cost = [&](uint32_t s, uint32_t b) {
            const uint32_t n = s + 1 == nks ? p.ksb - s * ksl : ksl, st = (n + PARTS - 1) / PARTS;
            const double hi = steps((units + b - 1) / b, st), lo = steps(units / b, st);  // blocks take one or the other
            return hi > lo ? hi : lo;
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
        // a shallow ring cannot keep the memory system busy: about 110 KB of copies in flight per multiprocessor saturate it
        const double in_flight = (double)SLOTS * (st - 1) * E::STAGE_BYTES;
        if (in_flight < 110.0 * 1024) est *= 110.0 * 1024 / in_flight;
        est += (nks > 1 ? 5.0 + 0.3 * nks : 0.0) + 0.01 * ksl * job.tokens;  // partial sums, their fence and the last arriver's pass; staging of the slice
        if (est < best - 1e-9) {
            best = est;
            p.ksl = ksl;
            p.nks = nks;
            plan.stages = st;
            uint32_t first = 0;
            for (uint32_t s = 0; s < nks; ++s) { p.blk_first[s] = first; first += blocks[s]; }
            for (uint32_t s = nks; s <= MAX_SLICES; ++s) p.blk_first[s] = first;
            plan.grid = first;
        }
    }
    if (best >= 1e30) return false;
    p.plane_pitch = p.ksl * 256 + E::PLANE_SKEW;
    p.gs_pitch = p.ksl * E::GS_BYTES + (16 + 128 - (p.ksl * E::GS_BYTES) % 128) % 128;
    plan.smem = smem_bytes<E, G, NT>(p.ksl, pair, plan.stages);
    p.partials = job.partials;
    p.counters = job.counters;
    p.status = job.counters + job.counters_len;
    p.push = job.push;
    if (p.push.ranks && (job.mode != ACT_NONE || job.count != 1 || job.tokens != 1)) return false;  // one plain matrix, one token only
    p.norm_weight = job.norm_weight;
    p.norm_input = job.norm_input;
    p.residual_out = job.residual_out;
    p.norm_eps = job.norm_eps;
    p.add0 = job.add0;
    if ((job.add0 || job.norm_weight) && NT != 1) return false;  // the folds exist in the one-token instance
    if (job.add0 && (job.count != 1 || job.mode != ACT_NONE || job.push.ranks || (uintptr_t)job.add0 % 4 != 0)) return false;  // one plain matrix, no push
    if (job.norm_weight && ((uintptr_t)job.norm_weight % 16 != 0 || (uintptr_t)job.norm_input % 16 != 0 || (uintptr_t)job.residual_out % 16 != 0)) return false;
    return true;
}

template <class E, class G, int NT, int STAGES>
static bool configure_one() {
    return cudaFuncSetAttribute(i8_kernel<E, G, NT, STAGES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax) == cudaSuccess &&
           cudaFuncSetAttribute(i8_kernel<E, G, NT, STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax) == cudaSuccess;
}
template <class E, class G, int STAGES>
static bool configure_fold() {
    return cudaFuncSetAttribute(i8_fold_kernel<E, G, STAGES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax) == cudaSuccess &&
           cudaFuncSetAttribute(i8_fold_kernel<E, G, STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax) == cudaSuccess;
}
template <class E, class G, int NT>
static bool configure_geometry() {
    if (NT == 1 && !(configure_fold<E, G, 2>() && configure_fold<E, G, 3>() && configure_fold<E, G, 4>() && configure_fold<E, G, 5>())) return false;
    return configure_one<E, G, NT, 2>() && configure_one<E, G, NT, 3>() && configure_one<E, G, NT, 4>() && configure_one<E, G, NT, 5>();
}

template <class E, class G, int NT>
static int launch_geometry(cudaStream_t s, const FastJob &job, const Params &p, const Plan &plan) {
    // launched so that it may overlap the tail of the kernel before it (see the kernel's prologue)
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(G::THREADS);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = job.serial ? 0 : 1;
    if (job.norm_weight || job.add0) {
        if (NT != 1) return 0;  // (fill_geometry has refused these)
        if (plan.share) {
            switch (plan.stages) {
            case 5: cudaLaunchKernelEx(&cfg, i8_fold_kernel<E, G, 5, true>, p); break;
            case 4: cudaLaunchKernelEx(&cfg, i8_fold_kernel<E, G, 4, true>, p); break;
            case 3: cudaLaunchKernelEx(&cfg, i8_fold_kernel<E, G, 3, true>, p); break;
            default: cudaLaunchKernelEx(&cfg, i8_fold_kernel<E, G, 2, true>, p); break;
            }
        } else {
            switch (plan.stages) {
            case 5: cudaLaunchKernelEx(&cfg, i8_fold_kernel<E, G, 5, false>, p); break;
            case 4: cudaLaunchKernelEx(&cfg, i8_fold_kernel<E, G, 4, false>, p); break;
            case 3: cudaLaunchKernelEx(&cfg, i8_fold_kernel<E, G, 3, false>, p); break;
            default: cudaLaunchKernelEx(&cfg, i8_fold_kernel<E, G, 2, false>, p); break;
            }
        }
        return 1;
    }
    if (plan.share) {
        switch (plan.stages) {
        case 5: cudaLaunchKernelEx(&cfg, i8_kernel<E, G, NT, 5, true>, p); break;
        case 4: cudaLaunchKernelEx(&cfg, i8_kernel<E, G, NT, 4, true>, p); break;
        case 3: cudaLaunchKernelEx(&cfg, i8_kernel<E, G, NT, 3, true>, p); break;
        default: cudaLaunchKernelEx(&cfg, i8_kernel<E, G, NT, 2, true>, p); break;
        }
    } else {
        switch (plan.stages) {
        case 5: cudaLaunchKernelEx(&cfg, i8_kernel<E, G, NT, 5, false>, p); break;
        case 4: cudaLaunchKernelEx(&cfg, i8_kernel<E, G, NT, 4, false>, p); break;
        case 3: cudaLaunchKernelEx(&cfg, i8_kernel<E, G, NT, 3, false>, p); break;
        default: cudaLaunchKernelEx(&cfg, i8_kernel<E, G, NT, 2, false>, p); break;
        }
    }
    return 1;
}

}  // namespace i8

// The parameters and launch plan of a job on the integer path (maps: also encode the tensor maps); false: not served.
bool q4k_i8_fill(const FastJob &job, i8::Params &p, i8::Plan &plan, bool maps);
bool q6k_i8_fill(const FastJob &job, i8::Params &p, i8::Plan &plan, bool maps);

// A uint8 tensor [rows][row_bytes] with `stride` bytes between rows, copied in boxes of box_rows x box_bytes (dispatch.cu).
bool encode_weight_map(CUtensorMap *map, const uint8_t *base, uint64_t row_bytes, uint64_t rows, uint64_t stride, uint32_t box_bytes, uint32_t box_rows);
bool encode_tiled_map(CUtensorMap *map, CUtensorMapDataType type, uint32_t elem_bytes, const void *base, uint64_t inner, uint64_t outer,
                      uint64_t stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle);

}  // namespace nu
