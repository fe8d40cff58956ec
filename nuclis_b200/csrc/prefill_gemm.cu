// Prefill GEMM for sm_100a: out[t][r] = sum_k W[r][k] * X[t][k] for many token rows, the
// weights block-quantized, the contraction on the 5th-generation tensor cores.
// Serves Backend.matmul beyond the small-batch kernels (the reference's tiles for this are
// nu_matmul_t, inference/src/backends/metal/kernels/matmul.metal:335-412: decode a K step of
// weights into a half tile in threadgroup memory, stage the activations, 8x8 MACs).
//
// One block computes a 128-row x BN-token tile of the output:
//   * warps 0..7 (256 threads: weight row tid & 127, column half tid >> 7) each decode 32 columns of
//     their row per K step to bf16 (vector decoders for 16-byte aligned Q4_K and the planar Q6_K /
//     Q8_0 forms: byte -> float through the 2^23 magic number, one FMA, packed conversion; the
//     generic per-16 decoder otherwise) and store them in shared memory in the 128-byte-swizzled
//     K-major layout the tensor core reads; the same warps later move the accumulator from tensor
//     memory to the output;
//   * warp 8 (one thread) brings the matching BN x 64 tile of bf16 activations with one TMA
//     tensor copy per K step (128-byte swizzle, so no thread touches those bytes);
//   * warp 9 (one thread) issues tcgen05.mma (M = 128, N = BN, K = 16, bf16 x bf16 -> f32) four
//     times per K step into a BN-column accumulator in tensor memory and commits to the
//     barrier that frees the stage.
// A ring of stages decouples the three. Every barrier wait is bounded; on expiry the block raises
// the status word, skips the rest of its work, still frees its tensor memory, and returns.
//
// Accuracy: weights and activations are rounded to bf16 (8 significant bits), products are exact,
// accumulation is F32: relative L2 error against the F64 reference about 3e-3 (bound 2e-2).
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstring>

#include "kernels.hpp"
#include "nu_device.cuh"

namespace nu {
namespace prefill {

constexpr int BM = 128;          // weight rows per tile = tensor-memory lanes
constexpr int BK = 64;           // columns per K step: one 128-byte swizzle row of bf16
constexpr int PRODUCER_WARPS = 8;  // decode threads: 128 rows x 2 column halves of a K step
constexpr int THREADS = (PRODUCER_WARPS + 2) * 32;  // + the TMA warp and the MMA warp
constexpr uint32_t SPIN_LIMIT = 1u << 24;

struct Params {
    CUtensorMap xmap;  // bf16 activations [tokens padded][columns], box BN rows x 64 columns, 128-byte swizzle
    const uint8_t *w;
    unsigned long long stride;
    uint32_t enc, layout;
    uint32_t fast;  // 1: the vector decoder of the encoding applies (aligned rows)
    uint32_t rows, columns, tokens;
    float *out;
    unsigned long long out_stride;
    uint32_t *status;
    // Grouped form (expert tensors): a block's token tile is one record of `tiles` ([0] the tile count, then from word 4 on
    // {expert, first gathered row, rows of the tile, first entry of the expert's slot-row list}), its weights are the
    // expert's matrix, and its output rows are scattered to the slot rows `slot_rows` names. Null: the plain form.
    const uint32_t *tiles;
    const uint32_t *slot_rows;
    unsigned long long expert_bytes;
    // Plain form with many token tiles: the grid is one-dimensional and walks `group` token tiles at a time through all
    // row tiles before it moves to the next group, so that the group's activations stay in L2 (0: the two-dimensional grid).
    uint32_t group, tok_tiles, row_tiles;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Bounded wait; also gives up at once when another thread of the block has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile in the 128-byte swizzle: rows of 128 bytes,
// groups of eight rows 1024 bytes apart. Fields: start address >> 4; leading offset (unused for this
// layout, 1); stride offset 1024 >> 4; descriptor version 1; swizzle mode 2 (128 bytes).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor, kind::f16: D f32, A and B bf16, both K-major, N and M of the instruction.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(a, b);
    return *(const uint32_t *)&pair;
}
// Byte j of w as a float, through the 2^23 magic number (one permute, one exact subtraction).
__device__ __forceinline__ float byte_f32(uint32_t w, int j) { return __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7650u + j)) - 8388608.0f; }

// Decodes columns [k0 + 16 q, + 16) of row r to bf16, as two 16-byte chunks: the generic path.
__device__ __forceinline__ void decode16_generic(const Params &p, const uint8_t *w, uint32_t r, uint32_t k0, uint32_t q, uint4 chunks[2]) {
    float v[16];
    const uint32_t seg = k0 / 16 + q;
    if (p.layout == 1) dequant16_planar_q6k(w, p.rows, p.columns / 256, r, seg, v);
    else if (p.layout == 2) dequant16_planar_q8_0(w, p.rows, p.columns, r, seg, v);
    else if (p.layout >= 3 && p.layout <= 5) dequant16_planar_block32(p.enc, w, p.rows, p.columns / 256, r, seg, v);
    else if (p.layout == 6) dequant16_planar_iq4_xs(w, p.rows, p.columns / 256, r, seg, v);
    else if (p.layout == 7) dequant16_planar_q2k(w, p.rows, p.columns / 256, r, seg, v);
    else if (p.layout == 8) dequant16_planar_q3k(w, p.rows, p.columns / 256, r, seg, v);
    else dequant16(p.enc, w + (size_t)r * p.stride, seg, v);
#pragma unroll
    for (int c = 0; c < 2; ++c)
        chunks[c] = make_uint4(pack_bf16(v[c * 8], v[c * 8 + 1]), pack_bf16(v[c * 8 + 2], v[c * 8 + 3]), pack_bf16(v[c * 8 + 4], v[c * 8 + 5]),
                               pack_bf16(v[c * 8 + 6], v[c * 8 + 7]));
}

// Four bytes of codes (one per byte of t4) -> four values (code * mul + add) as two packed bf16 pairs.
__device__ __forceinline__ void codes4_fma(uint32_t t4, float mul, float add, uint32_t &lo, uint32_t &hi) {
    lo = pack_bf16(fmaf(byte_f32(t4, 0), mul, add), fmaf(byte_f32(t4, 1), mul, add));
    hi = pack_bf16(fmaf(byte_f32(t4, 2), mul, add), fmaf(byte_f32(t4, 3), mul, add));
}
__device__ __forceinline__ uint4 ldg16(const uint8_t *ptr) { return __ldg((const uint4 *)ptr); }
// MODE: 0 the generic decoders (any encoding and layout), 1 Q4_K with 16-byte aligned rows, 2 planar Q6_K, 3 planar Q8_0,
// 4 GGUF Q8_0 rows, 5 Q5_K with 16-byte aligned rows, 6 the planar forms of Q5_0, Q5_1, Q4_0, IQ4_NL and IQ4_XS,
// 7 the planar forms of Q2_K and Q3_K, 8 GGUF rows of Q5_0, Q5_1, Q4_0 and IQ4_NL.
// BPS: blocks per SM the instance is built for (registers capped accordingly). Two blocks of two stages share an SM's
// shared and tensor memory: one block's epilogue and prologue run under the other's main loop.
template <int BN, int STAGES, int MODE, int BPS>
__global__ void __launch_bounds__(THREADS, BPS) prefill_kernel(const __grid_constant__ Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzled tiles sit on 1024-byte boundaries
    constexpr int A_BYTES = BM * BK * 2;   // 16 KiB
    constexpr int B_BYTES = BN * BK * 2;
    uint8_t *a_tiles = smem;                              // [STAGES][A_BYTES], 1024-byte aligned
    uint8_t *b_tiles = a_tiles + STAGES * A_BYTES;        // [STAGES][B_BYTES]
    uint64_t *bars = (uint64_t *)(b_tiles + STAGES * B_BYTES);
    // barriers: full_a[STAGES] (8 producer warps), full_b[STAGES] (TMA bytes), empty[STAGES] (MMA done), accum
    const uint32_t full_a = smem_u32(bars), full_b = smem_u32(bars + STAGES), empty = smem_u32(bars + 2 * STAGES), accum = smem_u32(bars + 3 * STAGES);
    uint32_t *tmem_slot = (uint32_t *)(bars + 3 * STAGES + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // token tiles vary fastest over the grid: the blocks running together share a few row tiles of weights (L2) 
    uint32_t bx = blockIdx.x, by = blockIdx.y;
    if (p.group) {
        const uint32_t per = p.group * p.row_tiles, grp = blockIdx.x / per, in = blockIdx.x - grp * per;
        const uint32_t gsize = min(p.group, p.tok_tiles - grp * p.group);  // the last group may be short
        by = in / gsize;
        bx = grp * p.group + (in - by * gsize);
    }
    const uint32_t row0 = by * BM;
    uint32_t tok0 = bx * BN, tile_rows = 0, list_first = 0;
    const uint8_t *wbase = p.w;
    if (p.tiles) {
        if (blockIdx.x >= p.tiles[0]) return;  // the grid is sized for the most tiles a routing can give; the whole block leaves
        const uint32_t *t = p.tiles + 4 + 4 * (size_t)blockIdx.x;
        wbase += (size_t)t[0] * p.expert_bytes;
        tok0 = t[1];
        tile_rows = t[2];
        list_first = t[3];
    }
    const uint32_t ksteps = p.columns / BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_a + s * 8, PRODUCER_WARPS);
            mbar_init(full_b + s * 8, 1);
            mbar_init(empty + s * 8, 1);
        }
        mbar_init(accum, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == PRODUCER_WARPS + 1) {
        // tensor memory: BN columns of 128 lanes of f32, allocated and later freed by this warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp < PRODUCER_WARPS) {
        // ---- decode producers: warp w owns weight rows 16 w .. 16 w + 15 of the tile, lane l row l & 15 and
        // piece l >> 4: the two lanes of a row read adjacent bytes (a warp-wide load touches 16 short runs
        // instead of 32 scattered 16-byte pieces: the load/store unit, not arithmetic, bounds this warp).
        // The bytes of a step are requested one step ahead of their use, so that the latency of the loads
        // hides behind the decoding of the step before; pointers advance, nothing is recomputed per step.
        const uint32_t r = warp * 16 + (lane & 15u), piece = lane >> 4;
        const uint32_t grow = min(row0 + r, p.rows - 1);  // rows past the matrix repeat the last one; never stored
        uint8_t *arow = a_tiles + (r >> 3) * 1024 + (r & 7) * 128;
        bool ok = true;
        uint32_t s = 0, round = 0;
        // Stores four 16-byte chunks of a step (chunk positions pos[0..3] of the row's eight) into the
        // stage's swizzled tile and hands the stage over.
        auto put = [&](const uint4 (&chunks)[4], uint32_t pos0, uint32_t pos1) -> bool {
            if (round && !mbar_wait(empty + s * 8, (round - 1) & 1u, abort_flag)) return false;
            uint8_t *dst = arow + s * A_BYTES;
            *(uint4 *)(dst + ((pos0 ^ (r & 7)) * 16)) = chunks[0];
            *(uint4 *)(dst + (((pos0 + 1) ^ (r & 7)) * 16)) = chunks[1];
            *(uint4 *)(dst + ((pos1 ^ (r & 7)) * 16)) = chunks[2];
            *(uint4 *)(dst + (((pos1 + 1) ^ (r & 7)) * 16)) = chunks[3];
            // make the generic-proxy stores visible to the tensor core's reads, then one arrival per warp
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(full_a + s * 8);
            if (++s == STAGES) { s = 0; ++round; }
            return true;
        };
        if (MODE == 1 || MODE == 5) {
            // Q4_K: a K step is one group pair of a superblock: 32 quant bytes whose low nibbles are the even
            // group (columns 0..31 of the step) and high nibbles the odd group (columns 32..63). Piece p holds
            // bytes 16 p .. 16 p + 15: columns 16 p .. + 15 of both groups. Values are (d*s)*q - dmin*m with one
            // rounding, like the reference decoder (inference/src/quant/decode.zig:147-170), then rounded to bf16.
            // Q5_K (MODE 5): 32 bytes of fifth bits sit between the header and the nibbles; bit g of byte c belongs to
            // column c of group g, so the piece's 16 bytes of them serve all four K steps of the superblock.
            constexpr bool FIFTH = MODE == 5;
            constexpr int SB_BYTES = FIFTH ? 176 : 144, QS = FIFTH ? 48 : 16;
            const uint8_t *blk = wbase + (size_t)grow * p.stride;
            const uint32_t nsb = p.columns / 256;
            // the five (six) 16-byte loads of a superblock are requested a whole superblock (four K steps) ahead
            uint4 hdr_n = ldg16(blk), q_n[4], f_n = make_uint4(0u, 0u, 0u, 0u);
            if (FIFTH) f_n = ldg16(blk + 16 + piece * 16);
#pragma unroll
            for (int j = 0; j < 4; ++j) q_n[j] = ldg16(blk + QS + j * 32 + piece * 16);
            for (uint32_t sb = 0; sb < nsb && ok; ++sb, blk += SB_BYTES) {
                const uint4 hdr = hdr_n, fifth = f_n;
                uint4 q_c[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) q_c[j] = q_n[j];
                if (sb + 1 < nsb) {
                    hdr_n = ldg16(blk + SB_BYTES);
                    if (FIFTH) f_n = ldg16(blk + SB_BYTES + 16 + piece * 16);
#pragma unroll
                    for (int j = 0; j < 4; ++j) q_n[j] = ldg16(blk + SB_BYTES + QS + j * 32 + piece * 16);
                }
                const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu))), dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 qq = q_c[j];
                    // six-bit scales and minima of groups 2j and 2j+1 out of the 12 packed bytes (words hdr.y, hdr.z, hdr.w)
                    float ds[2], ndm[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int sh = 8 * (2 * (j & 1) + e);
                        const uint32_t y = (hdr.y >> sh) & 0xffu, z = (hdr.z >> sh) & 0xffu, w = (hdr.w >> sh) & 0xffu;
                        const uint32_t s6 = j < 2 ? (y & 63u) : ((w & 15u) | ((y >> 6) << 4));
                        const uint32_t m6 = j < 2 ? (z & 63u) : ((w >> 4) | ((z >> 6) << 4));
                        ds[e] = __fmul_rn(d, (float)s6);
                        ndm[e] = -__fmul_rn(dmin, (float)m6);
                    }
                    const uint32_t words[4] = {qq.x, qq.y, qq.z, qq.w};
                    const uint32_t fw[4] = {fifth.x, fifth.y, fifth.z, fifth.w};
                    uint32_t even[4], odd[4];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        even[m] = words[m] & 0x0f0f0f0fu;
                        odd[m] = (words[m] >> 4) & 0x0f0f0f0fu;
                        if (FIFTH) {
                            even[m] |= (j < 2 ? fw[m] << (4 - 2 * j) : fw[m] >> (2 * j - 4)) & 0x10101010u;  // bit 2j of each byte to bit 4
                            odd[m] |= (j < 2 ? fw[m] << (3 - 2 * j) : fw[m] >> (2 * j - 3)) & 0x10101010u;   // bit 2j + 1
                        }
                    }
                    uint4 chunks[4];  // 0, 1: the even group's 16 columns; 2, 3: the odd group's
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        codes4_fma(even[c * 2], ds[0], ndm[0], chunks[c].x, chunks[c].y);
                        codes4_fma(even[c * 2 + 1], ds[0], ndm[0], chunks[c].z, chunks[c].w);
                        codes4_fma(odd[c * 2], ds[1], ndm[1], chunks[2 + c].x, chunks[2 + c].y);
                        codes4_fma(odd[c * 2 + 1], ds[1], ndm[1], chunks[2 + c].z, chunks[2 + c].w);
                    }
                    ok = put(chunks, piece * 2, 4 + piece * 2);
                    if (!ok) break;
                }
            }
        } else if (MODE == 2) {
            // Planar Q6_K (prepare.cu): K step j of a superblock holds 32-column runs 2j and 2j+1: quarters
            // 2 (j & 1) and 2 (j & 1) + 1 of half j >> 1. Piece ch is the planar chunk of column half ch: 16
            // columns of each run, one scale each; its 48 bytes serve two K steps (low nibbles: quarters 0, 1;
            // high nibbles: quarters 2, 3). Value = (d * scale) * (code - 32), exact.
            const uint32_t nsb = p.columns / 256;
            const uint8_t *rec = wbase + (size_t)grow * nsb * 208;
            const uint8_t *dp = wbase + (size_t)p.rows * nsb * 208 + (size_t)grow * 2;
            const size_t dstep = (size_t)p.rows * 2;
            // the loads of a superblock (two chunks of 48 bytes, 16 scale bytes, the super-scale) are requested a
            // whole superblock (four K steps) ahead
            uint4 raw_n[2][3];
            uint2 sc_n[2];  // the 8 scales of each half: bytes qr * 2 + ch
            auto fetch = [&](const uint8_t *record) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const uint8_t *chunk = record + (hh * 2 + piece) * 48;
                    raw_n[hh][0] = ldg16(chunk);
                    raw_n[hh][1] = ldg16(chunk + 16);
                    raw_n[hh][2] = ldg16(chunk + 32);
                    sc_n[hh] = *(const uint2 *)(record + 192 + hh * 8);
                }
            };
            fetch(rec);
            float d_n = __half2float(*(const __half *)dp);
            for (uint32_t sb = 0; sb < nsb && ok; ++sb, rec += 208) {
                const float d = d_n;
                uint4 raw_c[2][3];
                uint2 sc_c[2];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    raw_c[hh][0] = raw_n[hh][0]; raw_c[hh][1] = raw_n[hh][1]; raw_c[hh][2] = raw_n[hh][2];
                    sc_c[hh] = sc_n[hh];
                }
                if (sb + 1 < nsb) {
                    dp += dstep;
                    d_n = __half2float(*(const __half *)dp);
                    fetch(rec + 208);
                }
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const uint4 qla = raw_c[hh][0], qlb = raw_c[hh][1], qh = raw_c[hh][2];
                    const uint2 scs = sc_c[hh];
                    const uint32_t hw[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {  // K step 2 hh + jj: quarters 2 jj and 2 jj + 1
                        uint4 chunks[4];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int qr = 2 * jj + e;
                            const uint4 ql = e ? qlb : qla;
                            const uint32_t scw = qr < 2 ? scs.x : scs.y;
                            const float ds = __fmul_rn(d, (float)(int8_t)((scw >> (8 * ((qr & 1) * 2 + (int)piece))) & 0xffu));
                            const float bias = -32.0f * ds;  // exact: a power of two times ds
                            const uint32_t lw[4] = {ql.x, ql.y, ql.z, ql.w};
                            uint32_t packed[8];
#pragma unroll
                            for (int m = 0; m < 4; ++m) {
                                const uint32_t nib = (jj ? (lw[m] >> 4) : lw[m]) & 0x0f0f0f0fu;  // quarters 2, 3: high nibbles
                                const uint32_t top = ((hw[m] >> (2 * qr)) & 0x03030303u) << 4;
                                codes4_fma(nib | top, ds, bias, packed[m * 2], packed[m * 2 + 1]);
                            }
                            chunks[e * 2] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                            chunks[e * 2 + 1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        }
                        ok = put(chunks, piece * 2, 4 + piece * 2);
                        if (!ok) break;
                    }
                    if (!ok) break;
                }
            }
        } else if (MODE == 3) {
            // Planar Q8_0 (prepare.cu): 32 columns are one block; value = d * code, exact before the bf16 rounding.
            const uint8_t *q = wbase + (size_t)grow * p.columns + piece * 32;
            const uint8_t *dp = wbase + (size_t)p.rows * p.columns + ((size_t)piece * p.rows + grow) * 2;
            const size_t dstep = (size_t)p.rows * 4;  // two blocks per K step
            uint4 qa_n = ldg16(q), qb_n = ldg16(q + 16);
            float d_n = __half2float(*(const __half *)dp);
            for (uint32_t k = 0; k < ksteps && ok; ++k) {
                const uint4 qa = qa_n, qb = qb_n;
                const float d = d_n, bias = -128.0f * d_n;
                if (k + 1 < ksteps) {
                    q += BK; dp += dstep;
                    qa_n = ldg16(q); qb_n = ldg16(q + 16);
                    d_n = __half2float(*(const __half *)dp);
                }
                const uint32_t words[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                uint4 chunks[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    codes4_fma(words[c * 2] ^ 0x80808080u, d, bias, chunks[c].x, chunks[c].y);  // (code + 128) * d - 128 d
                    codes4_fma(words[c * 2 + 1] ^ 0x80808080u, d, bias, chunks[c].z, chunks[c].w);
                }
                ok = put(chunks, piece * 4, piece * 4 + 2);
            }
        } else if (MODE == 4) {
            // GGUF Q8_0 rows (34-byte blocks: an f16 scale, 32 codes; blocks start on 2-byte boundaries only). Piece p takes
            // block p of the K step. The codes are fetched as aligned 32-bit words around them and shifted into place
            // (the offset within a word is 0 or 2 bytes); an aligned word never reaches past a buffer whose size is a multiple
            // of four, and the word beyond the codes is only read when the shift needs it.
            const uint8_t *blk = wbase + (size_t)grow * p.stride + piece * 34;
            auto fetch = [&](const uint8_t *b, uint32_t (&w)[9], float &d) {
                d = __half2float(*(const __half *)b);
                const uintptr_t cp = (uintptr_t)(b + 2);
                const uint32_t *base = (const uint32_t *)(cp & ~(uintptr_t)3);
#pragma unroll
                for (int j = 0; j < 8; ++j) w[j] = __ldg(base + j);
                w[8] = (cp & 2) ? __ldg(base + 8) : 0u;
            };
            uint32_t w_n[9];
            float d_n;
            fetch(blk, w_n, d_n);
            for (uint32_t k = 0; k < ksteps && ok; ++k) {
                uint32_t w_c[9];
#pragma unroll
                for (int j = 0; j < 9; ++j) w_c[j] = w_n[j];
                const float d = d_n, bias = -128.0f * d_n;
                const uint32_t sh = (((uintptr_t)(blk + 2)) & 2) ? 16u : 0u;
                if (k + 1 < ksteps) {
                    blk += 68;
                    fetch(blk, w_n, d_n);
                }
                uint4 chunks[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t c0 = __funnelshift_r(w_c[c * 2], w_c[c * 2 + 1], sh), c1 = __funnelshift_r(w_c[c * 2 + 1], w_c[c * 2 + 2], sh);
                    codes4_fma(c0 ^ 0x80808080u, d, bias, chunks[c].x, chunks[c].y);  // (code + 128) * d - 128 d
                    codes4_fma(c1 ^ 0x80808080u, d, bias, chunks[c].z, chunks[c].w);
                }
                ok = put(chunks, piece * 4, piece * 4 + 2);
            }
        } else if (MODE == 6) {
            // The planar forms of the 32-element block encodings (prepare.cu, layouts 3..6: Q5_0, Q5_1, Q4_0, IQ4_NL, IQ4_XS):
            // piece p takes block 2k + p of K step k: 16 nibble bytes (low nibbles: columns 0..15 of the block, high: 16..31),
            // for Q5_0 / Q5_1 a 32-bit plane of fifth bits, and its scale(s) from the second plane. Every value is
            // code * mul + add with one rounding: the exact value the reference decoder rounds
            // (inference/src/quant/decode.zig:46-53, 73-81, 125-143, 214-228), then rounded to bf16.
            const uint32_t enc = p.enc, nsb = p.columns / 256;
            const bool fifth = enc == Q5_0 || enc == Q5_1, table = enc == IQ4_NL || enc == IQ4_XS;
            const uint32_t record = fifth ? 160u : 128u, sc_row = enc == Q5_1 ? 32u : enc == IQ4_XS ? 8u : 16u;
            const uint8_t *rec = wbase + (size_t)grow * nsb * record;
            const uint8_t *sc = wbase + (size_t)p.rows * nsb * record + (size_t)grow * sc_row;
            const size_t sc_step = (size_t)p.rows * sc_row;
            struct Raw { uint4 nib; uint32_t high; uint32_t d, m; uint2 hdr; };
            auto fetch = [&](uint32_t k) {
                const uint32_t sb = k >> 2, c = 2 * (k & 3u) + piece;
                const uint8_t *r8 = rec + (size_t)sb * record, *s8 = sc + (size_t)sb * sc_step;
                Raw raw;
                raw.nib = ldg16(r8 + c * 16);
                raw.high = fifth ? __ldg((const uint32_t *)(r8 + 128 + c * 4)) : 0u;
                raw.hdr = make_uint2(0u, 0u);
                raw.d = raw.m = 0;
                if (enc == IQ4_XS) raw.hdr = __ldg((const uint2 *)s8);
                else raw.d = __ldg((const unsigned short *)(s8 + c * 2));
                if (enc == Q5_1) raw.m = __ldg((const unsigned short *)(s8 + 16 + c * 2));
                return raw;
            };
            Raw next = fetch(0);
            for (uint32_t k = 0; k < ksteps && ok; ++k) {
                const Raw raw = next;
                if (k + 1 < ksteps) next = fetch(k + 1);
                float mul, add;
                if (enc == IQ4_XS) {
                    const uint32_t c = 2 * (k & 3u) + piece;
                    const int scale = (int)(((raw.hdr.y >> (4 * c)) & 15u) | (((raw.hdr.x >> (16 + 2 * c)) & 3u) << 4)) - 32;
                    mul = __fmul_rn(__half2float(__ushort_as_half((unsigned short)(raw.hdr.x & 0xffffu))), (float)scale);
                    add = -128.0f * mul;
                } else {
                    mul = __half2float(__ushort_as_half((unsigned short)raw.d));
                    add = enc == Q5_1 ? __half2float(__ushort_as_half((unsigned short)raw.m)) : enc == Q5_0 ? -16.0f * mul : enc == Q4_0 ? -8.0f * mul : -128.0f * mul;
                }
                const uint32_t nw[4] = {raw.nib.x, raw.nib.y, raw.nib.z, raw.nib.w};
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    if (table) {
                        // the table values of the nibbles of each half-word come out in nibble order: (lo0, hi0, lo1, hi1), (lo2, hi2, lo3, hi3)
                        const uint32_t a = iq4_lookup4(nw[m]), b = iq4_lookup4(nw[m] >> 16);
                        lo[m] = __byte_perm(a, b, 0x6420) ^ 0x80808080u;  // signed bytes biased to 0..255; the bias leaves through `add`
                        hi[m] = __byte_perm(a, b, 0x7531) ^ 0x80808080u;
                    } else {
                        lo[m] = nw[m] & 0x0f0f0f0fu;
                        hi[m] = (nw[m] >> 4) & 0x0f0f0f0fu;
                        if (fifth) {
                            lo[m] |= bits4_to_bit4((raw.high >> (4 * m)) & 15u);
                            hi[m] |= bits4_to_bit4((raw.high >> (16 + 4 * m)) & 15u);
                        }
                    }
                }
                uint4 chunks[4];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    codes4_fma(lo[c * 2], mul, add, chunks[c].x, chunks[c].y);
                    codes4_fma(lo[c * 2 + 1], mul, add, chunks[c].z, chunks[c].w);
                    codes4_fma(hi[c * 2], mul, add, chunks[2 + c].x, chunks[2 + c].y);
                    codes4_fma(hi[c * 2 + 1], mul, add, chunks[2 + c].z, chunks[2 + c].w);
                }
                ok = put(chunks, piece * 4, piece * 4 + 2);
            }
        } else if (MODE == 8) {
            // GGUF rows of Q5_0, Q5_1, Q4_0 and IQ4_NL (blocks of 22, 24 and 18 bytes on 2-byte boundaries): what an expert
            // tensor, which is never re-laid, is read as. Piece p takes block 2k + p of K step k. As for GGUF Q8_0 rows the
            // block is fetched as the aligned 32-bit words around it and shifted into place; a word that only holds bytes
            // past the block is read only when the shift needs it. The values are those of MODE 6.
            const uint32_t enc = p.enc;
            const bool fifth = enc == Q5_0 || enc == Q5_1, table = enc == IQ4_NL;
            const uint32_t bs = enc == Q5_0 ? 22u : enc == Q5_1 ? 24u : 18u;
            const uint8_t *blk = wbase + (size_t)grow * p.stride + piece * bs;
            struct Raw { uint32_t w[7]; uint32_t sh; };
            auto fetch = [&](const uint8_t *b8) {
                Raw raw;
                const uintptr_t at = (uintptr_t)b8;
                const uint32_t *base = (const uint32_t *)(at & ~(uintptr_t)3);
                raw.sh = (at & 2) ? 16u : 0u;
                const uint32_t need = (bs + (raw.sh ? 2u : 0u) + 3u) / 4u;  // words that hold bytes of the block
#pragma unroll
                for (int i = 0; i < 7; ++i) raw.w[i] = (uint32_t)i < need ? __ldg(base + i) : 0u;
                return raw;
            };
            Raw next = fetch(blk);
            for (uint32_t k = 0; k < ksteps && ok; ++k) {
                const Raw raw = next;
                if (k + 1 < ksteps) {
                    blk += 2 * bs;
                    next = fetch(blk);
                }
                uint32_t f[6];  // the block's bytes from its start, as words
#pragma unroll
                for (int i = 0; i < 6; ++i) f[i] = __funnelshift_r(raw.w[i], raw.w[i + 1], raw.sh);
                const float mul = __half2float(__ushort_as_half((unsigned short)(f[0] & 0xffffu)));
                const float add = enc == Q5_1 ? __half2float(__ushort_as_half((unsigned short)(f[0] >> 16))) : enc == Q5_0 ? -16.0f * mul : enc == Q4_0 ? -8.0f * mul : -128.0f * mul;
                const uint32_t high = enc == Q5_0 ? __funnelshift_r(f[0], f[1], 16) : f[1];  // bytes 2..5 (Q5_0) or 4..7 (Q5_1)
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    // the nibble bytes start at byte 6, 8 or 2 of the block
                    const uint32_t q = enc == Q5_0 ? __funnelshift_r(f[1 + m], f[2 + m], 16) : enc == Q5_1 ? f[2 + m] : __funnelshift_r(f[m], f[1 + m], 16);
                    if (table) {
                        const uint32_t a = iq4_lookup4(q), b = iq4_lookup4(q >> 16);
                        lo[m] = __byte_perm(a, b, 0x6420) ^ 0x80808080u;
                        hi[m] = __byte_perm(a, b, 0x7531) ^ 0x80808080u;
                    } else {
                        lo[m] = q & 0x0f0f0f0fu;
                        hi[m] = (q >> 4) & 0x0f0f0f0fu;
                        if (fifth) {
                            lo[m] |= bits4_to_bit4((high >> (4 * m)) & 15u);
                            hi[m] |= bits4_to_bit4((high >> (16 + 4 * m)) & 15u);
                        }
                    }
                }
                uint4 chunks[4];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    codes4_fma(lo[c * 2], mul, add, chunks[c].x, chunks[c].y);
                    codes4_fma(lo[c * 2 + 1], mul, add, chunks[c].z, chunks[c].w);
                    codes4_fma(hi[c * 2], mul, add, chunks[2 + c].x, chunks[2 + c].y);
                    codes4_fma(hi[c * 2 + 1], mul, add, chunks[2 + c].z, chunks[2 + c].w);
                }
                ok = put(chunks, piece * 4, piece * 4 + 2);
            }
        } else if (MODE == 7) {
            // The planar forms of Q2_K and Q3_K (prepare.cu, layouts 7 and 8). K step s of a superblock is the two-bit fields
            // 2 (s & 1) and 2 (s & 1) + 1 of the 32 code bytes of half s >> 1; piece p takes field j = 2 (s & 1) + p: 32
            // columns, groups 8 (s >> 1) + 2 j and the next. Q2_K: value = (d * scale) * code - dmin * minimum; Q3_K: the third
            // bit of a code is bit 4 (s >> 1) + j of the 32 mask bytes, value = (d * (scale - 32)) * (code - 4). One
            // rounding each, the value the reference decoder rounds (inference/src/quant/decode.zig:174-196, 260-275).
            const bool q3 = p.enc == Q3_K;
            const uint32_t nsb = p.columns / 256, record = q3 ? 96u : 80u, codes_at = q3 ? 32u : 16u;
            const uint8_t *rec = wbase + (size_t)grow * nsb * record;
            const uint8_t *tail = wbase + (size_t)p.rows * nsb * record + (q3 ? (size_t)(grow / 16) * 224 : (size_t)grow * 4);
            const size_t tail_step = q3 ? (size_t)(p.rows / 16) * 224 : (size_t)p.rows * 4;
            struct Raw { uint4 qa, qb, ma, mb; };
            auto fetch = [&](uint32_t k) {
                const uint8_t *r8 = rec + (size_t)(k >> 2) * record;
                Raw raw;
                raw.qa = ldg16(r8 + codes_at + ((k >> 1) & 1u) * 32);
                raw.qb = ldg16(r8 + codes_at + ((k >> 1) & 1u) * 32 + 16);
                raw.ma = raw.mb = make_uint4(0u, 0u, 0u, 0u);
                if (q3) { raw.ma = ldg16(r8); raw.mb = ldg16(r8 + 16); }
                return raw;
            };
            Raw next = fetch(0);
            uint32_t sw[4] = {0u, 0u, 0u, 0u};  // the scale bytes of the row's superblock: 16 (Q2_K) or 12 (Q3_K)
            float d = 0.0f, dmin = 0.0f;
            for (uint32_t k = 0; k < ksteps && ok; ++k) {
                const Raw raw = next;
                if (k + 1 < ksteps) next = fetch(k + 1);
                if ((k & 3u) == 0) {
                    const uint8_t *t8 = tail + (size_t)(k >> 2) * tail_step;
                    if (q3) {
                        const uint32_t *sc = (const uint32_t *)(t8 + (grow % 16) * 12);
                        sw[0] = __ldg(sc); sw[1] = __ldg(sc + 1); sw[2] = __ldg(sc + 2);
                        d = __half2float(__ushort_as_half(__ldg((const unsigned short *)(t8 + 192 + (grow % 16) * 2))));
                    } else {
                        const uint4 sc = ldg16(rec + (size_t)(k >> 2) * record);
                        sw[0] = sc.x; sw[1] = sc.y; sw[2] = sc.z; sw[3] = sc.w;
                        const uint32_t dd = __ldg((const uint32_t *)t8);
                        d = __half2float(__ushort_as_half((unsigned short)(dd & 0xffffu)));
                        dmin = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
                    }
                }
                const uint32_t n = (k >> 1) & 1u, j = 2 * (k & 1u) + piece, g0 = 8 * n + 2 * j;
                float mul[2], add[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t g = g0 + e;
                    if (q3) {
                        const uint32_t lowb = ((((g & 7u) >> 2) ? sw[1] : sw[0]) >> (8 * (g & 3u))) & 0xffu, nibble = g < 8 ? (lowb & 15u) : (lowb >> 4);
                        const uint32_t upper = (sw[2] >> (8 * (g & 3u) + 2 * (g >> 2))) & 3u;
                        mul[e] = __fmul_rn(d, (float)((int)(nibble | (upper << 4)) - 32));
                        add[e] = -4.0f * mul[e];
                    } else {
                        const uint32_t wsel = (g >> 2) == 0 ? sw[0] : (g >> 2) == 1 ? sw[1] : (g >> 2) == 2 ? sw[2] : sw[3];  // selects: the words stay in registers
                        const uint32_t b = (wsel >> (8 * (g & 3u))) & 0xffu;
                        mul[e] = __fmul_rn(d, (float)(b & 15u));
                        add[e] = -__fmul_rn(dmin, (float)(b >> 4));
                    }
                }
                const uint32_t qw[8] = {raw.qa.x, raw.qa.y, raw.qa.z, raw.qa.w, raw.qb.x, raw.qb.y, raw.qb.z, raw.qb.w};
                const uint32_t mw[8] = {raw.ma.x, raw.ma.y, raw.ma.z, raw.ma.w, raw.mb.x, raw.mb.y, raw.mb.z, raw.mb.w};
                const uint32_t bit = 4 * n + j;
                uint32_t codes[8];
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    codes[m] = (qw[m] >> (2 * j)) & 0x03030303u;
                    if (q3) codes[m] |= ((mw[m] >> bit) & 0x01010101u) << 2;
                }
                uint4 chunks[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    codes4_fma(codes[c * 2], mul[c >> 1], add[c >> 1], chunks[c].x, chunks[c].y);
                    codes4_fma(codes[c * 2 + 1], mul[c >> 1], add[c >> 1], chunks[c].z, chunks[c].w);
                }
                ok = put(chunks, piece * 4, piece * 4 + 2);
            }
        } else {
            for (uint32_t k = 0; k < ksteps && ok; ++k) {
                uint4 chunks[4];
                decode16_generic(p, wbase, grow, k * BK, piece * 2, &chunks[0]);
                decode16_generic(p, wbase, grow, k * BK, piece * 2 + 1, &chunks[2]);
                ok = put(chunks, piece * 4, piece * 4 + 2);
            }
        }
        // ---- epilogue: tensor memory -> output; warp w reads lanes 32 (w & 3) .. + 31 (its rows), half of the columns ----
        if (ok) ok = mbar_wait(accum, 0, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const uint32_t half = warp >> 2;
            const uint32_t out_row = row0 + (warp & 3u) * 32 + lane;
#pragma unroll 1
            for (int c0 = (int)half * (BN / 2); c0 < (int)(half + 1) * (BN / 2); c0 += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem + (((warp & 3u) * 32u) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (out_row < p.rows) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (p.tiles) {
                            if ((uint32_t)(c0 + j) < tile_rows) p.out[(size_t)p.slot_rows[list_first + c0 + j] * p.out_stride + out_row] = __uint_as_float(v[j]);
                        } else {
                            const uint32_t tok = tok0 + c0 + j;
                            if (tok < p.tokens) p.out[(size_t)tok * p.out_stride + out_row] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    } else if (warp == PRODUCER_WARPS) {
        // ---- activation tiles by TMA ----
        if (lane == 0) {
            bool ok = true;
            uint32_t issued = 0;
            for (uint32_t k = 0; k < ksteps && ok; ++k) {
                const uint32_t s = k % STAGES;
                if (k >= STAGES) ok = mbar_wait(empty + s * 8, ((k / STAGES) - 1) & 1u, abort_flag);
                if (!ok) break;
                mbar_expect_tx(full_b + s * 8, B_BYTES);
                tma_load_2d(smem_u32(b_tiles + s * B_BYTES), &p.xmap, k * BK, tok0, full_b + s * 8);
                ++issued;
            }
            if (*abort_flag) {
                // giving up: let the copies still in flight land before the block's shared memory is released
                for (uint32_t k = issued > STAGES ? issued - STAGES : 0; k < issued; ++k)
                    for (uint32_t i = 0; i < SPIN_LIMIT && !mbar_try_wait(full_b + (k % STAGES) * 8, (k / STAGES) & 1u); ++i) {}
            }
        }
    } else {
        // ---- the MMA thread ----
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BM, BN);
            bool ok = true;
            for (uint32_t k = 0; k < ksteps && ok; ++k) {
                const uint32_t s = k % STAGES, parity = (k / STAGES) & 1u;
                ok = mbar_wait(full_a + s * 8, parity, abort_flag) && mbar_wait(full_b + s * 8, parity, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(a_tiles + s * A_BYTES), b_addr = smem_u32(b_tiles + s * B_BYTES);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk)  // 16 columns = 32 bytes further along the swizzled row
                    mma_bf16(tmem, smem_desc(a_addr + kk * 32), smem_desc(b_addr + kk * 32), idesc, (k | kk) != 0);
                mma_commit(empty + s * 8);  // frees the stage when these MMAs have read it
            }
            if (ok) mma_commit(accum);
        }
    }
    __syncthreads();
    if (warp == PRODUCER_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)BN) : "memory");
    }
    if (tid == 0 && *abort_flag) atomicExch(p.status, 1u);
}

template <int BN, int STAGES> constexpr int smem_bytes() { return STAGES * (BM * BK * 2 + BN * BK * 2) + (3 * STAGES + 1) * 8 + 16 + 1024; }

}  // namespace prefill

bool encode_tiled_map(CUtensorMap *map, CUtensorMapDataType type, uint32_t elem_bytes, const void *base, uint64_t inner, uint64_t outer,
                      uint64_t stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle);

template <int BN, int STAGES, int MODE, int BPS>
static bool configure_one() {
    return cudaFuncSetAttribute(prefill::prefill_kernel<BN, STAGES, MODE, BPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, prefill::smem_bytes<BN, STAGES>()) == cudaSuccess;
}
template <int BN, int STAGES, int BPS>
static bool configure_bn() {
    return configure_one<BN, STAGES, 0, BPS>() && configure_one<BN, STAGES, 1, BPS>() && configure_one<BN, STAGES, 2, BPS>() && configure_one<BN, STAGES, 3, BPS>() &&
           configure_one<BN, STAGES, 4, BPS>() && configure_one<BN, STAGES, 5, BPS>() && configure_one<BN, STAGES, 6, BPS>() &&
           configure_one<BN, STAGES, 7, BPS>() && configure_one<BN, STAGES, 8, BPS>();
}

bool prefill_configure() { return configure_bn<256, 4, 1>() && configure_bn<256, 2, 2>() && configure_bn<128, 6, 1>() && configure_bn<64, 8, 1>() && configure_bn<64, 4, 2>(); }

static uint32_t pick_bn(uint32_t tokens) { return tokens > 128 ? 256 : tokens > 64 ? 128 : 64; }

template <int BN, int STAGES, int BPS>
static void launch_bn(dim3 grid, cudaStream_t s, const prefill::Params &p, int mode) {
    const int bytes = prefill::smem_bytes<BN, STAGES>();
    switch (mode) {
    case 1: prefill::prefill_kernel<BN, STAGES, 1, BPS><<<grid, prefill::THREADS, bytes, s>>>(p); break;
    case 2: prefill::prefill_kernel<BN, STAGES, 2, BPS><<<grid, prefill::THREADS, bytes, s>>>(p); break;
    case 3: prefill::prefill_kernel<BN, STAGES, 3, BPS><<<grid, prefill::THREADS, bytes, s>>>(p); break;
    case 4: prefill::prefill_kernel<BN, STAGES, 4, BPS><<<grid, prefill::THREADS, bytes, s>>>(p); break;
    case 5: prefill::prefill_kernel<BN, STAGES, 5, BPS><<<grid, prefill::THREADS, bytes, s>>>(p); break;
    case 6: prefill::prefill_kernel<BN, STAGES, 6, BPS><<<grid, prefill::THREADS, bytes, s>>>(p); break;
    case 7: prefill::prefill_kernel<BN, STAGES, 7, BPS><<<grid, prefill::THREADS, bytes, s>>>(p); break;
    case 8: prefill::prefill_kernel<BN, STAGES, 8, BPS><<<grid, prefill::THREADS, bytes, s>>>(p); break;
    default: prefill::prefill_kernel<BN, STAGES, 0, BPS><<<grid, prefill::THREADS, bytes, s>>>(p); break;
    }
}

bool prefill_supported(const PrefillJob &j) {
    if (layout(j.enc).elements == 0 || j.rows == 0 || j.tokens == 0) return false;
    if (j.columns == 0 || j.columns % 64 != 0) return false;
    if ((uintptr_t)j.in % 16 != 0 || j.in_stride % 8 != 0) return false;  // TMA: 16-byte aligned rows of bf16
    if ((uintptr_t)j.out % 4 != 0) return false;
    return true;
}

int launch_prefill(cudaStream_t s, const PrefillJob &j) {
    if (!prefill_supported(j)) return 0;
    prefill::Params p;
    memset(&p, 0, sizeof p);
    const uint32_t bn = pick_bn(j.tokens);
    // the activation buffer holds a multiple of 64 rows (the contract of matmul); rows past it read as zeros
    if (!encode_tiled_map(&p.xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, j.in, j.columns, j.padded_tokens, j.in_stride * 2, 64, bn, CU_TENSOR_MAP_SWIZZLE_128B))
        return 0;
    p.w = j.w; p.stride = j.stride; p.enc = j.enc; p.layout = j.layout;
    // the vector decoders read 16-byte pieces: GGUF Q4_K rows on 16-byte boundaries, or a planar form (always aligned)
    p.fast = (j.layout == 0 && j.enc == Q4_K && (uintptr_t)j.w % 16 == 0 && j.stride % 16 == 0 && j.columns % 256 == 0) || j.layout == 1 || j.layout == 2;
    p.rows = j.rows; p.columns = j.columns; p.tokens = j.tokens;
    p.out = j.out; p.out_stride = j.out_stride; p.status = j.status;
    dim3 grid((j.tokens + bn - 1) / bn, (j.rows + prefill::BM - 1) / prefill::BM);
    // Token tiles vary fastest over the grid, so the blocks running together share a few row tiles of weights. When the
    // activations of all token tiles no longer fit in L2 beside them (16,384 rows of 5,120 columns are 168 MB), every row
    // tile would stream them from HBM again: walk them in groups of about 48 MB instead.
    const size_t tile_bytes = (size_t)bn * j.columns * 2;
    if ((size_t)grid.x * tile_bytes > (size_t)(64u << 20) && (size_t)grid.x * grid.y < 0x7fffffffull) {
        p.group = (uint32_t)((size_t)(48u << 20) / tile_bytes);
        if (p.group < 1) p.group = 1;
        p.tok_tiles = grid.x;
        p.row_tiles = grid.y;
        grid = dim3(grid.x * grid.y, 1);
    }
    const bool q8_rows = j.layout == 0 && j.enc == Q8_0 && (uintptr_t)j.w % 4 == 0 && j.stride % 2 == 0;
    const bool q5k_rows = j.layout == 0 && j.enc == Q5_K && (uintptr_t)j.w % 16 == 0 && j.stride % 16 == 0 && j.columns % 256 == 0;
    const bool block32 = j.layout >= 3 && j.layout <= 6;
    const bool nibble_rows = j.layout == 0 && (j.enc == Q5_0 || j.enc == Q5_1 || j.enc == Q4_0 || j.enc == IQ4_NL) && (uintptr_t)j.w % 4 == 0 && j.stride % 2 == 0;
    const int mode = q8_rows ? 4 : q5k_rows ? 5 : block32 ? 6 : nibble_rows ? 8 : (j.layout == 7 || j.layout == 8) ? 7 : !p.fast ? 0 : j.enc == Q4_K ? 1 : j.layout == 1 ? 2 : 3;
    // Two blocks per SM (two stages each) when there are more blocks than SMs and the decoder is light enough for the
    // smaller register budget (measured: Q4_K 933 -> 1,067 TFLOP/s; planar Q6_K loses a little).
    const bool two = bn == 256 && (mode == 1 || mode == 3 || mode == 4 || mode == 5 || mode == 6 || mode == 7 || mode == 8) && (size_t)grid.x * grid.y > (size_t)j.sm_count;
    if (two) launch_bn<256, 2, 2>(grid, s, p, mode);
    else if (bn == 256) launch_bn<256, 4, 1>(grid, s, p, mode);
    else if (bn == 128) launch_bn<128, 6, 1>(grid, s, p, mode);
    else launch_bn<64, 8, 1>(grid, s, p, mode);
    return 1;
}

// ---- grouped form: the prefill of a mixture-of-experts layer --------------------------------------
// `Backend.matmulExperts` (ops/experts.zig:148-202; the reference's gathered tiles: kernels/matmul.metal:552-570,
// kernels/experts.metal:179-213). The slot rows arrive grouped by expert (the lists `expertLists` wrote). A gather
// pass copies each expert's input rows, rounded to bf16, into the scratch as whole tiles of 64 rows (the tail of an
// expert's last tile is zero), and writes one record per tile; the tensor-core kernel above then runs one block per
// (tile, 128 weight rows) on the expert's matrix and scatters its output rows through the list.

constexpr int GROUP_BN = 64;

// lists: [0] tile count of the reference's own tiling (unused here), [1] n, [2 .. 2 + experts] exclusive prefix offsets of
// the experts' slot rows, then 3 * bound words, then the n slot rows grouped by expert.
__global__ void __launch_bounds__(256) expert_gather_kernel(const uint32_t *lists, uint32_t experts, uint32_t bound, const float *in, size_t in_stride,
                                                            uint32_t in_group, uint32_t columns, __nv_bfloat16 *gathered, uint32_t *table) {
    __shared__ uint32_t found[4];  // expert, rows of this tile, first list entry, total tiles
    __shared__ uint32_t offsets[257];  // the experts' prefix offsets (at most 256 experts), read once by the block
    const uint32_t *slot_rows = lists + experts + 3 + 3 * (size_t)bound;
    const uint32_t tile = blockIdx.x, tid = threadIdx.x;
    for (uint32_t i = tid; i <= experts && i < 257; i += 256) offsets[i] = lists[2 + i];
    __syncthreads();
    if (tid == 0) {
        uint32_t at = 0;
        found[0] = 0xffffffffu;
        for (uint32_t e = 0; e < experts; ++e) {
            const uint32_t count = offsets[e + 1] - offsets[e], tiles = (count + GROUP_BN - 1) / GROUP_BN;
            if (tile >= at && tile < at + tiles) {
                found[0] = e;
                found[1] = min((uint32_t)GROUP_BN, count - (tile - at) * GROUP_BN);
                found[2] = offsets[e] + (tile - at) * GROUP_BN;
            }
            at += tiles;
        }
        found[3] = at;
        if (tile == 0) table[0] = at;
        if (found[0] != 0xffffffffu) {
            uint32_t *rec = table + 4 + 4 * (size_t)tile;
            rec[0] = found[0]; rec[1] = tile * GROUP_BN; rec[2] = found[1]; rec[3] = found[2];
        }
    }
    __syncthreads();
    if (found[0] == 0xffffffffu) return;
    const uint32_t rows = found[1], first = found[2];
    for (uint32_t i = 0; i < GROUP_BN; ++i) {
        __nv_bfloat16 *dst = gathered + ((size_t)tile * GROUP_BN + i) * columns;
        if (i < rows) {
            const float *src = in + (size_t)(slot_rows[first + i] / in_group) * in_stride;
            for (uint32_t c = tid; c < columns; c += 256) dst[c] = __float2bfloat16_rn(src[c]);
        } else {
            for (uint32_t c = tid; c < columns; c += 256) dst[c] = __float2bfloat16_rn(0.0f);
        }
    }
}

// Bytes of scratch the grouped form needs for `n` slot rows: the tile table, then the gathered bf16 rows.
size_t matmul_experts_scratch(uint32_t n, uint32_t experts, uint32_t columns) {
    const size_t tiles = (size_t)(n + GROUP_BN - 1) / GROUP_BN + (experts < n ? experts : n);
    return ((4 + 4 * tiles) * 4 + 1023) / 1024 * 1024 + tiles * GROUP_BN * columns * 2;
}

int launch_matmul_experts_fast(cudaStream_t s, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows, uint32_t columns,
                               const uint32_t *lists, uint32_t bound, uint32_t n, const float *in, size_t in_stride, uint32_t in_group, float *out, size_t out_stride,
                               void *scratch, size_t scratch_bytes, uint32_t *status) {
    if (layout(enc).elements == 0 || columns == 0 || columns % 64 != 0 || rows == 0 || n == 0) return 0;
    if (matmul_experts_scratch(n, experts, columns) > scratch_bytes || (uintptr_t)scratch % 1024 != 0 || (uintptr_t)out % 4 != 0) return 0;
    const size_t tiles = (size_t)(n + GROUP_BN - 1) / GROUP_BN + (experts < n ? experts : n);
    if (tiles > 65535u * 32u) return 0;
    uint32_t *table = (uint32_t *)scratch;
    __nv_bfloat16 *gathered = (__nv_bfloat16 *)((uint8_t *)scratch + ((4 + 4 * tiles) * 4 + 1023) / 1024 * 1024);
    prefill::Params p;
    memset(&p, 0, sizeof p);
    if (!encode_tiled_map(&p.xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, gathered, columns, tiles * GROUP_BN, (uint64_t)columns * 2, 64, GROUP_BN, CU_TENSOR_MAP_SWIZZLE_128B))
        return 0;
    expert_gather_kernel<<<(unsigned)tiles, 256, 0, s>>>(lists, experts, bound, in, in_stride, in_group, columns, gathered, table);
    p.w = w; p.stride = stride; p.enc = enc; p.layout = 0;
    p.fast = enc == Q4_K && (uintptr_t)w % 16 == 0 && stride % 16 == 0 && expert_bytes % 16 == 0 && columns % 256 == 0;
    p.rows = rows; p.columns = columns; p.tokens = (uint32_t)(tiles * GROUP_BN);
    p.out = out; p.out_stride = out_stride; p.status = status;
    p.tiles = table; p.slot_rows = lists + experts + 3 + 3 * (size_t)bound; p.expert_bytes = expert_bytes;
    dim3 grid((unsigned)tiles, (rows + prefill::BM - 1) / prefill::BM);
    // Two blocks of four stages per SM: with 64-row tiles the block is bound by its eight decoding warps, not by the tensor
    // core, and a second block doubles them (measured at 4,096 slot rows over 128 experts: the gate_up GEMM 425 -> see bench).
    const bool q8_rows = enc == Q8_0 && (uintptr_t)w % 4 == 0 && stride % 2 == 0 && expert_bytes % 4 == 0;
    const bool nibble_rows = (enc == Q5_0 || enc == Q5_1 || enc == Q4_0 || enc == IQ4_NL) && (uintptr_t)w % 4 == 0 && stride % 2 == 0 && expert_bytes % 4 == 0;
    const bool q5k_rows = enc == Q5_K && (uintptr_t)w % 16 == 0 && stride % 16 == 0 && expert_bytes % 16 == 0 && columns % 256 == 0;
    launch_bn<64, 4, 2>(grid, s, p, p.fast ? 1 : q8_rows ? 4 : q5k_rows ? 5 : nibble_rows ? 8 : 0);
    return 2;
}

// ---- F32 -> BF16 rows (the reference's matmul takes F32 activations) ------------------------------

__global__ void f32_to_bf16_rows_kernel(const float *in, size_t in_stride, __nv_bfloat16 *out, size_t out_stride, uint32_t columns, uint32_t tokens) {
    const size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (size_t)columns * tokens) return;
    const size_t t = id / columns, c = id % columns;
    out[t * out_stride + c] = __float2bfloat16_rn(in[t * in_stride + c]);
}

int launch_f32_to_bf16_rows(cudaStream_t s, const float *in, size_t in_stride, void *out, size_t out_stride, uint32_t columns, uint32_t tokens) {
    const size_t n = (size_t)columns * tokens;
    f32_to_bf16_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(in, in_stride, (__nv_bfloat16 *)out, out_stride, columns, tokens);
    return 1;
}

}  // namespace nu
