// Prefill GEMM for sm_100a: out[t][r] = sum_k W[r][k] * X[t][k] for many token rows, the
// weights block-quantized, the contraction on the 5th-generation tensor cores.
// Serves Backend.matmul beyond the small-batch kernels (the reference's tiles for this are
// nu_matmul_t, inference/src/backends/metal/kernels/matmul.metal:335-412: decode a K step of
// weights into a half tile in threadgroup memory, stage the activations, 8x8 MACs).
//
// One block computes a 128-row x BN-token tile of the output:
//   * warps 0..15 (512 threads: weight row tid & 127, column quarter tid >> 7) each decode 16 columns of
//     their row per K step to bf16 (vector decoders for 16-byte aligned Q4_K and the planar Q6_K /
//     Q8_0 forms: byte -> float through the 2^23 magic number, one FMA, packed conversion; the
//     generic per-16 decoder otherwise) and store them in shared memory in the 128-byte-swizzled
//     K-major layout the tensor core reads; the same warps later move the accumulator from tensor
//     memory to the output;
//   * warp 16 (one thread) brings the matching BN x 64 tile of bf16 activations with one TMA
//     tensor copy per K step (128-byte swizzle, so no thread touches those bytes);
//   * warp 17 (one thread) issues tcgen05.mma (M = 128, N = BN, K = 16, bf16 x bf16 -> f32) four
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
constexpr int PRODUCER_WARPS = 16; // decode threads: 128 rows x 4 column quarters of a K step
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
__device__ __forceinline__ void decode16_generic(const Params &p, uint32_t r, uint32_t k0, uint32_t q, uint4 chunks[2]) {
    float v[16];
    const uint32_t seg = k0 / 16 + q;
    if (p.layout == 1) dequant16_planar_q6k(p.w, p.rows, p.columns / 256, r, seg, v);
    else if (p.layout == 2) dequant16_planar_q8_0(p.w, p.rows, p.columns, r, seg, v);
    else dequant16(p.enc, p.w + (size_t)r * p.stride, seg, v);
#pragma unroll
    for (int c = 0; c < 2; ++c)
        chunks[c] = make_uint4(pack_bf16(v[c * 8], v[c * 8 + 1]), pack_bf16(v[c * 8 + 2], v[c * 8 + 3]), pack_bf16(v[c * 8 + 4], v[c * 8 + 5]),
                               pack_bf16(v[c * 8 + 6], v[c * 8 + 7]));
}

// The bytes a producer thread needs for one K step, requested one step ahead of their use so that
// the latency of the loads hides behind the decoding of the step before.
struct Raw {
    uint4 v[2];
    uint32_t s;  // scale bytes / f16 scale bits, by encoding
};

// Q4_K, rows 16-byte aligned: the 64 columns of a K step are one group pair; quarters 0, 1 are its
// even group (low nibbles of bytes 0..15, 16..31), quarters 2, 3 the odd group (high nibbles).
// Values are (d*s)*q - dmin*m with one rounding, like the reference decoder
// (inference/src/quant/decode.zig:147-170), then rounded to bf16.
__device__ __forceinline__ void load16_q4k(const Params &p, uint32_t r, uint32_t k0, uint32_t q, Raw &raw) {
    const uint8_t *block = p.w + (size_t)r * p.stride + (size_t)(k0 / 256) * 144;
    const uint32_t pair = (k0 / 64) & 3u;
    raw.v[0] = *(const uint4 *)block;
    raw.v[1] = *(const uint4 *)(block + 16 + pair * 32 + (q & 1u) * 16);
}
__device__ __forceinline__ void convert16_q4k(const Raw &raw, uint32_t k0, uint32_t q, uint4 chunks[2]) {
    const uint32_t pair = (k0 / 64) & 3u, half = q >> 1, grp = pair * 2 + half;
    const uint4 hdr = raw.v[0], qq = raw.v[1];
    // six-bit scale and minimum of group grp out of the 12 packed bytes (words hdr.y, hdr.z, hdr.w)
    const uint32_t lo_byte = grp & 3u;
    const uint32_t y = (hdr.y >> (8 * lo_byte)) & 0xffu, z = (hdr.z >> (8 * lo_byte)) & 0xffu, w = (hdr.w >> (8 * lo_byte)) & 0xffu;
    const uint32_t s6 = grp < 4 ? (y & 63u) : ((w & 15u) | ((y >> 6) << 4));
    const uint32_t m6 = grp < 4 ? (z & 63u) : ((w >> 4) | ((z >> 6) << 4));
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu))), dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    const float ds = __fmul_rn(d, (float)s6), ndm = -__fmul_rn(dmin, (float)m6);
    const uint32_t words[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint32_t packed[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t t4 = (half ? (words[c * 2 + h] >> 4) : words[c * 2 + h]) & 0x0f0f0f0fu;  // four codes, one per byte
            const float v0 = fmaf(byte_f32(t4, 0), ds, ndm), v1 = fmaf(byte_f32(t4, 1), ds, ndm);
            const float v2 = fmaf(byte_f32(t4, 2), ds, ndm), v3 = fmaf(byte_f32(t4, 3), ds, ndm);
            packed[h * 2] = pack_bf16(v0, v1);
            packed[h * 2 + 1] = pack_bf16(v2, v3);
        }
        chunks[c] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

// Planar Q8_0 (prepare.cu): 16 columns are half a block; value = d * code, exact before the bf16 rounding.
__device__ __forceinline__ void load16_q8_0_planar(const Params &p, uint32_t r, uint32_t k0, uint32_t q, Raw &raw) {
    const uint32_t blk = k0 / 32 + (q >> 1);
    raw.v[0] = *(const uint4 *)(p.w + (size_t)r * p.columns + k0 + q * 16);
    raw.s = *(const unsigned short *)(p.w + (size_t)p.rows * p.columns + ((size_t)blk * p.rows + r) * 2);
}
__device__ __forceinline__ void convert16_q8_0_planar(const Raw &raw, uint4 chunks[2]) {
    const float d = __half2float(__ushort_as_half((unsigned short)raw.s));
    const uint32_t words[4] = {raw.v[0].x, raw.v[0].y, raw.v[0].z, raw.v[0].w};
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint32_t packed[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t u = words[c * 2 + h] ^ 0x80808080u;  // code + 128
            const float v0 = (byte_f32(u, 0) - 128.0f) * d, v1 = (byte_f32(u, 1) - 128.0f) * d;
            const float v2 = (byte_f32(u, 2) - 128.0f) * d, v3 = (byte_f32(u, 3) - 128.0f) * d;
            packed[h * 2] = pack_bf16(v0, v1);
            packed[h * 2 + 1] = pack_bf16(v2, v3);
        }
        chunks[c] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

// Planar Q6_K (prepare.cu): the 16 columns are column half ch of quarter qr of half hh of a
// superblock: one planar chunk and one scale; value = (d * scale) * (code - 32), exact.
__device__ __forceinline__ void load16_q6k_planar(const Params &p, uint32_t r, uint32_t k0, uint32_t q, Raw &raw) {
    const uint32_t ksb = p.columns / 256, sb = k0 / 256, j = ((k0 / 32) & 7u) + (q >> 1), ch = q & 1u;  // 32-column run j, its half ch
    const uint32_t hh = j >> 2, qr = j & 3u;
    const uint8_t *rec = p.w + ((size_t)r * ksb + sb) * 208;
    const uint8_t *chunk = rec + (hh * 2 + ch) * 48;
    raw.v[0] = *(const uint4 *)(chunk + (qr & 1u) * 16);
    raw.v[1] = *(const uint4 *)(chunk + 32);
    const uint32_t scale = rec[192 + hh * 8 + qr * 2 + ch];
    const uint32_t dbits = *(const unsigned short *)(p.w + (size_t)p.rows * ksb * 208 + ((size_t)sb * p.rows + r) * 2);
    raw.s = scale | (dbits << 16);
}
__device__ __forceinline__ void convert16_q6k_planar(const Raw &raw, uint32_t k0, uint32_t q, uint4 chunks[2]) {
    const uint32_t qr = (((k0 / 32) & 7u) + (q >> 1)) & 3u;
    const float d = __half2float(__ushort_as_half((unsigned short)(raw.s >> 16)));
    const float ds = __fmul_rn(d, (float)(int8_t)(raw.s & 0xffu));
    const uint4 ql = raw.v[0], qh = raw.v[1];
    const uint32_t lw[4] = {ql.x, ql.y, ql.z, ql.w}, hw[4] = {qh.x, qh.y, qh.z, qh.w};
    uint32_t packed[8];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const uint32_t nib = ((qr >> 1) ? (lw[m] >> 4) : lw[m]) & 0x0f0f0f0fu;
        const uint32_t top = ((hw[m] >> (2 * qr)) & 0x03030303u) << 4;
        const uint32_t v = nib | top;  // four codes 0..63, one per byte
        packed[m * 2] = pack_bf16((byte_f32(v, 0) - 32.0f) * ds, (byte_f32(v, 1) - 32.0f) * ds);
        packed[m * 2 + 1] = pack_bf16((byte_f32(v, 2) - 32.0f) * ds, (byte_f32(v, 3) - 32.0f) * ds);
    }
    chunks[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    chunks[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}

// mode: 0 generic, 1 Q4_K, 2 planar Q6_K, 3 planar Q8_0
__device__ __forceinline__ uint32_t decode_mode(const Params &p) { return !p.fast ? 0u : p.enc == Q4_K ? 1u : p.layout == 1 ? 2u : 3u; }
__device__ __forceinline__ void load16(const Params &p, uint32_t mode, uint32_t r, uint32_t k0, uint32_t q, Raw &raw) {
    if (mode == 1) load16_q4k(p, r, k0, q, raw);
    else if (mode == 2) load16_q6k_planar(p, r, k0, q, raw);
    else if (mode == 3) load16_q8_0_planar(p, r, k0, q, raw);
}
__device__ __forceinline__ void convert16(const Params &p, uint32_t mode, const Raw &raw, uint32_t r, uint32_t k0, uint32_t q, uint4 chunks[2]) {
    if (mode == 1) convert16_q4k(raw, k0, q, chunks);
    else if (mode == 2) convert16_q6k_planar(raw, k0, q, chunks);
    else if (mode == 3) convert16_q8_0_planar(raw, chunks);
    else decode16_generic(p, r, k0, q, chunks);
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS, 1) prefill_kernel(const __grid_constant__ Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzled tiles sit on 1024-byte boundaries
    constexpr int A_BYTES = BM * BK * 2;   // 16 KiB
    constexpr int B_BYTES = BN * BK * 2;
    uint8_t *a_tiles = smem;                              // [STAGES][A_BYTES], 1024-byte aligned
    uint8_t *b_tiles = a_tiles + STAGES * A_BYTES;        // [STAGES][B_BYTES]
    uint64_t *bars = (uint64_t *)(b_tiles + STAGES * B_BYTES);
    // barriers: full_a[STAGES] (16 producer warps), full_b[STAGES] (TMA bytes), empty[STAGES] (MMA done), accum
    const uint32_t full_a = smem_u32(bars), full_b = smem_u32(bars + STAGES), empty = smem_u32(bars + 2 * STAGES), accum = smem_u32(bars + 3 * STAGES);
    uint32_t *tmem_slot = (uint32_t *)(bars + 3 * STAGES + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // token tiles vary fastest over the grid: the blocks running together share a few row tiles of weights (L2) 
    const uint32_t row0 = blockIdx.y * BM, tok0 = blockIdx.x * BN;
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
        // ---- decode producers: thread (r, q) owns 16 columns per K step of weight row row0 + r ----
        const uint32_t r = tid & 127u, q = tid >> 7;
        const uint32_t grow = min(row0 + r, p.rows - 1);  // rows past the matrix repeat the last one; never stored
        uint8_t *arow = a_tiles + (r >> 3) * 1024 + (r & 7) * 128;
        bool ok = true;
        const uint32_t mode = decode_mode(p);
        Raw raw;
        load16(p, mode, grow, 0, q, raw);
        for (uint32_t k = 0; k < ksteps && ok; ++k) {
            const uint32_t s = k % STAGES;
            const Raw cur = raw;
            if (k + 1 < ksteps) load16(p, mode, grow, (k + 1) * BK, q, raw);  // in flight while this step is decoded
            if (k >= STAGES) ok = mbar_wait(empty + s * 8, ((k / STAGES) - 1) & 1u, abort_flag);
            if (!ok) break;
            uint4 chunks[2];
            convert16(p, mode, cur, grow, k * BK, q, chunks);
#pragma unroll
            for (int c = 0; c < 2; ++c) *(uint4 *)(arow + s * A_BYTES + (((q * 2 + c) ^ (r & 7)) * 16)) = chunks[c];
            // make the generic-proxy stores visible to the tensor core's reads, then one arrival per warp
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(full_a + s * 8);
        }
        // ---- epilogue: tensor memory -> output; warps 0..7: warp w reads lanes 32 (w & 3) .. + 31 (its rows), half of the columns ----
        const uint32_t half = q & 1u;
        if (ok && q < 2) ok = mbar_wait(accum, 0, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok && q < 2) {
            const uint32_t out_row = row0 + r;
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
                        const uint32_t tok = tok0 + c0 + j;
                        if (tok < p.tokens) p.out[(size_t)tok * p.out_stride + out_row] = __uint_as_float(v[j]);
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

template <int BN, int STAGES>
static bool configure_bn() {
    return cudaFuncSetAttribute(prefill::prefill_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, prefill::smem_bytes<BN, STAGES>()) == cudaSuccess;
}

#ifndef NU_PREFILL_STAGES256
#define NU_PREFILL_STAGES256 4
#endif
#ifndef NU_PREFILL_MAXBN
#define NU_PREFILL_MAXBN 256
#endif
bool prefill_configure() { return configure_bn<256, NU_PREFILL_STAGES256>() && configure_bn<128, 6>() && configure_bn<64, 8>(); }

static uint32_t pick_bn(uint32_t tokens) { return tokens > 128 && NU_PREFILL_MAXBN >= 256 ? 256 : tokens > 64 ? 128 : 64; }

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
    if (bn == 256) prefill::prefill_kernel<256, NU_PREFILL_STAGES256><<<grid, prefill::THREADS, prefill::smem_bytes<256, NU_PREFILL_STAGES256>(), s>>>(p);
    else if (bn == 128) prefill::prefill_kernel<128, 6><<<grid, prefill::THREADS, prefill::smem_bytes<128, 6>(), s>>>(p);
    else prefill::prefill_kernel<64, 8><<<grid, prefill::THREADS, prefill::smem_bytes<64, 8>(), s>>>(p);
    return 1;
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
