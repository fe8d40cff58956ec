// Expert GEMV for the decode form of a mixture-of-experts layer: one launch multiplies every routed
// slot's input by the matrix of the expert the slot selected (Backend.matvecExperts /
// matvecExpertsGrouped, inference/src/backends/metal/ops/experts.zig:36-77; the reference's kernel
// is nu_matvec_experts, kernels/experts.metal:16-36). Specialized for the forms an expert
// tensor of the 26B-A4B-style layer is stored in: Q4_K (gate_up, [experts][2 ff][hidden]) and, for
// down ([experts][hidden][ff] with ff = 704 = 22 blocks), GGUF Q8_0, Q5_0, Q5_1, Q4_0 and IQ4_NL;
// everything else stays on the generic kernel.
//
// The work is a few to a few hundred megabytes spread over up to 64 small matrices picked by
// device-side indices, so the kernels use plain loads instead of tensor maps (an expert's address is
// known only on the device). A first version decoded every code to F32 (permute, subtract, FMA: six
// instructions per weight and lane all told) and was bound by instruction issue at 2.1 TB/s. This
// one keeps the codes as the bytes they are and multiplies them on the integer dot-product unit:
//
//  * The block turns its slot's input row into fixed point once: per chunk of columns (16 for Q4_K,
//    32 for Q8_0) X = round(x * 2^k), k chosen from the chunk's largest exponent so that |X| < 2^20,
//    split into three signed digits X = p2 * 2^14 + p1 * 2^7 + p0 with |p| <= 64, kept as three
//    byte planes in shared memory. An element is off by at most 2^-21 of its chunk's largest value.
//  * dp4a (four byte products added into an int32) then gives sum(code * p) exactly, for four
//    weights per instruction and digit; the three digit sums are recombined (Q4_K: in int32, a digit
//    sum is at most 16 * 15 * 64 and times 2^14 stays below 2^31; Q8_0: in F32, where 32 * 128 * 64 =
//    2^18 times 2^14 would not fit) and scaled by 2^-k and the block's scales in F32.
//  * Q4_K: 8 lanes per weight row, 4 rows per warp, 32 rows per block. Lane p of a row takes the
//    16-byte piece p of each superblock's 128 quant bytes: 16 low nibbles of group 2(p/2) and 16 high
//    nibbles of group 2(p/2)+1, columns 16(p&1).. of each; `w & 0x0f0f0f0f` is four codes ready for
//    dp4a. The minima multiply exact F32 sums of x prepared once per chunk.
//  * Q8_0: a block copies 32 weight rows into shared memory, then a lane per row and a warp per 32-column
//    block: the digits of a block are one broadcast address for the warp, the int8 codes go to dp4a as
//    they are (an earlier version gave a lane 8 codes at a time: twelve instructions per code all told).
//  * The weight bytes travel with cp.async into shared memory (Q4_K: a ring, six superblocks ahead; Q8_0:
//    the block's 32 rows at once, as 4-byte copies since its blocks are only 2-byte aligned) instead of
//    being held in registers: the first versions had one 16-byte load per lane in flight.
// Sums run in a fixed order: results do not depend on timing.
#include "kernels.hpp"
#include "nu_device.cuh"

namespace nu {
namespace {

constexpr int XQ_THREADS = 256;
constexpr int XQ_ROWS = 32;  // Q4_K: weight rows per block, 8 lanes each

__device__ __forceinline__ int dp4a_us(uint32_t codes, uint32_t digits, int c) {  // unsigned codes x signed digits
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(codes), "r"(digits), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t codes, uint32_t digits, int c) {  // signed codes x signed digits
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(codes), "r"(digits), "r"(c));
    return d;
}

// 6-bit scales and minima of groups 2j and 2j+1 of a Q4_K superblock, as two bytes each (group 2j in the low
// byte); y, z, w are scale bytes 0..3, 4..7, 8..11. No branch: the lanes of a warp hold different j.
__device__ __forceinline__ void q4k_pair_scales(uint32_t y, uint32_t z, uint32_t w, uint32_t j, uint32_t &s2, uint32_t &m2) {
    const uint32_t shift = (j & 1u) * 16;
    const uint32_t hy = (y >> shift) & 0xffffu, hz = (z >> shift) & 0xffffu, hw = (w >> shift) & 0xffffu;
    // groups 0..3: low six bits of bytes 0..3 / 4..7; groups 4..7: nibbles of bytes 8..11 plus the top two bits of bytes 0..7
    const uint32_t s_lo = hy & 0x3f3fu, m_lo = hz & 0x3f3fu;
    const uint32_t s_hi = (hw & 0x0f0fu) | ((hy >> 2) & 0x3030u), m_hi = ((hw >> 4) & 0x0f0fu) | ((hz >> 2) & 0x3030u);
    s2 = j < 2 ? s_lo : s_hi;
    m2 = j < 2 ? m_lo : m_hi;
}
// byte b of w as a float: 0x4b0000bb is 2^23 + b
__device__ __forceinline__ float byte_f32(uint32_t w, int b) { return __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7650u + b)) - 8388608.0f; }

// Power of two that brings a chunk whose largest magnitude is `mx` below 2^20, and its inverse. A chunk that
// is all zero (or too small to matter) is left as it is; one that holds an infinity or a NaN gets a NaN
// inverse so that the row's result is NaN, as the F32 arithmetic would give.
__device__ __forceinline__ void chunk_scale(float mx, float &scale, float &inv) {
    const uint32_t e = (__float_as_uint(mx) >> 23) & 0xffu;
    if (e == 255u) { scale = 0.0f; inv = __uint_as_float(0x7fc00000u); return; }
    if (e < 40u) { scale = 1.0f; inv = 1.0f; return; }
    scale = __uint_as_float((273u - e) << 23);  // 2^(146 - e): mx < 2^(e - 126) becomes < 2^20
    inv = __uint_as_float((e - 19u) << 23);     // 2^(e - 146)
}
// Three signed digits of X = p2 * 2^14 + p1 * 2^7 + p0, |X| <= 2^20: p0, p1 in [-64, 63], p2 in [-64, 64].
__device__ __forceinline__ void digits(float x, float scale, int &p0, int &p1, int &p2) {
    const int X = __float2int_rn(x * scale);
    p0 = ((X + 64) & 127) - 64;
    const int X1 = (X - p0) >> 7;
    p1 = ((X1 + 64) & 127) - 64;
    p2 = (X1 - p1) >> 7;
}
// Byte planes are padded by 32 bytes per 128 so that the eight lanes of a weight row, which read 16-byte
// chunks 0, 1, 4, 5, 8, 9, 12, 13 (or those + 2) of a superblock's 16, hit eight different groups of banks.
__device__ __forceinline__ uint32_t plane_offset(uint32_t byte) { return byte + (byte >> 7) * 32; }

constexpr int XQ_STAGES = 6;                        // superblocks in flight per lane
constexpr int XQ_RING = XQ_STAGES * XQ_ROWS * 144;  // bytes: a stage holds one superblock of each of the block's rows

__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void *dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ACT: 0 plain (a row of the tensor per output row); ACT_SILU / ACT_GELU: the tensor is [gate rows][up rows] and the
// output row i is act(gate row i) * (up row i): a block then takes 16 gate rows and their 16 up rows, and the two
// halves meet in shared memory (the activation pass behind the gate_up GEMV, ops/rowwise.zig:230-233, folded in).
template <int ACT>
__global__ void __launch_bounds__(XQ_THREADS) expert_gemv_q4k_kernel(const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                                                                     uint32_t ksb, const uint32_t *indices, const float *in, size_t in_stride,
                                                                     uint32_t in_group, float *out, size_t out_stride) {
    // [ring of weight stages][3 planes of digits, ksb * 320 bytes each][ksb * 16 pairs (inverse scale, sum of x)]
    // (one pair per 16 columns)
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t *ring = smem;
    uint8_t *planes = smem + XQ_RING;
    const uint32_t plane = ksb * 320;
    float2 *chunk = (float2 *)(planes + 3 * plane);
    // launched so that its blocks may be placed while the operator before it drains; nothing is read before this
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t slot = blockIdx.y;
    const uint32_t rl = threadIdx.x >> 3, p = threadIdx.x & 7;
    const uint32_t half = rows / 2;  // gated: the gate rows; `rows` counts both halves of the tensor
    const uint32_t pair_row = blockIdx.x * (XQ_ROWS / 2) + (rl & 15u);   // gated: the output row this lane's tensor row belongs to
    const uint32_t r = ACT ? (rl < 16 ? pair_row : half + pair_row) : blockIdx.x * XQ_ROWS + rl;
    const bool live = ACT ? pair_row < half : r < rows;
    // A corrupt routing buffer can never read past the tensor (experts.metal:25).
    const uint32_t expert = min(indices[slot], experts - 1);
    const uint8_t *row = w + (size_t)expert * expert_bytes + (size_t)(live ? r : 0) * stride;
    // The weight stream: lane p copies its 16-byte piece of the row's superblock (lane 0 also the 16-byte header)
    // into the stage, XQ_STAGES - 1 superblocks ahead of its use, without holding them in registers.
    uint8_t *const my_ring = ring + rl * 144;
    const uint8_t *src_next = row;
    uint32_t stage_next = 0, sb_next = 0;
    auto request = [&]() {
        if (live && sb_next < ksb) {
            uint8_t *dst = my_ring + stage_next * (XQ_ROWS * 144);
            cp_async16(dst + 16 + p * 16, src_next + 16 + p * 16);
            if (p == 0) cp_async16(dst, src_next);
        }
        cp_async_commit();
        ++sb_next;
        src_next += 144;
        stage_next = stage_next + 1 == XQ_STAGES ? 0 : stage_next + 1;
    };
    for (int i = 0; i < XQ_STAGES - 1; ++i) request();  // in flight while the input row is prepared

    const float *x = in + (size_t)(slot / in_group) * in_stride;
    for (uint32_t c = threadIdx.x; c < ksb * 16; c += XQ_THREADS) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 f = __ldg((const float4 *)x + c * 4 + i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
        float mx = 0.0f, bad = 0.0f;  // bad: 0 * x is NaN for an infinity or a NaN, which fmaxf would drop
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            mx = fmaxf(mx, fabsf(v[i]));
            bad += 0.0f * v[i];
        }
        mx += bad;
        float scale, inv;
        chunk_scale(mx, scale, inv);
        uint32_t d0[4], d1[4], d2[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            d0[i] = d1[i] = d2[i] = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                int p0, p1, p2;
                digits(v[4 * i + b], scale, p0, p1, p2);
                d0[i] |= (uint32_t)(p0 & 0xff) << (8 * b);
                d1[i] |= (uint32_t)(p1 & 0xff) << (8 * b);
                d2[i] |= (uint32_t)(p2 & 0xff) << (8 * b);
            }
        }
        const uint32_t off = plane_offset(c * 16);
        *(uint4 *)(planes + off) = make_uint4(d0[0], d0[1], d0[2], d0[3]);
        *(uint4 *)(planes + plane + off) = make_uint4(d1[0], d1[1], d1[2], d1[3]);
        *(uint4 *)(planes + 2 * plane + off) = make_uint4(d2[0], d2[1], d2[2], d2[3]);
        chunk[c] = make_float2(inv, ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7])) + (((v[8] + v[9]) + (v[10] + v[11])) + ((v[12] + v[13]) + (v[14] + v[15]))));
    }
    __syncthreads();
    float acc = 0.0f;
    const uint32_t c_lo = 4 * (p >> 1) + (p & 1u);  // this lane's 16-column chunks of a superblock: c_lo (low nibbles) and c_lo + 2
    // this lane's places, advanced by one superblock per turn: digits of chunk c_lo (those of c_lo + 2 sit 32 bytes on), the chunk pairs
    const uint8_t *dig = planes + plane_offset(c_lo * 16);
    const float2 *ch = chunk + c_lo;
    uint32_t stage = 0;
    for (uint32_t sb = 0; sb < ksb; ++sb) {
        request();
        cp_async_wait<XQ_STAGES - 1>();  // this lane's copies of superblock sb have landed
        __syncwarp();                    // and so have lane 0's (the header)
        if (live) {
            const uint8_t *src = my_ring + stage * (XQ_ROWS * 144);
            const uint4 hdr = *(const uint4 *)src;
            const uint4 q = *(const uint4 *)(src + 16 + p * 16);
            const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
            const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
            uint32_t s2, m2;
            q4k_pair_scales(hdr.y, hdr.z, hdr.w, p >> 1, s2, m2);
            const float s_lo = byte_f32(s2, 0), s_hi = byte_f32(s2, 1), m_lo = byte_f32(m2, 0), m_hi = byte_f32(m2, 1);
            const uint4 l0 = *(const uint4 *)dig, l1 = *(const uint4 *)(dig + plane), l2 = *(const uint4 *)(dig + 2 * plane);
            const uint4 h0 = *(const uint4 *)(dig + 32), h1 = *(const uint4 *)(dig + plane + 32), h2 = *(const uint4 *)(dig + 2 * plane + 32);
            const float2 k_lo = ch[0], k_hi = ch[2];
            const uint32_t ql[4] = {q.x & 0x0f0f0f0fu, q.y & 0x0f0f0f0fu, q.z & 0x0f0f0f0fu, q.w & 0x0f0f0f0fu};
            const uint32_t qh[4] = {(q.x >> 4) & 0x0f0f0f0fu, (q.y >> 4) & 0x0f0f0f0fu, (q.z >> 4) & 0x0f0f0f0fu, (q.w >> 4) & 0x0f0f0f0fu};
            int a0 = 0, a1 = 0, a2 = 0, b0 = 0, b1 = 0, b2 = 0;
            a0 = dp4a_us(ql[0], l0.x, a0); a0 = dp4a_us(ql[1], l0.y, a0); a0 = dp4a_us(ql[2], l0.z, a0); a0 = dp4a_us(ql[3], l0.w, a0);
            a1 = dp4a_us(ql[0], l1.x, a1); a1 = dp4a_us(ql[1], l1.y, a1); a1 = dp4a_us(ql[2], l1.z, a1); a1 = dp4a_us(ql[3], l1.w, a1);
            a2 = dp4a_us(ql[0], l2.x, a2); a2 = dp4a_us(ql[1], l2.y, a2); a2 = dp4a_us(ql[2], l2.z, a2); a2 = dp4a_us(ql[3], l2.w, a2);
            b0 = dp4a_us(qh[0], h0.x, b0); b0 = dp4a_us(qh[1], h0.y, b0); b0 = dp4a_us(qh[2], h0.z, b0); b0 = dp4a_us(qh[3], h0.w, b0);
            b1 = dp4a_us(qh[0], h1.x, b1); b1 = dp4a_us(qh[1], h1.y, b1); b1 = dp4a_us(qh[2], h1.z, b1); b1 = dp4a_us(qh[3], h1.w, b1);
            b2 = dp4a_us(qh[0], h2.x, b2); b2 = dp4a_us(qh[1], h2.y, b2); b2 = dp4a_us(qh[2], h2.z, b2); b2 = dp4a_us(qh[3], h2.w, b2);
            const float f_lo = (float)(a2 * 16384 + a1 * 128 + a0) * k_lo.x;
            const float f_hi = (float)(b2 * 16384 + b1 * 128 + b0) * k_hi.x;
            acc = fmaf(d * s_lo, f_lo, acc);
            acc = fmaf(d * s_hi, f_hi, acc);
            acc = fmaf(-(dmin * m_lo), k_lo.y, acc);
            acc = fmaf(-(dmin * m_hi), k_hi.y, acc);
        }
        dig += 320;
        ch += 16;
        stage = stage + 1 == XQ_STAGES ? 0 : stage + 1;
        __syncwarp();  // every lane is done with this stage before lane 0 refills its header
    }
    cp_async_wait<0>();
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (ACT) {
        __shared__ float gate_sums[XQ_ROWS / 2];
        if (p == 0 && rl < 16) gate_sums[rl] = acc;
        __syncthreads();
        if (p == 0 && rl >= 16 && live) {
            const float g = gate_sums[rl - 16];
            out[(size_t)slot * out_stride + pair_row] = (ACT == ACT_SILU ? silu_f32(g) : gelu_f32(g)) * acc;
        }
        return;
    }
    if (p == 0 && live) out[(size_t)slot * out_stride + r] = acc;
}

constexpr int X8_WARPS = 8;
constexpr int X8_ROWS = 32;  // weight rows per block: a lane per row

__global__ void __launch_bounds__(X8_WARPS * 32) expert_gemv_q8_0_kernel(const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                                                                         uint32_t blocks, const uint32_t *indices, const float *in, size_t in_stride,
                                                                         uint32_t in_group, float *out, size_t out_stride) {
    // [32 weight rows, `pitch` words each][3 planes of digits, blocks * 32 bytes each][blocks inverse scales][8 x 32 part sums]
    // A row is blocks * 34 / 4 whole words (the launcher takes an even number of blocks); the pitch is odd so that
    // the 32 lanes of a warp, one row each, read 32 different banks.
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t words = blocks * 34 / 4;
    const uint32_t pitch = words | 1u;
    uint32_t *tile = (uint32_t *)smem;
    uint8_t *planes = smem + (((size_t)X8_ROWS * pitch * 4 + 15) & ~(size_t)15);
    const uint32_t plane = blocks * 32;
    float *inv_scale = (float *)(planes + 3 * plane);
    float *parts = inv_scale + blocks;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t slot = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t expert = min(indices[slot], experts - 1);
    const uint32_t r0 = blockIdx.x * X8_ROWS;
    const uint32_t nrows = min((uint32_t)X8_ROWS, rows - r0);
    const uint8_t *base = w + (size_t)expert * expert_bytes + (size_t)r0 * stride;
    // the block's rows travel to shared memory as 4-byte copies (the 34-byte blocks are only 2-byte aligned),
    // consecutive threads on consecutive words of a row; all of them are in flight while the input row is prepared
    // (warp w takes rows w, w + 8, ...; its lanes consecutive words: no division in the loop)
    for (uint32_t r = warp; r < nrows; r += X8_WARPS) {
        const uint8_t *src = base + (size_t)r * stride;
        uint32_t *dst = tile + r * pitch;
        for (uint32_t c = lane; c < words; c += 32) cp_async4(dst + c, src + c * 4);
    }
    cp_async_commit();

    const float *x = in + (size_t)(slot / in_group) * in_stride;
    // a warp per block of 32 columns, a lane per column
    for (uint32_t b = warp; b < blocks; b += X8_WARPS) {
        const float v = __ldg(x + b * 32 + lane);
        float mx = fabsf(v), bad = 0.0f * v;  // bad: NaN for an infinity or a NaN, which fmaxf would drop
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            bad += __shfl_xor_sync(0xffffffffu, bad, o);
        }
        mx += bad;
        float scale, inv;
        chunk_scale(mx, scale, inv);
        int p0, p1, p2;
        digits(v, scale, p0, p1, p2);
        planes[b * 32 + lane] = (uint8_t)p0;
        planes[plane + b * 32 + lane] = (uint8_t)p1;
        planes[2 * plane + b * 32 + lane] = (uint8_t)p2;
        if (lane == 0) inv_scale[b] = inv;
    }
    cp_async_wait<0>();
    __syncthreads();
    // lane = row of the tile; warp w takes blocks w, w + 8, ...: the digits of a block are one address for the
    // whole warp (a broadcast), the codes 32 different banks
    float acc = 0.0f;
    if (lane < nrows) {
        const uint32_t *row = tile + lane * pitch;
        for (uint32_t b = warp; b < blocks; b += X8_WARPS) {
            // the block starts at byte 34 b of the row: scale in the low or high half of word 17 b / 2, codes after it
            const uint32_t first = (b * 34) >> 2;
            uint32_t c[8];
            float d;
            if (b & 1u) {  // bytes 34 b .. start in the middle of a word: scale high half, codes word-aligned
                d = __half2float(__ushort_as_half((unsigned short)(row[first] >> 16)));
#pragma unroll
                for (int i = 0; i < 8; ++i) c[i] = row[first + 1 + i];
            } else {       // scale low half, codes straddle words
                uint32_t wv[9];
#pragma unroll
                for (int i = 0; i < 9; ++i) wv[i] = row[first + i];
                d = __half2float(__ushort_as_half((unsigned short)(wv[0] & 0xffffu)));
#pragma unroll
                for (int i = 0; i < 8; ++i) c[i] = __funnelshift_r(wv[i], wv[i + 1], 16);
            }
            const uint4 *dg = (const uint4 *)(planes + b * 32);
            const uint4 *dg1 = (const uint4 *)(planes + plane + b * 32), *dg2 = (const uint4 *)(planes + 2 * plane + b * 32);
            int a0 = 0, a1 = 0, a2 = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 q0 = dg[h], q1 = dg1[h], q2 = dg2[h];
                a0 = dp4a_ss(c[4 * h], q0.x, a0); a0 = dp4a_ss(c[4 * h + 1], q0.y, a0); a0 = dp4a_ss(c[4 * h + 2], q0.z, a0); a0 = dp4a_ss(c[4 * h + 3], q0.w, a0);
                a1 = dp4a_ss(c[4 * h], q1.x, a1); a1 = dp4a_ss(c[4 * h + 1], q1.y, a1); a1 = dp4a_ss(c[4 * h + 2], q1.z, a1); a1 = dp4a_ss(c[4 * h + 3], q1.w, a1);
                a2 = dp4a_ss(c[4 * h], q2.x, a2); a2 = dp4a_ss(c[4 * h + 1], q2.y, a2); a2 = dp4a_ss(c[4 * h + 2], q2.z, a2); a2 = dp4a_ss(c[4 * h + 3], q2.w, a2);
            }
            // a digit sum is at most 32 * 128 * 64 = 2^18; times 2^14 it would not fit an int32: recombine in F32
            // (each term is below 2^24 in magnitude and a multiple of its power of two, so the sum is exact to 2^-24 relative)
            const float v = (float)a2 * 16384.0f + ((float)a1 * 128.0f + (float)a0);
            acc = fmaf(d * inv_scale[b], v, acc);
        }
    }
    parts[warp * 32 + lane] = acc;
    __syncthreads();
    if (warp == 0 && lane < nrows) {
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < X8_WARPS; ++k) sum += parts[k * 32 + lane];
        out[(size_t)slot * out_stride + r0 + lane] = sum;
    }
}

// ---- the 32-element blocks of four- and five-bit codes: Q5_0, Q5_1, Q4_0, IQ4_NL (GGUF rows) -------------------
// The forms a 26B-A4B-style file keeps its down experts in (inference/src/models/gemma4.zig:259-268). The scheme is
// the Q8_0 kernel's: the block's 32 weight rows travel to shared memory as 4-byte copies, a lane per row and a warp per
// block of 32 columns, the digits of a block one broadcast address. What differs is how a block's bytes become the
// 32 codes dp4a takes: the 16 nibble bytes hold elements 0..15 in their low and 16..31 in their high nibbles
// (inference/src/quant/decode.zig:46-53), Q5_0 / Q5_1 add a bit from a 32-bit plane (:125-143), IQ4_NL looks the
// nibble up in a table of signed bytes (:73-81). The offset (-16 d, -8 d, or m) multiplies the F32 sum of the
// block's 32 inputs, prepared once with the digits.
enum NibbleKind : int { NK_Q5_0 = 0, NK_Q5_1 = 1, NK_Q4_0 = 2, NK_IQ4_NL = 3 };

template <int KIND>
__global__ void __launch_bounds__(X8_WARPS * 32) expert_gemv_nibble_kernel(const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                                                                           uint32_t blocks, const uint32_t *indices, const float *in, size_t in_stride,
                                                                           uint32_t in_group, float *out, size_t out_stride) {
    constexpr uint32_t BS = KIND == NK_Q5_0 ? 22u : KIND == NK_Q5_1 ? 24u : 18u;          // bytes of a block
    constexpr uint32_t QS = KIND == NK_Q5_0 ? 6u : KIND == NK_Q5_1 ? 8u : 2u;             // where its nibble bytes start
    constexpr bool FIFTH = KIND == NK_Q5_0 || KIND == NK_Q5_1;
    // [32 weight rows, `pitch` words each (+ one word: a shifted read may touch the word after a row)][3 planes of digits,
    // blocks * 32 bytes each][blocks (inverse scale, sum of x) pairs][8 x 32 part sums]
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t words = blocks * BS / 4;
    const uint32_t pitch = words | 1u;
    uint32_t *tile = (uint32_t *)smem;
    uint8_t *planes = smem + (((size_t)(X8_ROWS * pitch + 1) * 4 + 15) & ~(size_t)15);
    const uint32_t plane = blocks * 32;
    float2 *chunk = (float2 *)(planes + 3 * plane);
    float *parts = (float *)(chunk + blocks);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t slot = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t expert = min(indices[slot], experts - 1);
    const uint32_t r0 = blockIdx.x * X8_ROWS;
    const uint32_t nrows = min((uint32_t)X8_ROWS, rows - r0);
    const uint8_t *base = w + (size_t)expert * expert_bytes + (size_t)r0 * stride;
    for (uint32_t r = warp; r < nrows; r += X8_WARPS) {
        const uint8_t *src = base + (size_t)r * stride;
        uint32_t *dst = tile + r * pitch;
        for (uint32_t c = lane; c < words; c += 32) cp_async4(dst + c, src + c * 4);
    }
    cp_async_commit();

    const float *x = in + (size_t)(slot / in_group) * in_stride;
    for (uint32_t b = warp; b < blocks; b += X8_WARPS) {
        const float v = __ldg(x + b * 32 + lane);
        float mx = fabsf(v), bad = 0.0f * v, sum = v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            bad += __shfl_xor_sync(0xffffffffu, bad, o);
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        mx += bad;
        float scale, inv;
        chunk_scale(mx, scale, inv);
        int p0, p1, p2;
        digits(v, scale, p0, p1, p2);
        planes[b * 32 + lane] = (uint8_t)p0;
        planes[plane + b * 32 + lane] = (uint8_t)p1;
        planes[2 * plane + b * 32 + lane] = (uint8_t)p2;
        if (lane == 0) chunk[b] = make_float2(inv, sum);
    }
    cp_async_wait<0>();
    __syncthreads();
    float acc = 0.0f;
    if (lane < nrows) {
        const uint32_t *row = tile + lane * pitch;
        for (uint32_t b = warp; b < blocks; b += X8_WARPS) {
            // the block starts at byte BS b of the row, on a 2-byte boundary: its fields are read as aligned words shifted
            // into place (the shift is the same for the whole warp)
            const uint32_t off = b * BS, first = off >> 2, sh = (off & 2u) * 8u;
            constexpr int NW = (int)(BS + 3) / 4 + 1;
            uint32_t raw[NW];
#pragma unroll
            for (int i = 0; i < NW; ++i) raw[i] = row[first + i];
            uint32_t f[NW - 1];  // the block's bytes from its start, as words
#pragma unroll
            for (int i = 0; i < NW - 1; ++i) f[i] = __funnelshift_r(raw[i], raw[i + 1], sh);
            const float d = __half2float(__ushort_as_half((unsigned short)(f[0] & 0xffffu)));
            // the nibble bytes start at byte QS of the block: 2 mod 4 (their words straddle those of f) except for Q5_1
            uint32_t qs[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) qs[i] = __funnelshift_r(f[QS / 4 + i], f[QS / 4 + i + 1 < NW - 1 ? QS / 4 + i + 1 : NW - 2], (QS & 2u) * 8u);
            uint32_t high = 0;
            if (FIFTH) high = KIND == NK_Q5_0 ? __funnelshift_r(f[0], f[1], 16) : f[1];  // bytes 2..5 (Q5_0) or 4..7 (Q5_1)
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (KIND == NK_IQ4_NL) {
                    const uint32_t a = iq4_lookup4(qs[i]), c = iq4_lookup4(qs[i] >> 16);  // (lo0, hi0, lo1, hi1), (lo2, hi2, lo3, hi3)
                    lo[i] = prmt_b32(a, c, 0x6420u);
                    hi[i] = prmt_b32(a, c, 0x7531u);
                } else {
                    lo[i] = qs[i] & 0x0f0f0f0fu;
                    hi[i] = (qs[i] >> 4) & 0x0f0f0f0fu;
                    if (FIFTH) {
                        lo[i] |= bits4_to_bit4((high >> (4 * i)) & 15u);
                        hi[i] |= bits4_to_bit4((high >> (16 + 4 * i)) & 15u);
                    }
                }
            }
            const uint4 *dg = (const uint4 *)(planes + b * 32);
            const uint4 *dg1 = (const uint4 *)(planes + plane + b * 32), *dg2 = (const uint4 *)(planes + 2 * plane + b * 32);
            int a0 = 0, a1 = 0, a2 = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 q0 = dg[h], q1 = dg1[h], q2 = dg2[h];
                const uint32_t *c = h ? hi : lo;
                if (KIND == NK_IQ4_NL) {
                    a0 = dp4a_ss(c[0], q0.x, a0); a0 = dp4a_ss(c[1], q0.y, a0); a0 = dp4a_ss(c[2], q0.z, a0); a0 = dp4a_ss(c[3], q0.w, a0);
                    a1 = dp4a_ss(c[0], q1.x, a1); a1 = dp4a_ss(c[1], q1.y, a1); a1 = dp4a_ss(c[2], q1.z, a1); a1 = dp4a_ss(c[3], q1.w, a1);
                    a2 = dp4a_ss(c[0], q2.x, a2); a2 = dp4a_ss(c[1], q2.y, a2); a2 = dp4a_ss(c[2], q2.z, a2); a2 = dp4a_ss(c[3], q2.w, a2);
                } else {
                    a0 = dp4a_us(c[0], q0.x, a0); a0 = dp4a_us(c[1], q0.y, a0); a0 = dp4a_us(c[2], q0.z, a0); a0 = dp4a_us(c[3], q0.w, a0);
                    a1 = dp4a_us(c[0], q1.x, a1); a1 = dp4a_us(c[1], q1.y, a1); a1 = dp4a_us(c[2], q1.z, a1); a1 = dp4a_us(c[3], q1.w, a1);
                    a2 = dp4a_us(c[0], q2.x, a2); a2 = dp4a_us(c[1], q2.y, a2); a2 = dp4a_us(c[2], q2.z, a2); a2 = dp4a_us(c[3], q2.w, a2);
                }
            }
            // a digit sum is below 2^18; times 2^14 it would not fit an int32: recombine in F32 (exact to 2^-24 relative)
            const float v = (float)a2 * 16384.0f + ((float)a1 * 128.0f + (float)a0);
            const float2 ch = chunk[b];
            acc = fmaf(d * ch.x, v, acc);
            if (KIND == NK_Q5_0) acc = fmaf(-16.0f * d, ch.y, acc);
            if (KIND == NK_Q4_0) acc = fmaf(-8.0f * d, ch.y, acc);
            if (KIND == NK_Q5_1) acc = fmaf(__half2float(__ushort_as_half((unsigned short)(f[0] >> 16))), ch.y, acc);
        }
    }
    parts[warp * 32 + lane] = acc;
    __syncthreads();
    if (warp == 0 && lane < nrows) {
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < X8_WARPS; ++k) sum += parts[k * 32 + lane];
        out[(size_t)slot * out_stride + r0 + lane] = sum;
    }
}

}  // namespace

constexpr uint32_t kMaxColumns = 16384;  // shared memory: about 4 bytes a column

// Opts both kernels into their dynamic shared memory sizes. The attribute belongs to the device that
// is current, so this runs once per handle, with the handle's device current (fast_configure).
bool expert_gemv_configure() {
    return cudaFuncSetAttribute(expert_gemv_q4k_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(XQ_RING + kMaxColumns / 256 * (3 * 320 + 128))) == cudaSuccess &&
           cudaFuncSetAttribute(expert_gemv_q4k_kernel<ACT_SILU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(XQ_RING + kMaxColumns / 256 * (3 * 320 + 128))) == cudaSuccess &&
           cudaFuncSetAttribute(expert_gemv_q4k_kernel<ACT_GELU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(XQ_RING + kMaxColumns / 256 * (3 * 320 + 128))) == cudaSuccess &&
           cudaFuncSetAttribute(expert_gemv_q8_0_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess &&
           cudaFuncSetAttribute(expert_gemv_nibble_kernel<NK_Q5_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess &&
           cudaFuncSetAttribute(expert_gemv_nibble_kernel<NK_Q5_1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess &&
           cudaFuncSetAttribute(expert_gemv_nibble_kernel<NK_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess &&
           cudaFuncSetAttribute(expert_gemv_nibble_kernel<NK_IQ4_NL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess;
}

// Returns the number of kernels launched: 0 when the shape is not one of the specialized forms.
int launch_matvec_experts_fast(cudaStream_t s, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                               uint32_t columns, const uint32_t *indices, uint32_t slots, const float *in, size_t in_stride, uint32_t in_group,
                               float *out, size_t out_stride) {
    if (slots > 65535) return 0;
    if ((uintptr_t)in % 16 != 0 || in_stride % 4 != 0) return 0;
    // The blocks may be placed while the operator before drains (the kernels wait for it before they read anything).
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (enc == Q4_K) {
        if (columns % 256 != 0 || columns > kMaxColumns) return 0;
        if ((uintptr_t)w % 16 != 0 || stride % 16 != 0 || expert_bytes % 16 != 0) return 0;
        const uint32_t ksb = columns / 256;
        cfg.gridDim = dim3((rows + XQ_ROWS - 1) / XQ_ROWS, slots);
        cfg.blockDim = dim3(XQ_THREADS);
        cfg.dynamicSmemBytes = XQ_RING + (size_t)ksb * (3 * 320 + 128);
        cudaLaunchKernelEx(&cfg, expert_gemv_q4k_kernel<0>, w, stride, expert_bytes, experts, rows, ksb, indices, in, in_stride, in_group, out, out_stride);
        return 1;
    }
    if (enc == Q8_0) {
        // rows travel as 4-byte copies: an even number of 34-byte blocks, rows and experts on 4-byte boundaries
        if (columns % 64 != 0 || columns > kMaxColumns) return 0;
        if ((uintptr_t)w % 4 != 0 || stride % 4 != 0 || expert_bytes % 4 != 0) return 0;
        const uint32_t blocks = columns / 32;
        const uint32_t pitch = (blocks * 34 / 4) | 1u;
        const size_t smem = (((size_t)X8_ROWS * pitch * 4 + 15) & ~(size_t)15) + (size_t)blocks * (3 * 32 + 4) + X8_WARPS * 32 * 4;
        if (smem > 200 * 1024) return 0;
        cfg.gridDim = dim3((rows + X8_ROWS - 1) / X8_ROWS, slots);
        cfg.blockDim = dim3(X8_WARPS * 32);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchKernelEx(&cfg, expert_gemv_q8_0_kernel, w, stride, expert_bytes, experts, rows, blocks, indices, in, in_stride, in_group, out, out_stride);
        return 1;
    }
    if (enc == Q5_0 || enc == Q5_1 || enc == Q4_0 || enc == IQ4_NL) {
        // rows travel as 4-byte copies: rows of whole words (an even number of 18- or 22-byte blocks), rows and experts on
        // 4-byte boundaries
        const uint32_t bs = enc == Q5_0 ? 22u : enc == Q5_1 ? 24u : 18u;
        if (columns % 32 != 0 || columns > kMaxColumns) return 0;
        const uint32_t blocks = columns / 32;
        if ((blocks * bs) % 4 != 0 || (uintptr_t)w % 4 != 0 || stride % 4 != 0 || expert_bytes % 4 != 0) return 0;
        const uint32_t pitch = (blocks * bs / 4) | 1u;
        const size_t smem = (((size_t)(X8_ROWS * pitch + 1) * 4 + 15) & ~(size_t)15) + (size_t)blocks * (3 * 32 + 8) + X8_WARPS * 32 * 4;
        if (smem > 200 * 1024) return 0;
        cfg.gridDim = dim3((rows + X8_ROWS - 1) / X8_ROWS, slots);
        cfg.blockDim = dim3(X8_WARPS * 32);
        cfg.dynamicSmemBytes = smem;
        if (enc == Q5_0) cudaLaunchKernelEx(&cfg, expert_gemv_nibble_kernel<NK_Q5_0>, w, stride, expert_bytes, experts, rows, blocks, indices, in, in_stride, in_group, out, out_stride);
        else if (enc == Q5_1) cudaLaunchKernelEx(&cfg, expert_gemv_nibble_kernel<NK_Q5_1>, w, stride, expert_bytes, experts, rows, blocks, indices, in, in_stride, in_group, out, out_stride);
        else if (enc == Q4_0) cudaLaunchKernelEx(&cfg, expert_gemv_nibble_kernel<NK_Q4_0>, w, stride, expert_bytes, experts, rows, blocks, indices, in, in_stride, in_group, out, out_stride);
        else cudaLaunchKernelEx(&cfg, expert_gemv_nibble_kernel<NK_IQ4_NL>, w, stride, expert_bytes, experts, rows, blocks, indices, in, in_stride, in_group, out, out_stride);
        return 1;
    }
    return 0;
}

// The gate_up GEMV with the activation pass folded in: out[slot][i] = act(gate row i) * (up row i), i < rows / 2, for a
// Q4_K tensor of [gate rows][up rows] per expert. 0: not one of the specialized forms (the caller runs the two operators).
int launch_matvec_experts_gated_fast(cudaStream_t s, uint32_t act, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                                     uint32_t columns, const uint32_t *indices, uint32_t slots, const float *in, size_t in_stride, uint32_t in_group,
                                     float *out, size_t out_stride) {
    if (slots > 65535 || enc != Q4_K || rows % 2 != 0 || (act != ACT_SILU && act != ACT_GELU)) return 0;
    if ((uintptr_t)in % 16 != 0 || in_stride % 4 != 0) return 0;
    if (columns % 256 != 0 || columns > kMaxColumns) return 0;
    if ((uintptr_t)w % 16 != 0 || stride % 16 != 0 || expert_bytes % 16 != 0) return 0;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const uint32_t ksb = columns / 256;
    cfg.gridDim = dim3((rows / 2 + XQ_ROWS / 2 - 1) / (XQ_ROWS / 2), slots);
    cfg.blockDim = dim3(XQ_THREADS);
    cfg.dynamicSmemBytes = XQ_RING + (size_t)ksb * (3 * 320 + 128);
    if (act == ACT_SILU) cudaLaunchKernelEx(&cfg, expert_gemv_q4k_kernel<ACT_SILU>, w, stride, expert_bytes, experts, rows, ksb, indices, in, in_stride, in_group, out, out_stride);
    else cudaLaunchKernelEx(&cfg, expert_gemv_q4k_kernel<ACT_GELU>, w, stride, expert_bytes, experts, rows, ksb, indices, in, in_stride, in_group, out, out_stride);
    return 1;
}

}  // namespace nu
