// Device-side block decoders shared by every kernel that must agree bit for
// bit with the CPU decoder (quant.row, inference/src/quant/decode.zig:30-103).
// Byte-indexed exactly like the reference so any alignment works; the fast
// kernels have their own packed unpackers and are checked against these.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace nu {

enum Encoding : uint32_t { F32 = 0, F16 = 1, Q4_0 = 2, Q5_0 = 6, Q5_1 = 7, Q8_0 = 8, Q2_K = 10, Q3_K = 11, Q4_K = 12, Q5_K = 13, Q6_K = 14, IQ4_NL = 20, IQ4_XS = 23, BF16 = 30 };

struct Layout { uint32_t elements, bytes; };

// encoding.zig:29-56 for the encodings this library serves; elements == 0 means unknown.
__host__ __device__ inline Layout layout(uint32_t id) {
    switch (id) {
    case F32: return {1, 4};
    case F16: return {1, 2};
    case Q4_0: return {32, 18};
    case Q5_0: return {32, 22};
    case Q5_1: return {32, 24};
    case Q8_0: return {32, 34};
    case Q2_K: return {256, 84};
    case Q3_K: return {256, 110};
    case Q4_K: return {256, 144};
    case Q5_K: return {256, 176};
    case Q6_K: return {256, 210};
    case IQ4_NL: return {32, 18};
    case IQ4_XS: return {256, 136};
    case BF16: return {1, 2};
    default: return {0, 0};
    }
}

// decode.zig:432-435: little-endian binary16 widened exactly.
__device__ __forceinline__ float half_at(const uint8_t *p) {
    const unsigned short bits = (unsigned short)p[0] | ((unsigned short)p[1] << 8);
    return __half2float(__ushort_as_half(bits));
}

// The sixteen values a four-bit IQ4 code selects (decode.zig:437), packed four to a word so that the
// lookup is a shift and a sign extension instead of a table in local memory.
__device__ __forceinline__ int iq4_value(uint32_t code) {
    const uint32_t w = code < 8 ? (code < 4 ? 0xbfad9881u : 0xf6eaddcfu) : (code < 12 ? 0x26190d01u : 0x71594535u);
    return (int)(int8_t)(w >> ((code & 3u) * 8));
}

// ---- packed forms of the same lookups, for the kernels that keep four codes in a word ----
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// The IQ4 values of the four nibbles in the low 16 bits of n, as signed bytes in nibble order. A permute takes a nibble's
// low three bits as a byte index into eight table entries; the entries 8..15 come from a second permute, and a third (in
// its sign-replicating mode, on n and n << 4, whose bytes have the nibbles' top bits as their signs) makes the byte mask
// that picks between the two.
__device__ __forceinline__ uint32_t iq4_lookup4(uint32_t n) {
    const uint32_t sel = n & 0x7777u;
    const uint32_t lo = prmt_b32(0xbfad9881u, 0xf6eaddcfu, sel), hi = prmt_b32(0x26190d01u, 0x71594535u, sel);
    const uint32_t upper = prmt_b32(n, n << 4, 0x9d8cu);
    return (lo & ~upper) | (hi & upper);
}
// Four bits of x into bit 4 of four bytes: bit i of x lands on bit 8 i of x * 0x00204081 (no two terms meet).
__device__ __forceinline__ uint32_t bits4_to_bit4(uint32_t x) { return ((x * 0x00204081u) & 0x01010101u) << 4; }

// Decodes the 16 consecutive values [16*seg, 16*seg+16) of one row.
// Products and the subtraction are separate IEEE operations (no contraction),
// as in the reference: (d*s)*q - (dmin*m) for Q4_K, (d*scale)*q for Q6_K.
__device__ __forceinline__ void dequant16(uint32_t enc, const uint8_t *row, uint32_t seg, float out[16]) {
    const uint32_t first = seg * 16;
    switch (enc) {
    case F32:
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint8_t *p = row + (size_t)(first + i) * 4;
            out[i] = __uint_as_float((uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24));
        }
        break;
    case F16:
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = half_at(row + (size_t)(first + i) * 2);
        break;
    case BF16:
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint8_t *p = row + (size_t)(first + i) * 2;
            out[i] = __uint_as_float(((uint32_t)p[0] | ((uint32_t)p[1] << 8)) << 16);
        }
        break;
    case Q8_0: {
        const uint8_t *block = row + (size_t)(first / 32) * 34;
        const float d = half_at(block);
        const uint8_t *q = block + 2 + (first % 32);
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = __fmul_rn(d, (float)(int8_t)q[i]);
        break;
    }
    case Q4_0: {
        // decode.zig:46-53: low nibbles are the first half of the block, high nibbles the second; code - 8
        const uint8_t *block = row + (size_t)(first / 32) * 18;
        const float d = half_at(block);
        const uint32_t shift = ((first % 32) / 16) * 4;
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = __fmul_rn(d, (float)((int)((block[2 + i] >> shift) & 15u) - 8));
        break;
    }
    case Q5_0:
    case Q5_1: {
        // decode.zig:125-143: Q4_0's nibble order, each code completed by its bit of the 32-bit plane
        const bool offset = enc == Q5_1;
        const uint8_t *block = row + (size_t)(first / 32) * (offset ? 24 : 22);
        const float d = half_at(block);
        const float m = offset ? half_at(block + 2) : 0.0f;
        const uint8_t *plane = block + (offset ? 4 : 2);
        const uint32_t qh = (uint32_t)plane[0] | ((uint32_t)plane[1] << 8) | ((uint32_t)plane[2] << 16) | ((uint32_t)plane[3] << 24);
        const uint32_t hi = (first % 32) / 16;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int q = (int)(((plane[4 + i] >> (hi * 4)) & 15u) | (((qh >> (i + hi * 16)) & 1u) << 4));
            out[i] = offset ? __fadd_rn(__fmul_rn(d, (float)q), m) : __fmul_rn(d, (float)(q - 16));
        }
        break;
    }
    case IQ4_NL: {
        // decode.zig:73-81: d * table[code]; low nibbles are the first 16 values of the block, high nibbles the next 16
        const uint8_t *block = row + (size_t)(first / 32) * 18;
        const float d = half_at(block);
        const uint32_t shift = ((first % 32) / 16) * 4;
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = __fmul_rn(d, (float)iq4_value((block[2 + i] >> shift) & 15u));
        break;
    }
    case IQ4_XS: {
        // decode.zig:214-228: eight groups of 32 under a six-bit scale biased by 32; the 16 values are half a group
        const uint8_t *block = row + (size_t)(first / 256) * 136;
        const uint32_t i0 = first % 256, g = i0 / 32;
        const uint32_t high = (uint32_t)block[2] | ((uint32_t)block[3] << 8);
        const uint32_t low = (block[4 + g / 2] >> (4 * (g % 2))) & 15u;
        const int scale = (int)(low | (((high >> (2 * g)) & 3u) << 4)) - 32;
        const float multiplier = __fmul_rn(half_at(block), (float)scale);
        const uint8_t *q = block + 8 + g * 16;
        const uint32_t shift = ((i0 % 32) / 16) * 4;
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = __fmul_rn(multiplier, (float)iq4_value((q[i] >> shift) & 15u));
        break;
    }
    case Q2_K: {
        // decode.zig:260-275: the 16 values are one group: a four-bit scale and minimum, two-bit codes in bit planes
        const uint8_t *block = row + (size_t)(first / 256) * 84;
        const uint32_t i0 = first % 256, g = i0 / 16;
        const float multiplier = __fmul_rn(half_at(block + 80), (float)(block[g] & 15u));
        const float offset = __fmul_rn(half_at(block + 82), (float)(block[g] >> 4));
        const uint8_t *q = block + 16 + (i0 / 128) * 32 + i0 % 32;
        const uint32_t shift = 2 * ((i0 % 128) / 32);
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = __fsub_rn(__fmul_rn(multiplier, (float)((q[i] >> shift) & 3u)), offset);
        break;
    }
    case Q3_K: {
        // decode.zig:174-196: biased six-bit scales; a clear high-mask bit means subtract four
        const uint8_t *block = row + (size_t)(first / 256) * 110;
        const uint32_t i0 = first % 256, g = i0 / 16;
        const uint8_t *scales = block + 96;
        const uint32_t nibble = g < 8 ? (scales[g] & 15u) : (uint32_t)(scales[g - 8] >> 4);
        const uint32_t upper = ((uint32_t)scales[8 + g % 4] >> (2 * (g / 4))) & 3u;
        const float multiplier = __fmul_rn(half_at(block + 108), (float)((int)(nibble | (upper << 4)) - 32));
        const uint8_t *q = block + 32 + (i0 / 128) * 32 + i0 % 32;
        const uint8_t *mask = block + i0 % 32;
        const uint32_t low_shift = 2 * ((i0 % 128) / 32), sign_shift = i0 / 32;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int low = (int)((q[i] >> low_shift) & 3u);
            out[i] = __fmul_rn(multiplier, (float)(low - (((mask[i] >> sign_shift) & 1u) ? 0 : 4)));
        }
        break;
    }
    case Q4_K:
    case Q5_K: {
        // decode.zig:147-170; Q5_K: 32 bytes of high bits at 16 (bit g of byte c belongs to group g), the nibbles after them
        const bool fifth = enc == Q5_K;
        const uint8_t *block = row + (size_t)(first / 256) * (fifth ? 176 : 144);
        const uint32_t in_block = first % 256;
        const uint32_t g = in_block / 32, c0 = in_block % 32;
        const uint8_t *sc = block + 4;
        uint32_t s, m;
        if (g < 4) {
            s = sc[g] & 63u;
            m = sc[g + 4] & 63u;
        } else {
            s = (sc[g + 4] & 15u) | ((uint32_t)(sc[g - 4] >> 6) << 4);
            m = (uint32_t)(sc[g + 4] >> 4) | ((uint32_t)(sc[g] >> 6) << 4);
        }
        const float multiplier = __fmul_rn(half_at(block), (float)s);
        const float offset = __fmul_rn(half_at(block + 2), (float)m);
        const uint8_t *qs = block + (fifth ? 48 : 16) + (g / 2) * 32 + c0;
        const uint32_t shift = (g & 1u) * 4;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            uint32_t q = (qs[i] >> shift) & 15u;
            if (fifth) q |= (((uint32_t)block[16 + c0 + i] >> g) & 1u) << 4;
            out[i] = __fsub_rn(__fmul_rn(multiplier, (float)q), offset);
        }
        break;
    }
    case Q6_K: {
        const uint8_t *block = row + (size_t)(first / 256) * 210;
        const uint32_t i0 = first % 256;
        const uint32_t hh = i0 / 128, quarter = (i0 % 128) / 32, c0 = i0 % 32;
        const float d = half_at(block + 208);
        const float ds = __fmul_rn(d, (float)(int8_t)block[192 + i0 / 16]);
        const uint8_t *ql = block + hh * 64 + (quarter % 2) * 32 + c0;
        const uint8_t *qh = block + 128 + hh * 32 + c0;
        const uint32_t low_shift = (quarter / 2) * 4, high_shift = quarter * 2;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int value = (int)(((ql[i] >> low_shift) & 15u) | (((qh[i] >> high_shift) & 3u) << 4)) - 32;
            out[i] = __fmul_rn(ds, (float)value);
        }
        break;
    }
    default:
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = 0.0f;
    }
}

// The same 16 values from the planar form of a Q6_K matrix (prepare.cu): `base` is the start of the
// matrix, `row` the row index. Bit-identical to dequant16 on the GGUF form.
__device__ __forceinline__ void dequant16_planar_q6k(const uint8_t *base, uint32_t rows, uint32_t ksb, uint32_t row, uint32_t seg, float out[16]) {
    const uint32_t sb = seg / 16, i0 = (seg % 16) * 16;
    const uint32_t hh = i0 / 128, quarter = (i0 % 128) / 32, ch = (i0 % 32) / 16, t = hh * 2 + ch;
    const uint8_t *rec = base + ((size_t)row * ksb + sb) * 208;
    const uint8_t *dp = base + (size_t)rows * ksb * 208 + ((size_t)sb * rows + row) * 2;
    const float ds = __fmul_rn(half_at(dp), (float)(int8_t)rec[192 + i0 / 16]);
    const uint8_t *ql = rec + t * 48 + (quarter % 2) * 16;
    const uint8_t *qh = rec + t * 48 + 32;
    const uint32_t low_shift = (quarter / 2) * 4, high_shift = quarter * 2;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int value = (int)(((ql[i] >> low_shift) & 15u) | (((qh[i] >> high_shift) & 3u) << 4)) - 32;
        out[i] = __fmul_rn(ds, (float)value);
    }
}

// The same from the planar form of a Q8_0 matrix (prepare.cu).
__device__ __forceinline__ void dequant16_planar_q8_0(const uint8_t *base, uint32_t rows, uint32_t columns, uint32_t row, uint32_t seg, float out[16]) {
    const uint8_t *q = base + (size_t)row * columns + (size_t)seg * 16;
    const uint8_t *dp = base + (size_t)rows * columns + ((size_t)(seg / 2) * rows + row) * 2;
    const float d = half_at(dp);
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = __fmul_rn(d, (float)(int8_t)q[i]);
}

// The same from the planar form of a Q5_0, Q5_1, Q4_0 or IQ4_NL matrix (prepare.cu): 16 values are one half of a block.
__device__ __forceinline__ void dequant16_planar_block32(uint32_t enc, const uint8_t *base, uint32_t rows, uint32_t ksb, uint32_t row, uint32_t seg, float out[16]) {
    const bool offset = enc == Q5_1, fifth = enc == Q5_0 || enc == Q5_1;
    const uint32_t record = fifth ? 160 : 128;
    const uint32_t sb = seg / 16, c = (seg % 16) / 2, hi = seg % 2;
    const uint8_t *rec = base + ((size_t)row * ksb + sb) * record;
    const uint8_t *sc = base + (size_t)rows * ksb * record + ((size_t)sb * rows + row) * (offset ? 32 : 16);
    const float d = half_at(sc + c * 2), m = offset ? half_at(sc + 16 + c * 2) : 0.0f;
    uint32_t qh = 0;
    if (fifth) {
        const uint8_t *plane = rec + 128 + c * 4;
        qh = (uint32_t)plane[0] | ((uint32_t)plane[1] << 8) | ((uint32_t)plane[2] << 16) | ((uint32_t)plane[3] << 24);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t code = (rec[c * 16 + i] >> (hi * 4)) & 15u;
        const int q = (int)(code | (((qh >> (i + hi * 16)) & 1u) << 4));
        out[i] = enc == IQ4_NL ? __fmul_rn(d, (float)iq4_value(code)) : enc == Q4_0 ? __fmul_rn(d, (float)(q - 8)) : offset ? __fadd_rn(__fmul_rn(d, (float)q), m) : __fmul_rn(d, (float)(q - 16));
    }
}

// The same from the planar form of an IQ4_XS matrix (prepare.cu).
__device__ __forceinline__ void dequant16_planar_iq4_xs(const uint8_t *base, uint32_t rows, uint32_t ksb, uint32_t row, uint32_t seg, float out[16]) {
    const uint32_t sb = seg / 16, g = (seg % 16) / 2, hi = seg % 2;
    const uint8_t *q = base + ((size_t)row * ksb + sb) * 128 + g * 16;
    const uint8_t *hdr = base + (size_t)rows * ksb * 128 + ((size_t)sb * rows + row) * 8;
    const uint32_t high = (uint32_t)hdr[2] | ((uint32_t)hdr[3] << 8);
    const uint32_t low = (hdr[4 + g / 2] >> (4 * (g % 2))) & 15u;
    const int scale = (int)(low | (((high >> (2 * g)) & 3u) << 4)) - 32;
    const float multiplier = __fmul_rn(half_at(hdr), (float)scale);
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = __fmul_rn(multiplier, (float)iq4_value((q[i] >> (hi * 4)) & 15u));
}

// The same from the planar forms of Q2_K and Q3_K matrices (prepare.cu).
__device__ __forceinline__ void dequant16_planar_q2k(const uint8_t *base, uint32_t rows, uint32_t ksb, uint32_t row, uint32_t seg, float out[16]) {
    const uint32_t sb = seg / 16, g = seg % 16, i0 = g * 16;
    const uint8_t *rec = base + ((size_t)row * ksb + sb) * 80;
    const uint8_t *tail = base + (size_t)rows * ksb * 80 + ((size_t)sb * rows + row) * 4;
    const float multiplier = __fmul_rn(half_at(tail), (float)(rec[g] & 15u));
    const float offset = __fmul_rn(half_at(tail + 2), (float)(rec[g] >> 4));
    const uint8_t *q = rec + 16 + (i0 / 128) * 32 + i0 % 32;
    const uint32_t shift = 2 * ((i0 % 128) / 32);
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = __fsub_rn(__fmul_rn(multiplier, (float)((q[i] >> shift) & 3u)), offset);
}
__device__ __forceinline__ void dequant16_planar_q3k(const uint8_t *base, uint32_t rows, uint32_t ksb, uint32_t row, uint32_t seg, float out[16]) {
    const uint32_t sb = seg / 16, g = seg % 16, i0 = g * 16;
    const uint8_t *rec = base + ((size_t)row * ksb + sb) * 96;
    const uint8_t *tile = base + (size_t)rows * ksb * 96 + ((size_t)sb * (rows / 16) + row / 16) * 224;
    const uint8_t *scales = tile + (row % 16) * 12;
    const uint32_t nibble = g < 8 ? (scales[g] & 15u) : (uint32_t)(scales[g - 8] >> 4);
    const uint32_t upper = ((uint32_t)scales[8 + g % 4] >> (2 * (g / 4))) & 3u;
    const float multiplier = __fmul_rn(half_at(tile + 192 + (row % 16) * 2), (float)((int)(nibble | (upper << 4)) - 32));
    const uint8_t *q = rec + 32 + (i0 / 128) * 32 + i0 % 32;
    const uint8_t *mask = rec + i0 % 32;
    const uint32_t low_shift = 2 * ((i0 % 128) / 32), sign_shift = i0 / 32;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int low = (int)((q[i] >> low_shift) & 3u);
        out[i] = __fmul_rn(multiplier, (float)(low - (((mask[i] >> sign_shift) & 1u) ? 0 : 4)));
    }
}

// F32 forms of the activations, as the reference's GPU kernels compute them
// (inference/src/backends/metal/kernels/common.metal:6-16).
__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float tanh_clamped(float x) { return tanhf(fminf(fmaxf(x, -20.0f), 20.0f)); }
__device__ __forceinline__ float gelu_f32(float x) {
    return 0.5f * x * (1.0f + tanh_clamped(0.7978845608028654f * x * (1.0f + 0.044715f * x * x)));
}

}  // namespace nu
