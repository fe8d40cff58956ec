// Planar re-layout of block-quantized matrices (no reference analogue).
//
// GGUF stores a Q6_K row as 210-byte blocks, so rows and blocks start on 2-byte
// boundaries: no vector load and no bulk copy can address them. At load time
// (the moment the reference wraps a tensor, inference/src/backends/metal/root.zig:217-230)
// a matrix may be re-laid once into the same number of bytes:
//
//   Q6_K, layout 1 (rows a multiple of 16):
//     main plane  [rows][superblocks][208]: for t = 0..3 (half hh = t >> 1 of the block, column
//                 half ch = t & 1): 16 bytes ql[hh*64 + 16ch ..], 16 bytes ql[hh*64 + 32 + 16ch ..],
//                 16 bytes qh[hh*32 + 16ch ..]; then the 16 scale bytes
//     scale plane [superblocks][rows] f16: the d of each block, transposed
//
//   Q8_0, layout 2 (rows a multiple of 16, columns a multiple of 256):
//     code plane  [rows][columns] int8: the 32 codes of each block, blocks in row order
//     scale plane [columns/32][rows] f16: the d of each block, transposed
//
//   Q5_0, layout 3, and Q5_1, layout 4 (rows a multiple of 16, columns a multiple of 256):
//     main plane  [rows][superblocks of 256 columns][160]: the 16 nibble bytes of each of the eight blocks
//                 (128 bytes), then their eight 32-bit planes of high bits (32 bytes)
//     scale plane [superblocks][rows][8] f16: the d of the eight blocks of a row's superblock side by side;
//                 Q5_1: [superblocks][rows][16]: the eight d, then the eight m
//
//   Q4_0 and IQ4_NL, layout 5 (18-byte blocks: d, 16 nibble bytes; the same conditions):
//     main plane  [rows][superblocks][128]: the 16 nibble bytes of each of the eight blocks
//     scale plane [superblocks][rows][8] f16
//
//   IQ4_XS, layout 6 (136-byte superblocks: d, 16 bits and 4 bytes of scales, 128 nibble bytes; the same conditions):
//     main plane  [rows][superblocks][128]: the nibble bytes
//     header plane [superblocks][rows][8]: the first eight bytes of each superblock
//
//   Q2_K, layout 7 (84-byte superblocks: 16 scale bytes, 64 code bytes, d, dmin; the same conditions):
//     main plane  [rows][superblocks][80]: the scale and code bytes
//     tail plane  [superblocks][rows][4]: d, dmin
//
//   Q3_K, layout 8 (110-byte superblocks: 32 mask bytes, 64 code bytes, 12 scale bytes, d; the same conditions):
//     main plane  [rows][superblocks][96]: the mask and code bytes
//     tail plane  [superblocks][rows / 16][224]: the 12 scale bytes of each of 16 rows, then their 16 d
//
// Every byte is copied, none is changed: decoding the planar form gives the
// values of the GGUF form bit for bit (dequant16_planar in nu_device.cuh).
#include "kernels.hpp"
#include "nu_device.cuh"

namespace nu {

uint32_t prepared_layout(uint32_t enc, uint32_t rows, uint32_t columns) {
    if (enc == Q6_K && rows % 16 == 0 && columns % 256 == 0) return 1;
    if (enc == Q8_0 && rows % 16 == 0 && columns % 256 == 0) return 2;
    if (enc == Q5_0 && rows % 16 == 0 && columns % 256 == 0) return 3;
    if (enc == Q5_1 && rows % 16 == 0 && columns % 256 == 0) return 4;
    if ((enc == Q4_0 || enc == IQ4_NL) && rows % 16 == 0 && columns % 256 == 0) return 5;
    if (enc == IQ4_XS && rows % 16 == 0 && columns % 256 == 0) return 6;
    if (enc == Q2_K && rows % 16 == 0 && columns % 256 == 0) return 7;
    if (enc == Q3_K && rows % 16 == 0 && columns % 256 == 0) return 8;
    return 0;
}

__global__ void prepare_q6k_kernel(const uint8_t *src, uint8_t *dst, uint32_t rows, uint32_t ksb) {
    const size_t blocks = (size_t)rows * ksb;
    const size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= blocks * 210) return;
    const size_t block = id / 210;
    const uint32_t b = (uint32_t)(id % 210);
    const uint32_t row = (uint32_t)(block / ksb), sb = (uint32_t)(block % ksb);
    const uint8_t *in = src + block * 210;
    if (b < 192) {
        const uint32_t t = b / 48, part = (b % 48) / 16, j = b % 16, hh = t >> 1, ch = t & 1;
        const uint32_t from = part == 0 ? hh * 64 + 16 * ch + j : part == 1 ? hh * 64 + 32 + 16 * ch + j : 128 + hh * 32 + 16 * ch + j;
        dst[block * 208 + b] = in[from];
    } else if (b < 208) {
        dst[block * 208 + b] = in[b];
    } else {
        dst[blocks * 208 + ((size_t)sb * rows + row) * 2 + (b - 208)] = in[b];
    }
}

__global__ void prepare_q8_0_kernel(const uint8_t *src, uint8_t *dst, uint32_t rows, uint32_t kb) {
    const size_t blocks = (size_t)rows * kb;
    const size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= blocks * 34) return;
    const size_t block = id / 34;
    const uint32_t b = (uint32_t)(id % 34);
    const uint32_t row = (uint32_t)(block / kb), blk = (uint32_t)(block % kb);
    if (b >= 2) dst[block * 32 + (b - 2)] = src[id];
    else dst[blocks * 32 + ((size_t)blk * rows + row) * 2 + b] = src[id];
}

// Q5_0 (22-byte blocks: d, 4 bytes of high bits, 16 nibble bytes), Q5_1 (24: d, m, high bits, nibbles) and
// Q4_0 / IQ4_NL (18: d, nibbles). head: the bytes of scales a block starts with; high: its bytes of high bits (4 or 0).
__global__ void prepare_block32_kernel(const uint8_t *src, uint8_t *dst, uint32_t rows, uint32_t ksb, uint32_t head, uint32_t high) {
    const uint32_t block_bytes = head + high + 16, record = 128 + 8 * high;
    const size_t blocks = (size_t)rows * ksb * 8;
    const size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= blocks * block_bytes) return;
    const size_t block = id / block_bytes;
    const uint32_t b = (uint32_t)(id % block_bytes);
    const uint32_t row = (uint32_t)(block / (ksb * 8)), kb = (uint32_t)(block % (ksb * 8)), sb = kb / 8, c = kb % 8;
    uint8_t *rec = dst + ((size_t)row * ksb + sb) * record;
    if (b >= head + high) {
        rec[c * 16 + (b - head - high)] = src[id];
    } else if (b >= head) {
        rec[128 + c * 4 + (b - head)] = src[id];
    } else {
        // d: bytes 0, 1; m (Q5_1): bytes 2, 3
        uint8_t *sc = dst + (size_t)rows * ksb * record + ((size_t)sb * rows + row) * (head * 8);
        sc[(b / 2) * 16 + c * 2 + (b & 1)] = src[id];
    }
}

__global__ void prepare_iq4_xs_kernel(const uint8_t *src, uint8_t *dst, uint32_t rows, uint32_t ksb) {
    const size_t blocks = (size_t)rows * ksb;
    const size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= blocks * 136) return;
    const size_t block = id / 136;
    const uint32_t b = (uint32_t)(id % 136);
    const uint32_t row = (uint32_t)(block / ksb), sb = (uint32_t)(block % ksb);
    if (b >= 8) dst[block * 128 + (b - 8)] = src[id];
    else dst[blocks * 128 + ((size_t)sb * rows + row) * 8 + b] = src[id];
}

__global__ void prepare_q2k_kernel(const uint8_t *src, uint8_t *dst, uint32_t rows, uint32_t ksb) {
    const size_t blocks = (size_t)rows * ksb;
    const size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= blocks * 84) return;
    const size_t block = id / 84;
    const uint32_t b = (uint32_t)(id % 84);
    const uint32_t row = (uint32_t)(block / ksb), sb = (uint32_t)(block % ksb);
    if (b < 80) dst[block * 80 + b] = src[id];
    else dst[blocks * 80 + ((size_t)sb * rows + row) * 4 + (b - 80)] = src[id];
}

__global__ void prepare_q3k_kernel(const uint8_t *src, uint8_t *dst, uint32_t rows, uint32_t ksb) {
    const size_t blocks = (size_t)rows * ksb;
    const size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= blocks * 110) return;
    const size_t block = id / 110;
    const uint32_t b = (uint32_t)(id % 110);
    const uint32_t row = (uint32_t)(block / ksb), sb = (uint32_t)(block % ksb);
    if (b < 96) {
        dst[block * 96 + b] = src[id];
        return;
    }
    uint8_t *tile = dst + blocks * 96 + ((size_t)sb * (rows / 16) + row / 16) * 224;
    if (b < 108) tile[(row % 16) * 12 + (b - 96)] = src[id];
    else tile[192 + (row % 16) * 2 + (b - 108)] = src[id];
}

__global__ void copy_bytes_kernel(const uint8_t *src, uint8_t *dst, size_t n) {
    const size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id < n) dst[id] = src[id];
}

int launch_prepare(cudaStream_t s, uint32_t enc, const uint8_t *src, uint8_t *dst, uint32_t rows, uint32_t columns) {
    const Layout l = layout(enc);
    const size_t bytes = (size_t)rows * (columns / l.elements) * l.bytes;
    const uint32_t to = prepared_layout(enc, rows, columns);
    if (to == 1) {
        prepare_q6k_kernel<<<(unsigned)((bytes + 255) / 256), 256, 0, s>>>(src, dst, rows, columns / 256);
    } else if (to == 2) {
        prepare_q8_0_kernel<<<(unsigned)((bytes + 255) / 256), 256, 0, s>>>(src, dst, rows, columns / 32);
    } else if (to == 3 || to == 4 || to == 5) {
        const uint32_t high = to == 5 ? 0u : 4u;
        prepare_block32_kernel<<<(unsigned)((bytes + 255) / 256), 256, 0, s>>>(src, dst, rows, columns / 256, (uint32_t)l.bytes - 16u - high, high);
    } else if (to == 7) {
        prepare_q2k_kernel<<<(unsigned)((bytes + 255) / 256), 256, 0, s>>>(src, dst, rows, columns / 256);
    } else if (to == 8) {
        prepare_q3k_kernel<<<(unsigned)((bytes + 255) / 256), 256, 0, s>>>(src, dst, rows, columns / 256);
    } else if (to == 6) {
        prepare_iq4_xs_kernel<<<(unsigned)((bytes + 255) / 256), 256, 0, s>>>(src, dst, rows, columns / 256);
    } else {
        copy_bytes_kernel<<<(unsigned)((bytes + 255) / 256), 256, 0, s>>>(src, dst, bytes);
    }
    return 1;
}

}  // namespace nu
