// Expert GEMV for the decode form of a mixture-of-experts layer: one launch multiplies every routed
// slot's input by the matrix of the expert the slot selected (Backend.matvecExperts /
// matvecExpertsGrouped, inference/src/backends/metal/ops/experts.zig:36-77; the reference's kernel
// is nu_matvec_experts, kernels/experts.metal:16-36). Specialized for the two forms an expert
// tensor of the 26B-A4B-style layer is stored in: Q4_K (gate_up, [experts][2 ff][hidden]) and
// GGUF Q8_0 (down, [experts][hidden][ff] with ff = 704 = 22 blocks); everything else stays on the
// generic kernel.
//
// The work is a few to a few hundred megabytes spread over up to 64 small matrices picked by
// device-side indices, so the kernels use plain loads instead of tensor maps (an expert's address is
// known only on the device) and aim at keeping enough 16-byte loads in flight:
//  * Q4_K: 8 lanes per weight row, 4 rows per warp, 32 rows per block. Lane p of a row takes the
//    16-byte piece p of each superblock's 128 quant bytes: 16 low nibbles of group 2(p/2) and 16 high
//    nibbles of group 2(p/2)+1, columns 16(p&1).. of each. Bytes become floats through the 2^23 magic
//    number (one permute, one subtract), products accumulate in F32; the group's d*scale and dmin*min
//    are applied once per piece, the minimum against a sum of x that the block prepares once per
//    16 columns. The slot's input row is staged in shared memory once per block.
//  * Q8_0: a warp per weight row; a lane takes 8-code quarters of the 34-byte blocks (2-byte aligned,
//    so 16-bit loads), x comes through the read-only cache.
// Sums run in a fixed order: results do not depend on timing.
#include "kernels.hpp"
#include "nu_device.cuh"

namespace nu {
namespace {

constexpr int XQ_THREADS = 256;
constexpr int XQ_ROWS = 32;  // weight rows per block: 8 lanes each

__device__ __forceinline__ uint4 ldg_stream16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// byte b of w as a float: 0x4b0000bb is 2^23 + b
__device__ __forceinline__ float byte_f32(uint32_t w, int b, float bias = 8388608.0f) { return __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7650u + b)) - bias; }

// 6-bit scale and minimum of group g of a Q4_K superblock; y, z, w are scale bytes 0..3, 4..7, 8..11.
__device__ __forceinline__ void q4k_scale_min(uint32_t y, uint32_t z, uint32_t w, uint32_t g, float &s, float &m) {
    const uint32_t sh = (g & 3u) * 8;
    const uint32_t by = (y >> sh) & 0xffu, bz = (z >> sh) & 0xffu, bw = (w >> sh) & 0xffu;
    if (g < 4) {
        s = (float)(by & 63u);
        m = (float)(bz & 63u);
    } else {
        s = (float)((bw & 15u) | ((by >> 6) << 4));
        m = (float)((bw >> 4) | ((bz >> 6) << 4));
    }
}

#ifndef NU_XQ_BATCH
#define NU_XQ_BATCH 1
#endif
constexpr int XQ_BATCH = NU_XQ_BATCH;  // superblocks whose bytes a lane requests before it uses any

// One piece (16 quant bytes, this lane's two half groups) of one superblock against the staged input.
__device__ __forceinline__ float q4k_piece(const uint4 &hdr, const uint4 &q, const float *xs, const float *sums, uint32_t sb, uint32_t p) {
    const uint32_t g_lo = 2 * (p >> 1), g_hi = g_lo + 1;
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    float s_lo, m_lo, s_hi, m_hi;
    q4k_scale_min(hdr.y, hdr.z, hdr.w, g_lo, s_lo, m_lo);
    q4k_scale_min(hdr.y, hdr.z, hdr.w, g_hi, s_hi, m_hi);
    const float *x_lo = xs + sb * 272 + (p >> 1) * 68 + (p & 1u) * 16, *x_hi = x_lo + 32;
    float a_lo = 0.0f, a_hi = 0.0f;
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = qw[i] & 0x0f0f0f0fu, hi = (qw[i] >> 4) & 0x0f0f0f0fu;
        const float4 xl = *(const float4 *)(x_lo + 4 * i), xh = *(const float4 *)(x_hi + 4 * i);
        a_lo = fmaf(byte_f32(lo, 0), xl.x, a_lo); a_lo = fmaf(byte_f32(lo, 1), xl.y, a_lo);
        a_lo = fmaf(byte_f32(lo, 2), xl.z, a_lo); a_lo = fmaf(byte_f32(lo, 3), xl.w, a_lo);
        a_hi = fmaf(byte_f32(hi, 0), xh.x, a_hi); a_hi = fmaf(byte_f32(hi, 1), xh.y, a_hi);
        a_hi = fmaf(byte_f32(hi, 2), xh.z, a_hi); a_hi = fmaf(byte_f32(hi, 3), xh.w, a_hi);
    }
    const float sum_lo = sums[sb * 16 + g_lo * 2 + (p & 1u)], sum_hi = sums[sb * 16 + g_hi * 2 + (p & 1u)];
    float acc = d * s_lo * a_lo;
    acc = fmaf(d * s_hi, a_hi, acc);
    acc = fmaf(-(dmin * m_lo), sum_lo, acc);
    return fmaf(-(dmin * m_hi), sum_hi, acc);
}

__global__ void __launch_bounds__(XQ_THREADS) expert_gemv_q4k_kernel(const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                                                                     uint32_t ksb, const uint32_t *indices, const float *in, size_t in_stride,
                                                                     uint32_t in_group, float *out, size_t out_stride) {
    // [ksb * 272] the slot's input row, every 64 columns followed by 4 floats of padding (the eight lanes of a
    // weight row then read from eight different groups of banks), then [ksb * 16] sums of 16 columns
    extern __shared__ __align__(16) float xs[];
    float *sums = xs + ksb * 272;
    // launched so that its blocks may be placed while the operator before it drains; nothing is read before this
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t slot = blockIdx.y;
    const uint32_t r = blockIdx.x * XQ_ROWS + (threadIdx.x >> 3), p = threadIdx.x & 7;
    const bool live = r < rows;
    // A corrupt routing buffer can never read past the tensor (experts.metal:25).
    const uint32_t expert = min(indices[slot], experts - 1);
    const uint8_t *row = w + (size_t)expert * expert_bytes + (size_t)(live ? r : 0) * stride;
    // the first batch of weight bytes is requested before the input row is staged
    uint4 hdr[XQ_BATCH], q[XQ_BATCH];
#pragma unroll
    for (int j = 0; j < XQ_BATCH; ++j)
        if (live && (uint32_t)j < ksb) {
            hdr[j] = ldg_stream16(row + (size_t)j * 144);
            q[j] = ldg_stream16(row + (size_t)j * 144 + 16 + p * 16);
        }
    const float *x = in + (size_t)(slot / in_group) * in_stride;
    for (uint32_t i = threadIdx.x; i < ksb * 64; i += XQ_THREADS) ((float4 *)xs)[i + (i >> 4)] = __ldg((const float4 *)x + i);
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < ksb * 16; i += XQ_THREADS) {
        const float4 *src = (const float4 *)xs + i * 4 + (i >> 2);
        const float4 a = src[0], b = src[1], c = src[2], d = src[3];
        sums[i] = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w)) + (((c.x + c.y) + (c.z + c.w)) + ((d.x + d.y) + (d.z + d.w)));
    }
    __syncthreads();
    float acc = 0.0f;
    if (live) {
        for (uint32_t sb0 = 0; sb0 < ksb; sb0 += XQ_BATCH) {
            if (sb0) {
#pragma unroll
                for (int j = 0; j < XQ_BATCH; ++j)
                    if (sb0 + j < ksb) {
                        hdr[j] = ldg_stream16(row + (size_t)(sb0 + j) * 144);
                        q[j] = ldg_stream16(row + (size_t)(sb0 + j) * 144 + 16 + p * 16);
                    }
            }
#pragma unroll
            for (int j = 0; j < XQ_BATCH; ++j)
                if (sb0 + j < ksb) acc += q4k_piece(hdr[j], q[j], xs, sums, sb0 + j, p);
        }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (p == 0 && live) out[(size_t)slot * out_stride + r] = acc;
}

constexpr int X8_WARPS = 8;  // weight rows per block
#ifndef NU_X8_BATCH
#define NU_X8_BATCH 1
#endif
constexpr int X8_BATCH = NU_X8_BATCH;  // quarters whose bytes a lane requests before it uses any (a 704-column row: 88 quarters, 3 per lane)

__global__ void __launch_bounds__(X8_WARPS * 32) expert_gemv_q8_0_kernel(const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                                                                         uint32_t blocks, const uint32_t *indices, const float *in, size_t in_stride,
                                                                         uint32_t in_group, float *out, size_t out_stride) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t slot = blockIdx.y, lane = threadIdx.x & 31;
    const uint32_t r = blockIdx.x * X8_WARPS + (threadIdx.x >> 5);
    if (r >= rows) return;
    const uint32_t expert = min(indices[slot], experts - 1);
    const uint8_t *row = w + (size_t)expert * expert_bytes + (size_t)r * stride;
    const float *x = in + (size_t)(slot / in_group) * in_stride;
    float acc = 0.0f;
    // quarter qi of the row: block qi / 4, codes 8 (qi & 3) .. +7
    for (uint32_t q0 = lane; q0 < blocks * 4; q0 += 32 * X8_BATCH) {
        unsigned short dh[X8_BATCH], c[X8_BATCH][4];
        float4 xa[X8_BATCH], xb[X8_BATCH];
#pragma unroll
        for (int j = 0; j < X8_BATCH; ++j) {
            const uint32_t qi = q0 + 32 * j;
            if (qi < blocks * 4) {
                const uint8_t *blk = row + (size_t)(qi >> 2) * 34;
                const unsigned short *codes = (const unsigned short *)(blk + 2 + (qi & 3u) * 8);
                dh[j] = __ldg((const unsigned short *)blk);
#pragma unroll
                for (int i = 0; i < 4; ++i) c[j][i] = __ldg(codes + i);
                const float *xp = x + (qi >> 2) * 32 + (qi & 3u) * 8;
                xa[j] = __ldg((const float4 *)xp);
                xb[j] = __ldg((const float4 *)xp + 1);
            }
        }
#pragma unroll
        for (int j = 0; j < X8_BATCH; ++j) {
            if (q0 + 32 * j < blocks * 4) {
                const uint32_t w0 = ((uint32_t)c[j][0] | ((uint32_t)c[j][1] << 16)) ^ 0x80808080u;  // code + 128
                const uint32_t w1 = ((uint32_t)c[j][2] | ((uint32_t)c[j][3] << 16)) ^ 0x80808080u;
                float a = 0.0f;
                a = fmaf(byte_f32(w0, 0, 8388736.0f), xa[j].x, a); a = fmaf(byte_f32(w0, 1, 8388736.0f), xa[j].y, a);
                a = fmaf(byte_f32(w0, 2, 8388736.0f), xa[j].z, a); a = fmaf(byte_f32(w0, 3, 8388736.0f), xa[j].w, a);
                a = fmaf(byte_f32(w1, 0, 8388736.0f), xb[j].x, a); a = fmaf(byte_f32(w1, 1, 8388736.0f), xb[j].y, a);
                a = fmaf(byte_f32(w1, 2, 8388736.0f), xb[j].z, a); a = fmaf(byte_f32(w1, 3, 8388736.0f), xb[j].w, a);
                acc = fmaf(__half2float(__ushort_as_half(dh[j])), a, acc);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[(size_t)slot * out_stride + r] = acc;
}

// NUCLIS_EXPERTS_GENERIC=1 keeps every expert GEMV on the generic kernel (for measurements and tests).
bool experts_generic_only() {
    static const bool on = [] { const char *e = getenv("NUCLIS_EXPERTS_GENERIC"); return e && e[0] == '1'; }();
    return on;
}

}  // namespace

// Returns the number of kernels launched: 0 when the shape is not one of the specialized forms.
int launch_matvec_experts_fast(cudaStream_t s, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                               uint32_t columns, const uint32_t *indices, uint32_t slots, const float *in, size_t in_stride, uint32_t in_group,
                               float *out, size_t out_stride) {
    if (experts_generic_only() || slots > 65535) return 0;
    if ((uintptr_t)in % 16 != 0 || in_stride % 4 != 0) return 0;
    // The blocks may be placed while the operator before drains (the kernels wait for it before they read anything).
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    if (enc == Q4_K) {
        if (columns % 256 != 0 || columns > 10240) return 0;  // the staged row and its sums: 4.5 bytes a column of shared memory
        if ((uintptr_t)w % 16 != 0 || stride % 16 != 0 || expert_bytes % 16 != 0) return 0;
        const uint32_t ksb = columns / 256;
        const size_t smem = (size_t)ksb * (272 + 16) * 4;
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(expert_gemv_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 10240 / 256 * (272 + 16) * 4) != cudaSuccess) return 0;
            configured = true;
        }
        dim3 grid((rows + XQ_ROWS - 1) / XQ_ROWS, slots);
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(XQ_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, expert_gemv_q4k_kernel, w, stride, expert_bytes, experts, rows, ksb, indices, in, in_stride, in_group, out, out_stride);
        return 1;
    }
    if (enc == Q8_0) {
        if (columns % 32 != 0) return 0;
        if ((uintptr_t)w % 2 != 0 || stride % 2 != 0 || expert_bytes % 2 != 0) return 0;
        dim3 grid((rows + X8_WARPS - 1) / X8_WARPS, slots);
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(X8_WARPS * 32);
        cfg.stream = s;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, expert_gemv_q8_0_kernel, w, stride, expert_bytes, experts, rows, columns / 32, indices, in, in_stride, in_group, out, out_stride);
        return 1;
    }
    return 0;
}

}  // namespace nu
