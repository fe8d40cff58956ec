// Q6_K decode GEMV (one activation row) for sm_100a, on the shared decode
// skeleton (decode_kernel.cuh; the scheme is described in gemv_q4k_decode.cu).
// The reference's kernel for this is nu_matvec_q6_k
// (inference/src/backends/metal/kernels/matvec.metal:227-264).
//
// Q6_K blocks are 210 bytes, so rows of a GGUF tensor start on 2-byte
// boundaries and nothing wider than a 16-bit load can read them in place.
// This kernel therefore reads the planar form that launch_prepare writes once
// at load time (prepare.cu): per (row, superblock) a 208-byte record in which
// the 48 bytes each quad lane needs are contiguous, plus a transposed plane of
// the f16 super-scales. Same bytes, same values, 16-byte aligned, fetched by
// one TMA box copy per 16 rows.
//
// Lane t of a quad owns half hh = t >> 1 of the superblock and column half
// ch = t & 1 of each of its four 32-column quarters: four scale groups of 16
// values. Codes are assembled as bytes low4 | high2 << 4 (0..63), spread to
// fp16 lanes (the fp16 subnormal code * 2^-24) and multiplied on the tensor
// core against the hi/lo pieces of x; the bias of 32 is folded into the sum
// of x over the group (kernels/matvec.metal:252): d * sc * (sum(code * x) - 32 * sum(x)).
#include "decode_kernel.cuh"

namespace nu {
namespace dec {

__device__ __forceinline__ uint32_t word4(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

struct Q6K {
    static constexpr int ROW_BYTES = 208;                   // one planar record
    static constexpr int MAIN_BYTES = 16 * ROW_BYTES;       // 3328
    static constexpr int TASK_BYTES = MAIN_BYTES + 128;     // + the 16 super-scales (32 bytes), padded to a multiple of 128
    static constexpr int GSUMS = 16;                        // activation sums per superblock: one per 16-column group

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, MAIN_BYTES + 32);
        tma_load_2d(dst, &p.map[seg], sb * ROW_BYTES, row0, bar, policy);
        tma_load_2d(dst + MAIN_BYTES, &p.map2[seg], row0 * 2, sb, bar, policy);
    }
    // Float4 ci of a superblock (columns 4ci..4ci+3): half hh, quarter qr, column half ch, word m.
    // Lane t = 2 hh + ch keeps its 64 values as (qr, m) -> 8 bytes each, 128 bytes in all.
    __device__ static __forceinline__ uint32_t x_offset(uint32_t i) {
        const uint32_t sb = i >> 6, ci = i & 63u;
        const uint32_t hh = ci >> 5, qr = (ci >> 3) & 3u, ch = (ci >> 2) & 1u, m = ci & 3u;
        return (sb * 4 + hh * 2 + ch) * PAIR_PITCH + (qr * 4 + m) * 8;
    }
    // 16-column group sum: four consecutive threads hold a group; stored so that lane t reads its four as one float4.
    __device__ static __forceinline__ void group_sum(float *gsum, uint32_t i, float s, uint32_t lane) {
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if ((lane & 3) == 0) {
            const uint32_t sb = i >> 6, ci = i & 63u;
            const uint32_t hh = ci >> 5, qr = (ci >> 3) & 3u, ch = (ci >> 2) & 1u;
            gsum[sb * 16 + (hh * 2 + ch) * 4 + qr] = s;
        }
    }
    __device__ static __forceinline__ void task(const uint8_t *task, const uint8_t *xb, const float *gsum, uint32_t g, uint32_t t, float acc[2]) {
        uint4 la[2], lb[2], hb[2], sc[2];
        float d[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint8_t *row = task + (g + 8 * h) * ROW_BYTES;
            la[h] = *(const uint4 *)(row + t * 48);       // low nibbles: quarter 0, high nibbles: quarter 2
            lb[h] = *(const uint4 *)(row + t * 48 + 16);  // quarters 1 and 3
            hb[h] = *(const uint4 *)(row + t * 48 + 32);  // two high bits of all four quarters
            sc[h] = *(const uint4 *)(row + 192);
            d[h] = __half2float(*(const __half *)(task + MAIN_BYTES + (g + 8 * h) * 2));
        }
        const float4 gs = *(const float4 *)(gsum + t * 4);
        const float gsv[4] = {gs.x, gs.y, gs.z, gs.w};
        const uint32_t hh = t >> 1, ch = t & 1u;
#pragma unroll
        for (int qr = 0; qr < 4; ++qr) {
            float c[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                uint32_t a[4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t w = word4((qr & 1) ? lb[h] : la[h], m), hw = word4(hb[h], m);
                    const uint32_t nib = (qr >> 1) ? (w >> 4) : w;
                    const uint32_t top = (qr == 0 ? (hw << 4) : qr == 1 ? (hw << 2) : qr == 2 ? hw : (hw >> 2)) & 0x30303030u;
                    const uint32_t v = (nib & 0x0f0f0f0fu) | top;   // four codes 0..63, one per byte
                    a[h] = __byte_perm(v, 0u, 0x4240);              // columns +0, +2 as fp16 subnormals
                    a[2 + h] = __byte_perm(v, 0u, 0x4341);          // columns +1, +3
                }
                const uint2 b = *(const uint2 *)(xb + (qr * 4 + m) * 8);
                if (m == 0) mma16816_first(c, a, b.x, b.y);
                else mma16816(c, a, b.x, b.y);
            }
            // scale of group hh*8 + qr*2 + ch: byte 2*(qr&1) + ch of word hh*2 + (qr>>1) of the 16 scale bytes
            const float bias = -32.0f * gsv[qr];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t sw = (hh ? ((qr >> 1) ? sc[h].w : sc[h].z) : ((qr >> 1) ? sc[h].y : sc[h].x)) ^ 0x80808080u;
                const float fm = __uint_as_float(__byte_perm(sw, 0x4b000000u, 0x7650u + 2 * (qr & 1) + ch));  // 2^23 + sc + 128
                const float ds = (fm - 8388736.0f) * d[h];  // d * sc: the subtraction is exact, one rounding as in the decoder
                const float inner = fmaf(c[2 * h] + c[2 * h + 1], 16777216.0f, bias);
                acc[h] = fmaf(ds, inner, acc[h]);
            }
        }
    }
};

static bool fill(const FastJob &job, Params &p, bool maps) {
    if (job.enc != Q6_K || job.layout != 1) return false;
    if (!fill_common<Q6K>(job, p)) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.rows % 16 != 0) return false;
        const uint8_t *dplane = g.w + (size_t)g.rows * p.ksb * 208;
        if (maps && !encode_weight_map(&p.map[s], g.w, (uint64_t)p.ksb * 208, g.rows, (uint64_t)p.ksb * 208, 208, 16)) return false;
        if (maps && !encode_weight_map(&p.map2[s], dplane, (uint64_t)g.rows * 2, p.ksb, (uint64_t)g.rows * 2, 32, 1)) return false;
    }
    return true;
}

}  // namespace dec

bool q6k_decode_configure() { return dec::configure<dec::Q6K>(); }

bool q6k_decode_supported(const FastJob &job) {
    dec::Params p;
    return dec::fill(job, p, false);
}

int launch_q6k_decode(cudaStream_t s, const FastJob &job) {
    dec::Params p;
    if (!dec::fill(job, p, true)) return 0;
    return dec::launch<dec::Q6K>(s, job, p);
}

}  // namespace nu
