// Q4_K decode GEMV (one activation row) for sm_100a: the kernel behind
// Backend.matvec and single-row matvecSegments on Q4_K weights
// (inference/src/backends/metal/ops/matvec.zig:85-116, 268-343; the reference's
// kernel for this is nu_matvec_q4_k, kernels/matvec.metal:161-209).
//
// The HBM stream is the only large traffic: every weight byte is read once.
// A task is 16 weight rows by one superblock (2304 bytes); one TMA tensor copy
// (cp.async.bulk.tensor.2d + mbarrier) brings it to shared memory, each warp
// keeps its own ring of stages filled a few tasks ahead, and the 16 or 20 warps
// of an SM keep about 100 KB of copies in flight. The lanes then read their 16-byte
// pieces with 128-bit shared loads (a quad of lanes reads the 128 contiguous
// quant bytes of a superblock row).
//
// Arithmetic. The 4-bit codes are exact in fp16: a code masked in place in its
// 16-bit lane is the fp16 subnormal code * 2^-24 (or * 2^-20 for a high
// nibble), so it becomes an mma.sync.m16n8k16 A operand with no conversion.
// The activation row is scaled by a power of two and split into fp16 pieces
// hi + lo (22 significant bits); products of fp16 values are exact and are
// accumulated in F32 by the tensor core.
// With one token the 8 columns of the B operand are free, so B is made block
// diagonal: lane t of a quad owns group pair t of the superblock (groups 2t and
// 2t+1, its own 32 quant bytes), supplies that pair's codes as its four k
// indices, and columns 2t (hi) and 2t+1 (lo) of B hold x for those k only.
// Each lane thus receives the sums of its own group, needs only its own
// group's 6-bit scale and minimum, and applies d*scale once per group per
// superblock: sum_g d*s_g*sum(q*x) - dmin*sum_g m_g*sum(x), the factored form
// of kernels/matvec.metal:197.
//
// Work split. K is cut into `nks` slices; a unit is a 16-row tile by one slice,
// a task one superblock of a unit. Units are dealt to persistent blocks (one per
// SM) in contiguous, slice-major ranges of equal task count. A block's warps
// are 4 unit slots x P K parts (20 warps, P = 5; gate/up pairs 16 warps, P = 4):
// in each step four units are in work, warp (slot, part) takes superblocks
// part, part+P, ... of its unit, keeps the sums in registers and leaves 16 row
// sums in a shared-memory slot. The warps of a slot meet at a named barrier of
// their own and the parts of the unit are added in part order. With
// several slices those sums go to a global scratch array and the last block to
// arrive for a row tile adds them in slice order. No sum depends on timing.
#include "decode_kernel.cuh"

#include "../../include/nuclis_cuda.h"

namespace nu {
namespace dec {

__device__ __forceinline__ uint32_t word(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// d*s (with the 2^24 / 2^20 of the subnormal codes) and dmin*m of this lane's two groups, for one row.
struct RowScales {
    float ds_e, ds_o, dm_e, dm_o;
};
__device__ __forceinline__ RowScales row_scales(const uint4 &hdr, uint32_t t) {
    const uint32_t shift = (t & 1u) * 16;
    const uint32_t y = (hdr.y >> shift) & 0xffffu, z = (hdr.z >> shift) & 0xffffu, w = (hdr.w >> shift) & 0xffffu;
    // groups 0..3: low six bits of bytes 0..3 / 4..7; groups 4..7: nibbles of bytes 8..11 plus the top two bits of bytes 0..7
    const uint32_t s_lo = y & 0x3f3fu, m_lo = z & 0x3f3fu;
    const uint32_t s_hi = (w & 0x0f0fu) | ((y >> 2) & 0x3030u), m_hi = ((w >> 4) & 0x0f0fu) | ((z >> 2) & 0x3030u);
    const uint32_t s2 = t < 2 ? s_lo : s_hi, m2 = t < 2 ? m_lo : m_hi;
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    // byte -> float through the 2^23 magic number: one permute and one FMA each
    const float se = __uint_as_float(__byte_perm(s2, 0x4b000000u, 0x7650)), so = __uint_as_float(__byte_perm(s2, 0x4b000000u, 0x7651));
    const float me = __uint_as_float(__byte_perm(m2, 0x4b000000u, 0x7650)), mo = __uint_as_float(__byte_perm(m2, 0x4b000000u, 0x7651));
    const float de = d * 16777216.0f, d_odd = d * 1048576.0f;
    RowScales r;
    r.ds_e = fmaf(se, de, -8388608.0f * de);
    r.ds_o = fmaf(so, d_odd, -8388608.0f * d_odd);
    r.dm_e = fmaf(me, dmin, -8388608.0f * dmin);
    r.dm_o = fmaf(mo, dmin, -8388608.0f * dmin);
    return r;
}


struct Q4K {
    static constexpr int ROW_BYTES = 144;             // one superblock of one row
    static constexpr int TASK_BYTES = 16 * ROW_BYTES; // 2304, a multiple of 128
    static constexpr int GSUMS = 8;                   // activation sums kept per superblock: one per 32-column group

    __device__ static __forceinline__ void issue(const Params &p, uint32_t seg, uint32_t sb, uint32_t row0, uint32_t dst, uint32_t bar, uint64_t policy) {
        mbar_expect_tx(bar, TASK_BYTES);
        tma_load_2d(dst, &p.map[seg], sb * ROW_BYTES, row0, bar, policy);
    }
    // Float4 i of the activation row (columns 4i..4i+3): 16 of them per group pair, pairs PAIR_PITCH apart.
    __device__ static __forceinline__ uint32_t x_offset(uint32_t i) { return (i >> 4) * PAIR_PITCH + (i & 15u) * 8; }
    // 32-column group sum: eight consecutive threads hold a group.
    __device__ static __forceinline__ void group_sum(float *gsum, uint32_t i, float s, uint32_t lane) {
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if ((lane & 7) == 0) gsum[i >> 3] = s;
    }
    // One task: rows g and g+8 of the tile, this lane's group pair t (groups 2t, 2t+1).
    __device__ static __forceinline__ void task(const uint8_t *task, const uint8_t *xb, const float *gsum, uint32_t g, uint32_t t, float acc[2]) {
        uint4 hdr[2], q0[2], q1[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint8_t *row = task + (g + 8 * h) * ROW_BYTES;
            hdr[h] = *(const uint4 *)row;
            q0[h] = *(const uint4 *)(row + 16 + t * 32);
            q1[h] = *(const uint4 *)(row + 32 + t * 32);
        }
        float ce[4], co[4];  // even group / odd group: (hi, lo) sums of row g, (hi, lo) of row g+8
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t w0 = i < 4 ? word(q0[0], i) : word(q1[0], i - 4);
            const uint32_t w1 = i < 4 ? word(q0[1], i) : word(q1[1], i - 4);
            const uint32_t s0 = w0 >> 8, s1 = w1 >> 8;
            uint32_t ae[4], ao[4];
            ae[0] = w0 & 0x000f000fu; ae[1] = w1 & 0x000f000fu; ae[2] = s0 & 0x000f000fu; ae[3] = s1 & 0x000f000fu;
            ao[0] = w0 & 0x00f000f0u; ao[1] = w1 & 0x00f000f0u; ao[2] = s0 & 0x00f000f0u; ao[3] = s1 & 0x00f000f0u;
            const uint2 be = *(const uint2 *)(xb + i * 8);  // the zero block is as long as a pair's 128 bytes
            const uint2 bo = *(const uint2 *)(xb + 64 + i * 8);
            if (i == 0) {
                mma16816_first(ce, ae, be.x, be.y);
                mma16816_first(co, ao, bo.x, bo.y);
            } else {
                mma16816(ce, ae, be.x, be.y);
                mma16816(co, ao, bo.x, bo.y);
            }
        }
        const float2 gs = *(const float2 *)(gsum + t * 2);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const RowScales r = row_scales(hdr[h], t);
            float a = fmaf(r.ds_e, ce[2 * h] + ce[2 * h + 1], acc[h]);
            a = fmaf(r.ds_o, co[2 * h] + co[2 * h + 1], a);
            a = fmaf(-r.dm_e, gs.x, a);
            acc[h] = fmaf(-r.dm_o, gs.y, a);
        }
    }
};

static bool fill(const FastJob &job, Params &p, bool maps) {
    if (job.enc != Q4_K || job.layout != 0) return false;
    if (!fill_common<Q4K>(job, p)) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.stride % 16 != 0) return false;
        if (maps && !encode_weight_map(&p.map[s], g.w, (uint64_t)p.ksb * 144, g.rows, g.stride, 144, 16)) return false;
    }
    return true;
}

}  // namespace dec

bool q4k_decode_configure() { return dec::configure<dec::Q4K>(); }

bool q4k_decode_supported(const FastJob &job) {
    dec::Params p;
    return dec::fill(job, p, false);
}

int launch_q4k_decode(cudaStream_t s, const FastJob &job) {
    dec::Params p;
    if (!dec::fill(job, p, true)) return 0;
    return dec::launch<dec::Q4K>(s, job, p);
}

// ---- the entry point that allocates nothing ------------------------------------------------------
// The split-K sums and arrival counters of the decode kernel normally live in memory the handle
// allocated at creation. Here they live in an array that is part of the loaded library image.

namespace {
constexpr size_t kStaticPartialFloats = 256 * 1024;  // 1 MiB of partial sums
constexpr size_t kStaticCounters = 4096;             // output tiles of 16 rows: matrices of up to 65,536 rows
struct StaticScratch {
    float partials[kStaticPartialFloats];
    uint32_t counters[kStaticCounters + 1];  // + the status word the kernel raises when a bounded wait runs out
};
static __device__ __align__(256) StaticScratch g_static_scratch;

struct StaticDevice {
    bool ready = false;
    StaticScratch *scratch = nullptr;  // the device address of g_static_scratch on this device
    int sm_count = 0;
};
StaticDevice g_static_devices[64];
}  // namespace

}  // namespace nu

extern "C" int nu_cuda_matvec_q4k_static(const void *weights, size_t stride, uint32_t rows, uint32_t columns, const float *input, float *output,
                                         void *stream, char *err, size_t err_cap) {
    using namespace nu;
    auto fail = [&](int status, const char *what) {
        if (err && err_cap) snprintf(err, err_cap, "%s", what);
        return status;
    };
    if (!weights || !input || !output || rows == 0 || columns == 0) return fail(NU_ERR_INVALID_SHAPE, "matvec_q4k_static: null pointer or empty shape");
    if (columns % 256 != 0 || stride != (size_t)columns / 256 * 144) return fail(NU_ERR_INVALID_SHAPE, "matvec_q4k_static: rows must be whole, contiguous Q4_K superblocks");
    if (rows > 65536u || columns > 20480u)
        return fail(NU_ERR_TOO_LARGE, "matvec_q4k_static: beyond the built-in scratch (65,536 rows, 20,480 columns, 1 MiB of partial sums)");
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return fail(NU_ERR_INIT, "matvec_q4k_static: no current CUDA device");
    StaticDevice &d = g_static_devices[device];
    if (!d.ready) {
        // Once per device, with that device current: in host code the array's name is only a stand-in,
        // the kernel needs the address the symbol has on this device.
        void *ptr = nullptr;
        cudaDeviceProp prop{};
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return fail(NU_ERR_INIT, "matvec_q4k_static: cudaGetSymbolAddress failed");
        if (cudaGetDeviceProperties(&prop, device) != cudaSuccess || prop.major != 10) return fail(NU_ERR_INIT, "matvec_q4k_static: needs an sm_100 device");
        if (!q4k_decode_configure()) return fail(NU_ERR_INIT, "matvec_q4k_static: kernel set-up failed");
        d.scratch = (StaticScratch *)ptr;
        d.sm_count = prop.multiProcessorCount;
        d.ready = true;
    }
    FastJob job{};
    job.enc = Q4_K; job.layout = 0; job.columns = columns; job.tokens = 1; job.in = input; job.in_stride = columns;
    job.count = 1; job.mode = ACT_NONE;
    job.seg[0] = {(const uint8_t *)weights, stride, rows, output, rows};
    job.partials = d.scratch->partials; job.partials_floats = kStaticPartialFloats;
    job.counters = d.scratch->counters; job.counters_len = kStaticCounters;
    job.sm_count = d.sm_count;
    job.serial = true;  // the caller's stream may hold a kernel that writes these weights: no early start of the weight stream
    dec::Params p;
    if (!dec::fill(job, p, true))
        return fail(NU_ERR_TOO_LARGE, "matvec_q4k_static: beyond the built-in scratch (65,536 rows, 20,480 columns, 1 MiB of partial sums) or pointers not 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    // The array keeps whatever the last call left: the counters and the status word must start at zero.
    if (cudaMemsetAsync(d.scratch->counters, 0, sizeof d.scratch->counters, s) != cudaSuccess) return fail(NU_ERR_EXECUTION, "matvec_q4k_static: clearing the counters failed");
    dec::launch<dec::Q4K>(s, job, p);
    if (cudaGetLastError() != cudaSuccess) return fail(NU_ERR_EXECUTION, "matvec_q4k_static: launch failed");
    return NU_OK;
}
