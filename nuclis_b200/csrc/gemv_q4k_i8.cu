// Q4_K GEMV and small-batch GEMM (1..8 activation rows) for sm_100a on the integer tensor path: the
// kernel behind Backend.matvec, matvecRows, small matmul and matvecSegments on Q4_K weights
// (inference/src/backends/metal/ops/matvec.zig:85-188, 268-343; the reference's kernels for this are
// nu_matvec_q4_k, kernels/matvec.metal:161-209, and nu_matvec_rows_q4_k, kernels/matvec_rows.metal:34-128).
//
// The HBM stream is the only large traffic: every weight byte is read once, whatever the number of
// activation rows. A task is 16 weight rows by one superblock (2304 bytes). The five warps of a unit slot
// share a ring of stages; one TMA tensor copy (cp.async.bulk.tensor.2d + mbarrier) brings 16 rows by five
// superblocks (11,520 bytes, 720 contiguous bytes per row) into a stage, one task for each of the five.
//
// Arithmetic (i8_kernel.cuh has the scheme). A Q4_K superblock row holds 128 quant bytes: byte j of
// the 32-byte chunk c carries element j of group 2c in its low nibble and of group 2c + 1 in its high
// nibble. A word masked with 0x0f0f0f0f is four codes of the even group as bytes; masked with
// 0xf0f0f0f0 it is four codes of the odd group times 16, still bytes (at most 240), so no shift is
// spent: the odd groups get an accumulator of their own and the factor 16 is undone once per
// superblock. One m16n8k32 mma covers one 32-column scale group of 16 rows: lane t of a quad supplies
// the group's columns 8t..8t+7 (eight consecutive quant bytes, one 64-bit shared load per row), and
// the 6-bit group scale multiplies the int32 sums afterwards. Per superblock and row:
//   out += d * inv * sum_g s_g * sum_k(q * X)  -  dmin * inv * sum_g m_g * sum_k(X),
// the factored form of kernels/matvec.metal:197 with X the fixed-point activations and inv the power
// of two that scaled them. The minima go through the tensor core too: an m16n8k8 f16 step whose A
// holds a row's eight 6-bit minima and whose B holds the eight group sums of X (as fp16 pieces hi + lo).
#include "i8_q4k.cuh"

#include "../../include/nuclis_cuda.h"

namespace nu {
namespace i8 {

using Plain = Q4KPlain;
using Dense = Q4KDense;
using Quad = Q4KDense;  // three or four tokens: the 15-warp geometry (two mmas a group want the wide form's registers), no K cut forced by the digit rows

static bool fill(const FastJob &job, Params &p, Plan &plan, bool maps) {
    if (job.enc != Q4_K || job.layout != 0) return false;
    const bool ok = job.tokens == 1 ? fill_geometry<Q4K, Plain, 1>(job, p, plan) : job.tokens == 2 ? fill_geometry<Q4K, Plain, 2>(job, p, plan) : job.tokens <= 4 ? fill_geometry<Q4K, Quad, 4>(job, p, plan) : fill_geometry<Q4K, Dense, 8>(job, p, plan);
    if (!ok) return false;
    for (uint32_t s = 0; s < job.count; ++s) {
        const FastSegment &g = job.seg[s];
        if (g.stride % 16 != 0) return false;
        if (maps && !encode_tiled_map(&p.map[s], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, g.w, (uint64_t)p.ksb * 36, g.rows, g.stride, Q4K::ROW_PITCH / 4, 16, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
    }
    return true;
}

static int launch(cudaStream_t s, const FastJob &job, const Params &p, const Plan &plan) {
    return plan.nt == 1 ? launch_geometry<Q4K, Plain, 1>(s, job, p, plan) : plan.nt == 2 ? launch_geometry<Q4K, Plain, 2>(s, job, p, plan) : plan.nt == 4 ? launch_geometry<Q4K, Quad, 4>(s, job, p, plan) : launch_geometry<Q4K, Dense, 8>(s, job, p, plan);
}

}  // namespace i8

bool q4k_i8_fill(const FastJob &job, i8::Params &p, i8::Plan &plan, bool maps) { return i8::fill(job, p, plan, maps); }

bool q4k_i8_configure() {
    return i8::configure_geometry<i8::Q4K, i8::Plain, 1>() && i8::configure_geometry<i8::Q4K, i8::Plain, 2>() && i8::configure_geometry<i8::Q4K, i8::Quad, 4>() &&
           i8::configure_geometry<i8::Q4K, i8::Dense, 8>();
}

bool q4k_i8_supported(const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    return i8::fill(job, p, plan, false);
}

int launch_q4k_i8(cudaStream_t s, const FastJob &job) {
    i8::Params p;
    i8::Plan plan;
    if (!i8::fill(job, p, plan, true)) return 0;
    return i8::launch(s, job, p, plan);
}

bool q4k_i8_plan(const FastJob &job, uint32_t *slices, uint32_t *blocks) {
    i8::Params p;
    i8::Plan plan;
    if (!i8::fill(job, p, plan, false)) return false;
    if (slices) *slices = p.nks;
    if (blocks) *blocks = plan.grid;
    return true;
}

// ---- the entry point that allocates nothing ------------------------------------------------------
// The split-K sums and arrival counters of the kernel normally live in memory the handle
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

FastJob static_job(const void *weights, size_t stride, uint32_t rows, uint32_t columns, const float *input, float *output, float *partials, uint32_t *counters,
                   int sm_count) {
    FastJob job{};
    job.enc = Q4_K; job.layout = 0; job.columns = columns; job.tokens = 1; job.in = input; job.in_stride = columns;
    job.count = 1; job.mode = ACT_NONE;
    job.seg[0] = {(const uint8_t *)weights, stride, rows, output, rows};
    job.partials = partials; job.partials_floats = kStaticPartialFloats;
    job.counters = counters; job.counters_len = kStaticCounters;
    job.sm_count = sm_count;
    job.serial = true;  // the caller's stream may hold a kernel that writes these weights: no early start of the weight stream
    return job;
}
}  // namespace

}  // namespace nu

extern "C" int nu_cuda_matvec_q4k_static_plan(uint32_t rows, uint32_t columns, uint32_t sm_count, uint32_t *slices, uint32_t *blocks) {
    using namespace nu;
    if (rows == 0 || columns == 0 || columns % 256 != 0 || sm_count == 0) return NU_ERR_INVALID_SHAPE;
    if (rows > 65536u || columns > 20480u) return NU_ERR_TOO_LARGE;
    // no device is touched: the pointers only have to look aligned
    const FastJob job = static_job((const void *)256, (size_t)columns / 256 * 144, rows, columns, (const float *)256, (float *)256, (float *)256, (uint32_t *)256, (int)sm_count);
    return q4k_i8_plan(job, slices, blocks) ? NU_OK : NU_ERR_TOO_LARGE;
}

extern "C" int nu_cuda_matvec_q4k_static(const void *weights, size_t stride, uint32_t rows, uint32_t columns, const float *input, float *output,
                                         void *stream, char *err, size_t err_cap) {
    using namespace nu;
    auto fail = [&](int status, const char *what) {
        if (err && err_cap) snprintf(err, err_cap, "%s", what);
        return status;
    };
    if (!weights || !input || !output || rows == 0 || columns == 0) return fail(NU_ERR_INVALID_SHAPE, "matvec_q4k_static: null pointer or empty shape");
    if (columns % 256 != 0 || stride != (size_t)columns / 256 * 144) return fail(NU_ERR_INVALID_SHAPE, "matvec_q4k_static: rows must be whole, contiguous Q4_K superblocks");
    if ((uintptr_t)weights % 16 != 0 || (uintptr_t)input % 16 != 0 || (uintptr_t)output % 4 != 0)
        return fail(NU_ERR_INVALID_SHAPE, "matvec_q4k_static: weights and input must be 16-byte aligned, output 4-byte aligned");
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
        if (!q4k_i8_configure()) return fail(NU_ERR_INIT, "matvec_q4k_static: kernel set-up failed");
        d.scratch = (StaticScratch *)ptr;
        d.sm_count = prop.multiProcessorCount;
        d.ready = true;
    }
    const FastJob job = static_job(weights, stride, rows, columns, input, output, d.scratch->partials, d.scratch->counters, d.sm_count);
    i8::Params p;
    i8::Plan plan;
    if (!i8::fill(job, p, plan, true)) return fail(NU_ERR_TOO_LARGE, "matvec_q4k_static: no way to cut this shape fits the built-in scratch");
    cudaStream_t s = (cudaStream_t)stream;
    // The array keeps whatever the last call left: the counters and the status word must start at zero.
    if (cudaMemsetAsync(d.scratch->counters, 0, sizeof d.scratch->counters, s) != cudaSuccess) return fail(NU_ERR_EXECUTION, "matvec_q4k_static: clearing the counters failed");
    i8::launch(s, job, p, plan);
    if (cudaGetLastError() != cudaSuccess) return fail(NU_ERR_EXECUTION, "matvec_q4k_static: launch failed");
    return NU_OK;
}

extern "C" int nu_cuda_matvec_q4k_static_status(void *stream, uint32_t *status) {
    using namespace nu;
    int device = -1;
    if (!status || cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return NU_ERR_INVALID_SHAPE;
    StaticDevice &d = g_static_devices[device];
    if (!d.ready) { *status = 0; return NU_OK; }
    cudaStream_t s = (cudaStream_t)stream;
    if (cudaMemcpyAsync(status, d.scratch->counters + kStaticCounters, sizeof *status, cudaMemcpyDeviceToHost, s) != cudaSuccess) return NU_ERR_EXECUTION;
    return cudaStreamSynchronize(s) == cudaSuccess ? NU_OK : NU_ERR_EXECUTION;
}
