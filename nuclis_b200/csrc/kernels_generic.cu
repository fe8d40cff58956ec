// Plain kernels: the decode-and-FMA matvec/matmul that serves any encoding at
// any alignment (the role of nu_matvec / nu_matvec_rows / nu_matvec_experts,
// inference/src/backends/metal/kernels/matvec.metal:5-21, matvec_rows.metal:274-298,
// experts.metal:16-36), the standalone row decoder (nu_embed, rowwise.metal:3-11)
// and the element-wise, routing and combine kernels of the expert path
// (experts.metal:46-120, 153-161). These are the slow, obviously-right forms the
// specialized kernels are checked against on the device.
#include <cuda_bf16.h>

#include <utility>

#include "kernels.hpp"
#include "nu_device.cuh"

namespace nu {

// The small kernels of the expert chain are launched so that their blocks may be placed while the operator
// before them drains; each starts with griddepcontrol.wait, after which the earlier operator's writes are
// visible, so nothing else changes. Saves part of the launch latency between short dependent kernels.
template <typename... KArgs, typename... Args>
static void launch_after_previous(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args &&...args) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
__device__ __forceinline__ void wait_for_previous_operator() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
}

// ---- row decode ------------------------------------------------------------

// Decodes 16 values of row r: from the GGUF rows, or from the planar form of prepare.cu.
__device__ __forceinline__ void decode16(uint32_t enc, uint32_t layout, const uint8_t *w, size_t stride, uint32_t rows, uint32_t columns, uint32_t r,
                                         uint32_t seg, float v[16]) {
    if (layout == 1) dequant16_planar_q6k(w, rows, columns / 256, r, seg, v);
    else if (layout == 2) dequant16_planar_q8_0(w, rows, columns, r, seg, v);
    else if (layout >= 3 && layout <= 5) dequant16_planar_block32(enc, w, rows, columns / 256, r, seg, v);
    else if (layout == 6) dequant16_planar_iq4_xs(w, rows, columns / 256, r, seg, v);
    else if (layout == 7) dequant16_planar_q2k(w, rows, columns / 256, r, seg, v);
    else if (layout == 8) dequant16_planar_q3k(w, rows, columns / 256, r, seg, v);
    else dequant16(enc, w + (size_t)r * stride, seg, v);
}

__global__ void dequant_row_kernel(uint32_t enc, uint32_t layout, const uint8_t *w, size_t stride, uint32_t rows, uint32_t row, uint32_t columns,
                                   float *out_f32, __nv_bfloat16 *out_bf16) {
    const uint32_t seg = blockIdx.x * blockDim.x + threadIdx.x;
    if (seg >= columns / 16) return;
    float v[16];
    decode16(enc, layout, w, stride, rows, columns, row, seg, v);
    if (out_f32) {
#pragma unroll
        for (int i = 0; i < 16; ++i) out_f32[seg * 16 + i] = v[i];
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) out_bf16[seg * 16 + i] = __float2bfloat16_rn(v[i]);
    }
}

int launch_dequant_row(cudaStream_t s, uint32_t enc, uint32_t layout, const uint8_t *w, size_t stride, uint32_t rows, uint32_t row, uint32_t columns,
                       void *out, bool out_bf16) {
    const uint32_t segments = columns / 16;
    dequant_row_kernel<<<(segments + 255) / 256, 256, 0, s>>>(enc, layout, w, stride, rows, row, columns, out_bf16 ? nullptr : (float *)out,
                                                             out_bf16 ? (__nv_bfloat16 *)out : nullptr);
    return 1;
}

// ---- generic matvec / matmul ------------------------------------------------

constexpr int GENERIC_TOKENS = 8;   // token rows one warp accumulates at once
constexpr int GENERIC_WARPS = 8;    // warps (= weight rows) per block

template <bool IN_BF16>
__device__ __forceinline__ float load_in(const void *in, size_t index) {
    if (IN_BF16) return __bfloat162float(((const __nv_bfloat16 *)in)[index]);
    return ((const float *)in)[index];
}

// One warp per weight row; lanes stride over 16-value segments; each decoded
// value is multiplied into up to 8 token accumulators; tokens beyond 8 are
// covered by blockIdx.y.
template <bool IN_BF16>
__device__ __forceinline__ void generic_row(uint32_t enc, uint32_t layout, const uint8_t *w, size_t stride, uint32_t rows, uint32_t columns,
                                            const void *in, size_t in_stride, uint32_t tokens, float *out, size_t out_stride, uint32_t r) {
    const uint32_t lane = threadIdx.x & 31;
    float acc[GENERIC_TOKENS];
#pragma unroll
    for (int t = 0; t < GENERIC_TOKENS; ++t) acc[t] = 0.0f;
    for (uint32_t seg = lane; seg < columns / 16; seg += 32) {
        float v[16];
        decode16(enc, layout, w, stride, rows, columns, r, seg, v);
#pragma unroll
        for (int t = 0; t < GENERIC_TOKENS; ++t) {
            if ((uint32_t)t < tokens) {
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[t] = fmaf(v[i], load_in<IN_BF16>(in, (size_t)t * in_stride + seg * 16 + i), acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < GENERIC_TOKENS; ++t) {
        float a = acc[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0 && (uint32_t)t < tokens) out[(size_t)t * out_stride + r] = a;
    }
}

template <bool IN_BF16>
__global__ void matmul_generic_kernel(uint32_t enc, uint32_t layout, const uint8_t *w, size_t stride, uint32_t rows, uint32_t columns,
                                      const void *in, size_t in_stride, float *out, size_t out_stride, uint32_t tokens) {
    const uint32_t r = blockIdx.x * GENERIC_WARPS + (threadIdx.x >> 5);
    if (r >= rows) return;
    const uint32_t t0 = blockIdx.y * GENERIC_TOKENS;
    const uint32_t n = min(tokens - t0, (uint32_t)GENERIC_TOKENS);
    const void *x = IN_BF16 ? (const void *)((const __nv_bfloat16 *)in + (size_t)t0 * in_stride)
                            : (const void *)((const float *)in + (size_t)t0 * in_stride);
    generic_row<IN_BF16>(enc, layout, w, stride, rows, columns, x, in_stride, n, out + (size_t)t0 * out_stride, out_stride, r);
}

int launch_matmul_generic(cudaStream_t s, uint32_t enc, uint32_t layout, const uint8_t *w, size_t stride, uint32_t rows, uint32_t columns,
                          const void *in, bool in_bf16, size_t in_stride, float *out, size_t out_stride, uint32_t tokens) {
    dim3 grid((rows + GENERIC_WARPS - 1) / GENERIC_WARPS, (tokens + GENERIC_TOKENS - 1) / GENERIC_TOKENS);
    if (in_bf16)
        matmul_generic_kernel<true><<<grid, GENERIC_WARPS * 32, 0, s>>>(enc, layout, w, stride, rows, columns, in, in_stride, out, out_stride, tokens);
    else
        matmul_generic_kernel<false><<<grid, GENERIC_WARPS * 32, 0, s>>>(enc, layout, w, stride, rows, columns, in, in_stride, out, out_stride, tokens);
    return 1;
}

__global__ void matvec_experts_generic_kernel(uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts,
                                              uint32_t rows, uint32_t columns, const uint32_t *indices,
                                              const float *in, size_t in_stride, uint32_t in_group, float *out, size_t out_stride) {
    const uint32_t slot = blockIdx.y;
    const uint32_t r = blockIdx.x * GENERIC_WARPS + (threadIdx.x >> 5);
    if (r >= rows) return;
    // A corrupt routing buffer can never read past the tensor (experts.metal:25).
    const uint32_t expert = min(indices[slot], experts - 1);
    generic_row<false>(enc, 0, w + (size_t)expert * expert_bytes, stride, rows, columns, in + (size_t)(slot / in_group) * in_stride, 0, 1,
                       out + (size_t)slot * out_stride, 0, r);
}

int launch_matvec_experts_generic(cudaStream_t s, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes,
                                  uint32_t experts, uint32_t rows, uint32_t columns, const uint32_t *indices, uint32_t slots,
                                  const float *in, size_t in_stride, uint32_t in_group, float *out, size_t out_stride) {
    dim3 grid((rows + GENERIC_WARPS - 1) / GENERIC_WARPS, slots);
    matvec_experts_generic_kernel<<<grid, GENERIC_WARPS * 32, 0, s>>>(enc, w, stride, expert_bytes, experts, rows, columns, indices,
                                                                      in, in_stride, in_group, out, out_stride);
    return 1;
}

// ---- prefill expert path: slot rows grouped by expert, then gathered tiles ------------------
// (inference/src/backends/metal/ops/experts.zig:119-202). The lists buffer holds, in 32-bit words:
// [0] tile count, [1] n, [2 .. 2 + experts] exclusive prefix offsets, then `bound` tiles of
// (expert, first, count), then the n slot rows grouped by expert, in slot order within an expert.

constexpr int EXPERT_TILE = 32;

// One block of 32 warps; warp w owns the w-th contiguous part of the slot rows. Pass 1 counts each part's rows per expert
// (shared-memory atomics); a prefix over the parts, expert by expert, turns the counts into the place where each part's
// rows of an expert start; pass 2 walks the parts again, 32 rows at a time: the lanes that hold the same expert find one
// another with a match, take consecutive places in lane order (= slot order) and their first lane moves the expert's
// place on. The order within an expert is the slot order, and the work is one pass over the rows, not rows x experts.
constexpr int LISTS_WARPS = 32;

__global__ void __launch_bounds__(LISTS_WARPS * 32) expert_lists_kernel(const uint32_t *indices, uint32_t n, uint32_t experts, uint32_t bound, uint32_t *lists) {
    __shared__ uint32_t place[LISTS_WARPS][256];  // pass 1: rows of expert e in part w; then: where they start in the list
    __shared__ uint32_t offsets[257];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    uint32_t *tiles = lists + experts + 3, *rows = tiles + 3 * (size_t)bound;
    for (uint32_t i = tid; i < LISTS_WARPS * 256; i += LISTS_WARPS * 32) (&place[0][0])[i] = 0;
    __syncthreads();
    const uint32_t per = ((n + LISTS_WARPS - 1) / LISTS_WARPS + 31u) & ~31u;  // whole groups of 32 rows
    const uint32_t lo = min(warp * per, n), hi = min(lo + per, n);
    for (uint32_t i = lo + lane; i < hi; i += 32) atomicAdd(&place[warp][min(__ldg(indices + i), experts - 1)], 1u);
    __syncthreads();
    // per expert: its rows in all parts; then the experts' exclusive prefix (one thread: at most 256 steps) and the tiles
    uint32_t total = 0;
    if (tid < experts)
        for (int w = 0; w < LISTS_WARPS; ++w) total += place[w][tid];
    if (tid < 256) offsets[tid] = tid < experts ? total : 0;
    __syncthreads();
    if (tid == 0) {
        uint32_t at = 0, ntiles = 0;
        for (uint32_t x = 0; x < experts; ++x) {
            const uint32_t c = offsets[x];
            offsets[x] = at;
            for (uint32_t first = 0; first < c; first += EXPERT_TILE) {
                tiles[3 * ntiles] = x;
                tiles[3 * ntiles + 1] = at + first;
                tiles[3 * ntiles + 2] = min((uint32_t)EXPERT_TILE, c - first);
                ++ntiles;
            }
            at += c;
        }
        offsets[experts] = at;
        lists[0] = ntiles;
        lists[1] = n;
    }
    __syncthreads();
    if (tid <= experts) lists[2 + tid] = offsets[tid];
    if (tid < experts) {
        uint32_t at = offsets[tid];
        for (int w = 0; w < LISTS_WARPS; ++w) {
            const uint32_t c = place[w][tid];
            place[w][tid] = at;
            at += c;
        }
    }
    __syncthreads();
    for (uint32_t i0 = lo; i0 < hi; i0 += 32) {
        const uint32_t i = i0 + lane;
        const bool live = i < hi;
        const uint32_t e = live ? min(__ldg(indices + i), experts - 1) : 0xffffffffu;
        const uint32_t same = __match_any_sync(0xffffffffu, e);
        if (live) {
            const uint32_t before = __popc(same & ((1u << lane) - 1u));
            const uint32_t at = place[warp][e];
            rows[at + before] = i;
        }
        __syncwarp();
        if (live && lane == (uint32_t)__ffs((int)same) - 1u) place[warp][e] += __popc(same);
        __syncwarp();
    }
}

int launch_expert_lists(cudaStream_t s, const uint32_t *indices, uint32_t n, uint32_t experts, uint32_t bound, uint32_t *lists) {
    expert_lists_kernel<<<1, LISTS_WARPS * 32, 0, s>>>(indices, n, experts, bound, lists);
    return 1;
}

// One block per (tile of up to 32 slot rows of one expert, group of GENERIC_WARPS weight rows); a warp
// takes one weight row and the tile's slot rows eight at a time: the expert's weights are decoded once per
// eight slot rows instead of once per slot row.
__global__ void matmul_experts_generic_kernel(uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                                              uint32_t columns, const uint32_t *lists, uint32_t bound, const float *in, size_t in_stride,
                                              uint32_t in_group, float *out, size_t out_stride) {
    const uint32_t tile = blockIdx.y;
    if (tile >= lists[0]) return;
    const uint32_t *tiles = lists + experts + 3, *slot_rows = tiles + 3 * (size_t)bound;
    const uint32_t expert = min(tiles[3 * tile], experts - 1), first = tiles[3 * tile + 1], count = tiles[3 * tile + 2];
    const uint32_t r = blockIdx.x * GENERIC_WARPS + (threadIdx.x >> 5);
    if (r >= rows) return;
    const uint32_t lane = threadIdx.x & 31;
    const uint8_t *we = w + (size_t)expert * expert_bytes;
    for (uint32_t c0 = 0; c0 < count; c0 += GENERIC_TOKENS) {
        const uint32_t nt = min(count - c0, (uint32_t)GENERIC_TOKENS);
        const float *x[GENERIC_TOKENS];
        uint32_t slot[GENERIC_TOKENS];
#pragma unroll
        for (int t = 0; t < GENERIC_TOKENS; ++t) {
            slot[t] = slot_rows[first + c0 + min((uint32_t)t, nt - 1)];
            x[t] = in + (size_t)(slot[t] / in_group) * in_stride;
        }
        float acc[GENERIC_TOKENS];
#pragma unroll
        for (int t = 0; t < GENERIC_TOKENS; ++t) acc[t] = 0.0f;
        for (uint32_t seg = lane; seg < columns / 16; seg += 32) {
            float v[16];
            decode16(enc, 0, we, stride, rows, columns, r, seg, v);
#pragma unroll
            for (int t = 0; t < GENERIC_TOKENS; ++t) {
                if ((uint32_t)t < nt) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[t] = fmaf(v[i], x[t][seg * 16 + i], acc[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < GENERIC_TOKENS; ++t) {
            float a = acc[t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            if (lane == 0 && (uint32_t)t < nt) out[(size_t)slot[t] * out_stride + r] = a;
        }
    }
}

int launch_matmul_experts_generic(cudaStream_t s, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                                  uint32_t columns, const uint32_t *lists, uint32_t bound, const float *in, size_t in_stride, uint32_t in_group,
                                  float *out, size_t out_stride) {
    dim3 grid((rows + GENERIC_WARPS - 1) / GENERIC_WARPS, bound);
    matmul_experts_generic_kernel<<<grid, GENERIC_WARPS * 32, 0, s>>>(enc, w, stride, expert_bytes, experts, rows, columns, lists, bound, in, in_stride,
                                                                      in_group, out, out_stride);
    return 1;
}

// ---- act(gate) * up ----------------------------------------------------------

__global__ void act_mul_rows_kernel(uint32_t act, const float *gate, const float *up, float *out, uint32_t width, uint32_t rows,
                                    size_t gate_stride, size_t up_stride, size_t out_stride) {
    wait_for_previous_operator();
    const size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (size_t)width * rows) return;
    const size_t r = id / width, i = id % width;
    const float g = gate[r * gate_stride + i];
    const float a = act == ACT_SILU ? silu_f32(g) : (act == ACT_GELU ? gelu_f32(g) : g);
    out[r * out_stride + i] = a * up[r * up_stride + i];
}

int launch_act_mul_rows(cudaStream_t s, uint32_t act, const float *gate, const float *up, float *out,
                        uint32_t width, uint32_t rows, size_t gate_stride, size_t up_stride, size_t out_stride) {
    const size_t n = (size_t)width * rows;
    launch_after_previous(act_mul_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), s, act, gate, up, out, width, rows, gate_stride, up_stride, out_stride);
    return 1;
}

// ---- weighted RMS norm, alone or with the residual add in front -----------------------------------
// `Backend.rmsNorm` / `addRmsNorm` / `add` (ops/rowwise.zig:37-51, 76-93, 199-202; the arithmetic of cpu rmsNorm,
// backends/cpu/vector.zig:53-64). A block per token row. The row is read once: every thread keeps its float4 pieces
// (the summed residual, when an input is added) in registers between the sum of squares and the scaled write, so rows
// of up to NORM_THREADS * 4 * NORM_KEEP floats cost one pass over memory; longer rows re-read what does not fit.
// With ADD the updated residual is stored as well. `output` may alias the residual exactly.

constexpr int NORM_THREADS = 256;
constexpr int NORM_KEEP = 8;  // float4 pieces a thread keeps: rows of up to 8192 floats in one pass

template <bool ADD>
__global__ void __launch_bounds__(NORM_THREADS) norm_rows_kernel(float *residual, const float *input, const float *weight, float *output, uint32_t width,
                                                                  size_t in_stride, size_t out_stride, float eps) {
    __shared__ float partial[NORM_THREADS / 32];
    wait_for_previous_operator();
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    float *x = residual + (size_t)row * in_stride;
    const float *s = ADD ? input + (size_t)row * in_stride : nullptr;
    float *y = output + (size_t)row * out_stride;
    const bool vec = width % 4 == 0 && in_stride % 4 == 0 && out_stride % 4 == 0 && ((uintptr_t)residual | (uintptr_t)output | (uintptr_t)weight | (ADD ? (uintptr_t)input : 0)) % 16 == 0;
    float4 kept[NORM_KEEP];
    float sum = 0.0f;
    if (vec) {
        const uint32_t pieces = width / 4;
#pragma unroll
        for (int k = 0; k < NORM_KEEP; ++k) {
            const uint32_t i = tid + k * NORM_THREADS;
            if (i < pieces) {
                float4 v = ((const float4 *)x)[i];
                if (ADD) {
                    const float4 a = ((const float4 *)s)[i];
                    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                    ((float4 *)x)[i] = v;
                }
                kept[k] = v;
                sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        for (uint32_t i = tid + NORM_KEEP * NORM_THREADS; i < pieces; i += NORM_THREADS) {
            float4 v = ((const float4 *)x)[i];
            if (ADD) {
                const float4 a = ((const float4 *)s)[i];
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                ((float4 *)x)[i] = v;
            }
            sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (uint32_t i = tid; i < width; i += NORM_THREADS) {
            float v = x[i];
            if (ADD) { v += s[i]; x[i] = v; }
            sum += v * v;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((tid & 31) == 0) partial[tid >> 5] = sum;
    __syncthreads();  // every thread has read (and, with ADD, written back) its part of the row
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < NORM_THREADS / 32; ++w) total += partial[w];
    const float scale = rsqrtf(total / (float)width + eps);
    if (vec) {
        const uint32_t pieces = width / 4;
#pragma unroll
        for (int k = 0; k < NORM_KEEP; ++k) {
            const uint32_t i = tid + k * NORM_THREADS;
            if (i < pieces) {
                const float4 v = kept[k], g = ((const float4 *)weight)[i];
                ((float4 *)y)[i] = make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
            }
        }
        for (uint32_t i = tid + NORM_KEEP * NORM_THREADS; i < pieces; i += NORM_THREADS) {
            const float4 v = ((const float4 *)x)[i], g = ((const float4 *)weight)[i];
            ((float4 *)y)[i] = make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
        }
    } else {
        for (uint32_t i = tid; i < width; i += NORM_THREADS) y[i] = x[i] * scale * weight[i];
    }
}

int launch_norm_rows(cudaStream_t s, float *residual, const float *input, const float *weight, float *output, uint32_t width, uint32_t rows, size_t in_stride,
                     size_t out_stride, float eps) {
    if (input) launch_after_previous(norm_rows_kernel<true>, dim3(rows), dim3(NORM_THREADS), s, residual, input, weight, output, width, in_stride, out_stride, eps);
    else launch_after_previous(norm_rows_kernel<false>, dim3(rows), dim3(NORM_THREADS), s, residual, input, weight, output, width, in_stride, out_stride, eps);
    return 1;
}

__global__ void add_kernel(float *x, const float *y, size_t count) {
    wait_for_previous_operator();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) x[i] += y[i];
}

int launch_add(cudaStream_t s, float *x, const float *y, size_t count) {
    launch_after_previous(add_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), s, x, y, count);
    return 1;
}

// ---- router -------------------------------------------------------------------
// `Backend.route` (ops/experts.zig:29-34; the arithmetic of cpu.experts.route, backends/cpu/experts.zig:50-79).
// One warp per token row, the logits in registers (lane l holds experts l, l + 32, ...; at most 256 experts):
// the maximum and the sum of exp by warp shuffles, then k rounds of a warp-wide arg-max by (logit descending,
// index ascending) on the logits themselves, so that the rounding of exp cannot reorder near ties. Round r's
// expert and probability stay in lane r mod 32 until the end; the selected probabilities are added in slot
// order, as a serial loop would, and the weights are renormalized over them with the sum clamped below at
// the smallest normal F16. No shared memory, no block barrier.

constexpr int ROUTE_WARPS = 4;
constexpr int ROUTE_PER_LANE = 8;  // 256 experts at most
constexpr int ROUTE_MAX_K = 64;

__global__ void __launch_bounds__(ROUTE_WARPS * 32) route_kernel(const float *logits, uint32_t experts, uint32_t k, uint32_t rows, size_t in_stride,
                                                                  uint32_t *indices, float *weights) {
    wait_for_previous_operator();
    const uint32_t lane = threadIdx.x & 31, row = blockIdx.x * ROUTE_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;  // whole warps leave together
    const float *src = logits + (size_t)row * in_stride;
    float v[ROUTE_PER_LANE], top = -INFINITY;
#pragma unroll
    for (int j = 0; j < ROUTE_PER_LANE; ++j) {
        const uint32_t e = lane + 32u * j;
        v[j] = e < experts ? src[e] : -INFINITY;
        top = fmaxf(top, v[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    float prob[ROUTE_PER_LANE], total = 0.0f;
#pragma unroll
    for (int j = 0; j < ROUTE_PER_LANE; ++j) {
        prob[j] = lane + 32u * j < experts ? expf(v[j] - top) : 0.0f;
        total += prob[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    uint32_t used = 0, kept_index[ROUTE_MAX_K / 32] = {0u, 0u};
    float kept_prob[ROUTE_MAX_K / 32] = {0.0f, 0.0f}, chosen = 0.0f;
    for (uint32_t r = 0; r < k; ++r) {
        // this lane's best unused expert: its experts ascend with j, so a strict comparison keeps the lowest index of a tie
        float best = -INFINITY, best_prob = 0.0f;
        uint32_t best_e = 0xffffffffu;
#pragma unroll
        for (int j = 0; j < ROUTE_PER_LANE; ++j) {
            const uint32_t e = lane + 32u * j;
            const bool open = e < experts && !((used >> j) & 1u);
            if (open && (best_e == 0xffffffffu || v[j] > best)) { best = v[j]; best_e = e; best_prob = prob[j]; }
        }
        // the warp's best: larger logit first, lower index on equal logits
        float win = best;
        uint32_t win_e = best_e;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, win, o);
            const uint32_t other_e = __shfl_xor_sync(0xffffffffu, win_e, o);
            if (other_e != 0xffffffffu && (win_e == 0xffffffffu || other > win || (other == win && other_e < win_e))) { win = other; win_e = other_e; }
        }
        const float p = __shfl_sync(0xffffffffu, best_prob, win_e & 31u) / total;  // the owner's lane holds it as its own best
        if ((win_e & 31u) == lane) used |= 1u << (win_e >> 5);
        chosen += p;
        if ((r & 31u) == lane) {
            if (r < 32) { kept_index[0] = win_e; kept_prob[0] = p; }
            else { kept_index[1] = win_e; kept_prob[1] = p; }
        }
    }
    const float norm = fmaxf(chosen, 6.103515625e-5f);
    if (lane < k) {
        indices[(size_t)row * k + lane] = kept_index[0];
        weights[(size_t)row * k + lane] = kept_prob[0] / norm;
    }
    if (lane + 32 < k) {
        indices[(size_t)row * k + lane + 32] = kept_index[1];
        weights[(size_t)row * k + lane + 32] = kept_prob[1] / norm;
    }
}

int launch_route(cudaStream_t s, const float *logits, uint32_t experts, uint32_t k, uint32_t rows, size_t in_stride,
                 uint32_t *indices, float *weights) {
    launch_after_previous(route_kernel, dim3((rows + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), s, logits, experts, k, rows, in_stride, indices, weights);
    return 1;
}

// ---- combine --------------------------------------------------------------------
// `Backend.combineExperts` (ops/experts.zig:79-92): out[row] = sum over the row's slots, in slot order, of
// weight * (scale of the slot's expert) * values[slot]. A thread owns VEC adjacent columns of one token row
// and walks the slots once; the slot factors are the same address for a whole warp (one broadcast load).

template <int VEC>
__global__ void __launch_bounds__(128) combine_experts_kernel(const float *values, const float *weights, const uint32_t *indices, const float *scales,
                                                              float *out, uint32_t columns, uint32_t slots, size_t in_stride, size_t out_stride,
                                                              uint32_t experts) {
    wait_for_previous_operator();
    const uint32_t row = blockIdx.y, c0 = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (c0 >= columns) return;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
    const size_t first = (size_t)row * slots;
    for (uint32_t s = 0; s < slots; ++s) {
        float factor = weights[first + s];
        if (scales) factor *= scales[min(indices[first + s], experts - 1)];
        const float *src = values + (first + s) * in_stride + c0;
        if (VEC == 4) {
            const float4 x = *(const float4 *)src;
            acc[0] = fmaf(factor, x.x, acc[0]); acc[1] = fmaf(factor, x.y, acc[1]);
            acc[2] = fmaf(factor, x.z, acc[2]); acc[3] = fmaf(factor, x.w, acc[3]);
        } else {
            acc[0] = fmaf(factor, src[0], acc[0]);
        }
    }
    float *dst = out + (size_t)row * out_stride + c0;
    if (VEC == 4) *(float4 *)dst = make_float4(acc[0], acc[1], acc[2], acc[3]);
    else dst[0] = acc[0];
}

// ---- greedy selection over the output head's logits ---------------------------------------------
// `Backend.argmax` (ops/sampling.zig:73-86): the index of the largest logit, the lowest index on ties,
// 0xffffffff when any logit is NaN or infinite. One kernel: every block reduces a strided share to one
// (value, index, non-finite) record in the scratch, and the block that arrives last (an arrival counter
// that it leaves at zero) reduces the records in block order; nothing depends on timing.

constexpr int ARGMAX_BLOCKS = 128;
constexpr int ARGMAX_THREADS = 256;

__device__ __forceinline__ void argmax_better(float &v, uint32_t &idx, float ov, uint32_t oi) {
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
}

__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_kernel(const float *logits, uint32_t count, float *records, uint32_t *counter, uint32_t *result) {
    __shared__ float sv[ARGMAX_THREADS / 32];
    __shared__ uint32_t si[ARGMAX_THREADS / 32], sbad[ARGMAX_THREADS / 32], last_block;
    wait_for_previous_operator();
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float v = -INFINITY;
    uint32_t idx = 0xffffffffu, bad = 0;
    for (uint32_t i = blockIdx.x * ARGMAX_THREADS + tid; i < count; i += gridDim.x * ARGMAX_THREADS) {
        const float x = logits[i];
        bad |= !isfinite(x);
        argmax_better(v, idx, x, i);
    }
    auto block_reduce = [&]() {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
            bad |= __shfl_xor_sync(0xffffffffu, bad, o);
            argmax_better(v, idx, ov, oi);
        }
        if (lane == 0) { sv[warp] = v; si[warp] = idx; sbad[warp] = bad; }
        __syncthreads();
        if (tid == 0)
            for (int w = 1; w < ARGMAX_THREADS / 32; ++w) {
                bad |= sbad[w];
                argmax_better(v, idx, sv[w], si[w]);
            }
    };
    block_reduce();
    if (tid == 0) {
        records[blockIdx.x * 4 + 0] = v;
        records[blockIdx.x * 4 + 1] = __uint_as_float(idx);
        records[blockIdx.x * 4 + 2] = __uint_as_float(bad);
        __threadfence();
        last_block = atomicAdd(counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last_block) return;
    __threadfence();
    v = -INFINITY; idx = 0xffffffffu; bad = 0;
    if (tid < gridDim.x) {
        v = __ldcg(records + tid * 4);
        idx = __float_as_uint(__ldcg(records + tid * 4 + 1));
        bad = __float_as_uint(__ldcg(records + tid * 4 + 2));
    }
    __syncthreads();
    block_reduce();
    if (tid == 0) {
        *result = bad ? 0xffffffffu : idx;
        *counter = 0;  // leave the scratch as it was found
    }
}

int launch_argmax(cudaStream_t s, const float *logits, uint32_t count, float *records, uint32_t *counter, uint32_t *result) {
    uint32_t blocks = (count + ARGMAX_THREADS - 1) / ARGMAX_THREADS;
    if (blocks > ARGMAX_BLOCKS) blocks = ARGMAX_BLOCKS;
    launch_after_previous(argmax_kernel, dim3(blocks), dim3(ARGMAX_THREADS), s, logits, count, records, counter, result);
    return 1;
}

// Expert parallelism: a rank that holds experts [first, first + count) keeps the routed slots it
// owns (index made local) and silences the others (index 0, weight 0), so that the grouped
// operators run unchanged and the partial outputs of the ranks add up to the full result.
__global__ void route_local_kernel(const uint32_t *indices, const float *weights, uint32_t n, uint32_t first, uint32_t count, uint32_t *local_indices,
                                   float *local_weights) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t e = indices[i];
    const bool mine = e >= first && e - first < count;
    local_indices[i] = mine ? e - first : 0u;
    local_weights[i] = mine ? weights[i] : 0.0f;
}

int launch_route_local(cudaStream_t s, const uint32_t *indices, const float *weights, uint32_t n, uint32_t first, uint32_t count, uint32_t *local_indices,
                       float *local_weights) {
    route_local_kernel<<<(n + 127) / 128, 128, 0, s>>>(indices, weights, n, first, count, local_indices, local_weights);
    return 1;
}

int launch_combine_experts(cudaStream_t s, const float *values, const float *weights, const uint32_t *indices, const float *scales,
                           float *out, uint32_t columns, uint32_t slots, uint32_t rows, size_t in_stride, size_t out_stride, uint32_t experts) {
    const bool vec = columns % 4 == 0 && in_stride % 4 == 0 && out_stride % 4 == 0 && (uintptr_t)values % 16 == 0 && (uintptr_t)out % 16 == 0;
    if (vec)
        launch_after_previous(combine_experts_kernel<4>, dim3((columns / 4 + 127) / 128, rows), dim3(128), s, values, weights, indices, scales, out, columns, slots,
                              in_stride, out_stride, experts);
    else
        launch_after_previous(combine_experts_kernel<1>, dim3((columns + 127) / 128, rows), dim3(128), s, values, weights, indices, scales, out, columns, slots,
                              in_stride, out_stride, experts);
    return 1;
}

}  // namespace nu
