// Launchers of the CUDA kernels. Raw device pointers and a stream in; shapes
// have been validated by the caller (backend.cu). Every launcher returns the
// number of kernels it enqueued (0 on a launch error, see cudaGetLastError).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace nu {

// ---- plain decode-and-FMA kernels (any encoding, any alignment) -----------

// Decodes `columns` values of one row to F32 or BF16.
// `w` is the start of the matrix, `row` the row to decode; `layout` as in nu_matrix.
int launch_dequant_row(cudaStream_t s, uint32_t enc, uint32_t layout, const uint8_t *w, size_t stride, uint32_t rows, uint32_t row, uint32_t columns,
                       void *out, bool out_bf16);

// out[t][r] = sum_c W[r,c] * in[t,c]; one warp per weight row, F32 FMA in
// segment order, warp-shuffle reduction. `in_bf16` reads BF16 activations.
int launch_matmul_generic(cudaStream_t s, uint32_t enc, uint32_t layout, const uint8_t *w, size_t stride, uint32_t rows, uint32_t columns,
                          const void *in, bool in_bf16, size_t in_stride, float *out, size_t out_stride, uint32_t tokens);

// Gathered form: slot s uses matrix `indices[s]` (clamped) and input row s / in_group.
// 0 when the shape is not one of the specialized forms (expert_gemv.cu); the caller then uses the generic kernel.
int launch_matvec_experts_fast(cudaStream_t s, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                               uint32_t columns, const uint32_t *indices, uint32_t slots, const float *in, size_t in_stride, uint32_t in_group,
                               float *out, size_t out_stride);
// The same with the activation pass folded in (a tensor of [gate rows][up rows] per expert; out row i = act(gate i) * up i).
int launch_matvec_experts_gated_fast(cudaStream_t s, uint32_t act, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                                     uint32_t columns, const uint32_t *indices, uint32_t slots, const float *in, size_t in_stride, uint32_t in_group,
                                     float *out, size_t out_stride);
bool expert_gemv_configure();
int launch_matvec_experts_generic(cudaStream_t s, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes,
                                  uint32_t experts, uint32_t rows, uint32_t columns, const uint32_t *indices, uint32_t slots,
                                  const float *in, size_t in_stride, uint32_t in_group, float *out, size_t out_stride);

// ---- element-wise and routing kernels -------------------------------------

enum Act : uint32_t { ACT_NONE = 0, ACT_SILU = 1, ACT_GELU = 2 };
// out[r][i] = act(gate[r][i]) * up[r][i]; out may alias gate exactly.
int launch_act_mul_rows(cudaStream_t s, uint32_t act, const float *gate, const float *up, float *out,
                        uint32_t width, uint32_t rows, size_t gate_stride, size_t up_stride, size_t out_stride);
// output[row] = rms_norm(residual[row] (+ input[row], stored back into residual)) * weight; input may be null.
int launch_norm_rows(cudaStream_t s, float *residual, const float *input, const float *weight, float *output, uint32_t width, uint32_t rows, size_t in_stride,
                     size_t out_stride, float eps);
int launch_add(cudaStream_t s, float *x, const float *y, size_t count);
int launch_route(cudaStream_t s, const float *logits, uint32_t experts, uint32_t k, uint32_t rows, size_t in_stride,
                 uint32_t *indices, float *weights);
// Index of the largest of `count` logits (lowest index on ties; 0xffffffff if any is not finite). `records`: 4 floats per block
// of scratch (at most 128 blocks); `counter`: one zero word, left zero.
int launch_argmax(cudaStream_t s, const float *logits, uint32_t count, float *records, uint32_t *counter, uint32_t *result);
int launch_expert_lists(cudaStream_t s, const uint32_t *indices, uint32_t n, uint32_t experts, uint32_t bound, uint32_t *lists);
int launch_matmul_experts_generic(cudaStream_t s, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows,
                                  uint32_t columns, const uint32_t *lists, uint32_t bound, const float *in, size_t in_stride, uint32_t in_group,
                                  float *out, size_t out_stride);
int launch_route_local(cudaStream_t s, const uint32_t *indices, const float *weights, uint32_t n, uint32_t first, uint32_t count, uint32_t *local_indices,
                       float *local_weights);
int launch_combine_experts(cudaStream_t s, const float *values, const float *weights, const uint32_t *indices, const float *scales,
                           float *out, uint32_t columns, uint32_t slots, uint32_t rows, size_t in_stride, size_t out_stride, uint32_t experts);

// ---- fused dequant tensor-core GEMV / small-M GEMM (1..8 token rows) ------

// Where a one-token GEMV sends its output rows when an allreduce over peer memory follows it: slot
// [parity][rank] of every rank's inbox (push_allreduce.cu), as (value, tag) words.
struct PushTarget {
    uint2 *inbox[8];
    uint32_t ranks, rank;   // ranks == 0: no push, the output goes to `out`
    uint32_t capacity;      // words per inbox slot
    const uint32_t *seq;    // the allreduce's sequence number in this rank's memory
};
// Tag of the words of call `seq`: never 0, which is what an inbox word holds before anything was pushed to it.
__host__ __device__ inline uint32_t push_tag(uint32_t seq) { return seq + 1u ? seq + 1u : 1u; }
struct FastSegment {
    const uint8_t *w;  // first row of the (expert's) matrix
    size_t stride;     // bytes per weight row
    uint32_t rows;
    float *out;        // [tokens][out_stride]
    size_t out_stride;
};
struct FastJob {
    uint32_t enc;
    uint32_t layout;  // 0: GGUF rows; 1, 2: the planar forms made by launch_prepare (see prepare.cu)
    uint32_t columns;
    uint32_t tokens;  // 1..8
    const float *in;  // [tokens][in_stride]
    size_t in_stride;
    uint32_t count;  // segments, 1..4
    uint32_t mode;   // ACT_NONE: plain; ACT_SILU/ACT_GELU: out = act(seg0) * seg1 (count == 2)
    FastSegment seg[4];
    // Scratch owned by the handle: split-K partial sums and arrival counters
    // (zero between launches; the kernel leaves them zero).
    float *partials;
    size_t partials_floats;
    uint32_t *counters;
    size_t counters_len;
    int sm_count;
    bool serial;  // a weights buffer was written earlier in the same recording: no early start of the weight stream
    PushTarget push;
    // The add + RMS norm ahead of the projections, folded into the kernel's staging pass when norm_weight is set
    // (i8_kernel.cuh, Params): `in` is then the residual rows, norm_input what is added to them (or null),
    // residual_out where the sums go (or null); all at in_stride.
    const float *norm_weight;
    const float *norm_input;
    float *residual_out;
    float norm_eps;
    const float *add0;  // not null: the output rows of the (single, plain) segment are add0[...] + the products, at the output's stride
};
// Opts every variant into its dynamic shared memory size; once per device, outside any capture.
bool fast_configure();
// Whether the fast kernel serves this job (encoding, alignment, sizes, scratch).
bool fast_supported(const FastJob &job);
int launch_fast(cudaStream_t s, const FastJob &job);

// ---- 1..8 activation rows on Q4_K, integer tensor path (gemv_q4k_i8.cu) ------------
bool q4k_i8_configure();
bool q4k_i8_supported(const FastJob &job);
int launch_q4k_i8(cudaStream_t s, const FastJob &job);
// The K slices and blocks the launch would use (host arithmetic only).
bool q4k_i8_plan(const FastJob &job, uint32_t *slices, uint32_t *blocks);
// ---- 1..8 activation rows on planar Q6_K, integer tensor path (gemv_q6k_i8.cu) -----
bool q6k_i8_configure();
bool q6k_i8_supported(const FastJob &job);
int launch_q6k_i8(cudaStream_t s, const FastJob &job);
// ---- 1..8 activation rows on planar Q8_0, integer tensor path (gemv_q8_0_i8.cu) -----
bool q8_0_i8_configure();
bool q8_0_i8_supported(const FastJob &job);
int launch_q8_0_i8(cudaStream_t s, const FastJob &job);
// ---- 1..8 activation rows on planar Q5_0 / Q5_1 / Q4_0 / IQ4_NL, integer tensor path (gemv_block32_i8.cu) -
bool block32_i8_configure();
bool block32_i8_supported(const FastJob &job);
int launch_block32_i8(cudaStream_t s, const FastJob &job);

// ---- 1..8 activation rows on Q5_K, integer tensor path (gemv_q5k_i8.cu) ------------
bool q5k_i8_configure();
bool q5k_i8_supported(const FastJob &job);
int launch_q5k_i8(cudaStream_t s, const FastJob &job);

// ---- 1..8 activation rows on planar Q2_K / Q3_K, integer tensor path (gemv_q23k_i8.cu) -
bool q23k_i8_configure();
bool q23k_i8_supported(const FastJob &job);
int launch_q23k_i8(cudaStream_t s, const FastJob &job);
// ---- a run of one-token integer-path jobs as one persistent launch (gemv_chain.cu) --
constexpr int kChainMax = 16;
bool chain_configure();
bool chain_supported(const FastJob &job);
// jobs[0..n), 2 <= n <= kChainMax, in order; arrivals: two zero words the kernel leaves zero. 0: nothing was launched.
int launch_chain(cudaStream_t s, const FastJob *jobs, uint32_t n, uint32_t *arrivals, int sm_count);
// ---- prefill GEMM on tcgen05 (many token rows, bf16 operands, f32 accumulate) -------
struct PrefillJob {
    uint32_t enc, layout;
    const uint8_t *w;
    size_t stride;
    uint32_t rows, columns;
    const void *in;          // bf16 [padded_tokens][in_stride]
    size_t in_stride;        // in elements
    uint32_t tokens, padded_tokens;
    float *out;              // [tokens][out_stride]
    size_t out_stride;
    uint32_t *status;
    int sm_count;
};
bool prefill_configure();
bool prefill_supported(const PrefillJob &job);
int launch_prefill(cudaStream_t s, const PrefillJob &job);
// The prefill of a mixture-of-experts layer on the tensor cores: slot rows grouped by expert (`lists`, as launch_expert_lists
// wrote them), gathered into whole 64-row tiles in `scratch`, one block per (tile, 128 weight rows). 0 when the form does not apply.
size_t matmul_experts_scratch(uint32_t n, uint32_t experts, uint32_t columns);
int launch_matmul_experts_fast(cudaStream_t s, uint32_t enc, const uint8_t *w, size_t stride, size_t expert_bytes, uint32_t experts, uint32_t rows, uint32_t columns,
                               const uint32_t *lists, uint32_t bound, uint32_t n, const float *in, size_t in_stride, uint32_t in_group, float *out, size_t out_stride,
                               void *scratch, size_t scratch_bytes, uint32_t *status);
int launch_f32_to_bf16_rows(cudaStream_t s, const float *in, size_t in_stride, void *out, size_t out_stride, uint32_t columns, uint32_t tokens);

// ---- one-shot allreduce over peer memory (push_allreduce.cu) ------------------------
constexpr int PUSH_MAX_RANKS = 8;
constexpr int PUSH_MAX_BLOCKS = 32;
struct PushParams {
    float *buf;                         // this rank's vector, summed in place
    uint32_t count, ranks, rank;
    uint32_t capacity;                  // 8-byte words per inbox slot
    uint2 *inbox[PUSH_MAX_RANKS];       // every rank's inbox [2][ranks][capacity] of (value, tag); inbox[rank] is local
    uint32_t *seq;                      // local: sequence number, finished blocks, sticky failure
    uint32_t *status;
    unsigned long long wait_ns;         // how long a rank polls for its peers' words before it gives up
    float *add_to;                      // not null: the sums are added to this vector (a residual) instead of replacing `buf`
};
int launch_push_allreduce(cudaStream_t s, const PushParams &p);
// The second half alone: the vector was already pushed (by the GEMV that produced it) into every inbox, this rank's included.
int launch_gather_sum(cudaStream_t s, const PushParams &p);

// ---- planar re-layout of a matrix for the specialized kernels ---------------------
// Layout the matrix takes after preparation: 0 when the specialized kernels read the GGUF rows as they are.
uint32_t prepared_layout(uint32_t enc, uint32_t rows, uint32_t columns);
int launch_prepare(cudaStream_t s, uint32_t enc, const uint8_t *src, uint8_t *dst, uint32_t rows, uint32_t columns);

}  // namespace nu
