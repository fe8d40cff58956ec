/*
 * nuclis_cuda.h: C ABI of the B200 (sm_100a) backend for nuclis's
 * quantized-weight matmul path.
 *
 * The engine's Metal backend reaches its GPU through 16 generic `nu_metal_*`
 * functions (inference/src/backends/metal/root.zig:28-44, implemented in
 * inference/src/backends/metal/bridge.m) that compile shader source at start
 * and record untyped dispatches. CUDA kernels are compiled ahead of time, so
 * this ABI keeps the bridge's lifecycle functions (create, buffers,
 * begin/commit/discard, GPU seconds, profile) and replaces the untyped
 * `nu_metal_dispatch` with one typed entry point per operator of
 * `metal.Backend` (inference/src/backends/metal/ops/{matvec,matmul,experts,
 * rowwise}.zig). Each declaration cites the reference interface it replaces.
 *
 * Conventions, as in bridge.m:49-51 and root.zig:7-10:
 *   - `int` results: 0 is success, any other value one of `nu_status`.
 *   - An opaque handle per device context. A handle is NOT thread-safe: one
 *     thread owns it, one recording is open at a time.
 *   - Every shape or length violation is reported BEFORE anything is recorded;
 *     a recording that met an error is dropped with `nu_cuda_discard`.
 *   - `nu_cuda_commit` submits and waits: afterwards every recorded write is
 *     visible to `nu_cuda_buffer_download`.
 *   - Buffers are named by `(id, offset, len)` triples (`Buffer` of
 *     root.zig:62-86); ids are never reused.
 *   - Matrices are row-major GGUF rows, `columns` contiguous and block
 *     quantized (`cpu.Matrix`, inference/src/backends/cpu/root.zig:28-36).
 *
 * Plain C: pointers, sizes and fixed-width integers only.
 */
#ifndef NUCLIS_CUDA_H
#define NUCLIS_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error set: quant.Error (inference/src/quant/decode.zig:22), cpu.Error
 * (backends/cpu/root.zig:38) and the Metal backend's own errors
 * (backends/metal/root.zig), as integers. */
typedef enum nu_status {
    NU_OK = 0,
    NU_ERR_UNSUPPORTED_ENCODING = 1, /* error.UnsupportedTensorEncoding */
    NU_ERR_INVALID_ROW_LENGTH = 2,   /* error.InvalidRowLength */
    NU_ERR_INVALID_BYTE_LENGTH = 3,  /* error.InvalidByteLength */
    NU_ERR_INVALID_SHAPE = 4,        /* error.InvalidShape */
    NU_ERR_MERGE_DECLINED = 5,       /* error.MergeDeclined (ops/matvec.zig:245-257) */
    NU_ERR_NOT_RECORDING = 6,        /* error.MetalNotRecording */
    NU_ERR_ALREADY_RECORDING = 7,    /* error.MetalAlreadyRecording */
    NU_ERR_BUFFER = 8,               /* error.MetalBufferFailed */
    NU_ERR_EXECUTION = 9,            /* error.MetalExecutionFailed */
    NU_ERR_INIT = 10,                /* error.MetalInitializationFailed */
    NU_ERR_COMM = 11,                /* collective set-up or call failed (no reference analogue) */
    NU_ERR_TOO_LARGE = 12            /* beyond a fixed capacity of this library */
} nu_status;

/* GGML encoding ids served (inference/src/tensor/encoding.zig:29-56). */
enum { NU_F32 = 0, NU_F16 = 1, NU_Q4_0 = 2, NU_Q5_0 = 6, NU_Q5_1 = 7, NU_Q8_0 = 8, NU_Q2_K = 10, NU_Q3_K = 11, NU_Q4_K = 12, NU_Q5_K = 13, NU_Q6_K = 14, NU_IQ4_NL = 20, NU_IQ4_XS = 23, NU_BF16 = 30 };

/* `Buffer` of backends/metal/root.zig:62-86 without the host pointer: device
 * memory is not host-addressable here; use upload/download. */
typedef struct nu_buffer {
    uint32_t id;
    uint32_t reserved;
    uint64_t offset; /* bytes from the start of buffer `id` */
    uint64_t len;    /* bytes this view may touch */
} nu_buffer;

/* `cpu.Matrix` (backends/cpu/root.zig:31-36): `bytes` is the byte length of
 * the whole matrix; the row stride is bytes / rows. */
typedef struct nu_matrix {
    uint32_t encoding;
    uint32_t layout; /* 0: GGUF rows as stored in the file; otherwise the value nu_cuda_matrix_prepare returned */
    uint64_t rows;
    uint64_t columns;
    uint64_t bytes;
} nu_matrix;

/* `cpu.ExpertMatrix` (backends/cpu/experts.zig:20-43): experts contiguous. */
typedef struct nu_expert_matrix {
    uint32_t encoding;
    uint32_t reserved;
    uint64_t experts;
    uint64_t rows;
    uint64_t columns;
    uint64_t bytes;
} nu_expert_matrix;

/* `Segment` and `SegmentMode` of ops/matvec.zig:223-225. */
typedef struct nu_segment {
    nu_buffer weights;
    nu_matrix matrix;
    nu_buffer output;
} nu_segment;
enum { NU_SEGMENTS_PLAIN = 0, NU_SEGMENTS_SILU_MUL_PAIR = 1, NU_SEGMENTS_GELU_MUL_PAIR = 2 };

/* `CombineShape` of ops/experts.zig:80. */
typedef struct nu_combine_shape {
    uint64_t columns, slots, rows, experts, in_stride, out_stride;
} nu_combine_shape;

typedef struct nu_cuda nu_cuda;

/* ---- lifecycle (bridge.m nu_metal_create / nu_metal_destroy) ------------- */

/* Opens CUDA device `device`, creates the stream all work runs on and the
 * library's fixed scratch. NULL on failure with a message in `err`. */
nu_cuda *nu_cuda_create(int device, char *err, size_t err_cap);
void nu_cuda_destroy(nu_cuda *h);
/* Message of the last failed call on this handle ("" if none). */
const char *nu_cuda_last_error(const nu_cuda *h);
/* Name of a status code, e.g. "InvalidShape". */
const char *nu_cuda_status_name(int status);
/* `Backend.generic_only` (root.zig:99-104): force the plain decode-and-FMA
 * kernels even where a specialized kernel applies. */
int nu_cuda_set_generic_only(nu_cuda *h, int on);
/* No counterpart in the reference. With `on` != 0, one-token matvecs on the
 * specialized kernels that are recorded back to back (a decode layer's QKV, O,
 * gate/up pair and down projections) are launched as ONE persistent kernel that
 * walks them in order, a grid-wide barrier between two of them: the weight
 * stream of an operator starts while other blocks still finish the one before.
 * Same results bit for bit. Off by default: on a B200 the barrier and the
 * per-operator set-up inside one resident block cost more than the launches
 * they replace (225 against 289 tokens/s on the 64-layer stack). Takes effect
 * at the next operator recorded. */
int nu_cuda_set_chaining(nu_cuda *h, int on);

/* ---- buffers (nu_metal_buffer_create / wrap / contents / release) -------- */

/* Zero-filled device buffer of `len` bytes owned by the handle. */
int nu_cuda_buffer_create(nu_cuda *h, size_t len, uint32_t *id);
/* Copies host bytes into / out of a buffer; refused while recording. These
 * replace nu_metal_buffer_contents: device memory has no host pointer. */
int nu_cuda_buffer_upload(nu_cuda *h, uint32_t id, size_t offset, const void *src, size_t len);
int nu_cuda_buffer_download(nu_cuda *h, uint32_t id, size_t offset, void *dst, size_t len);
/* `Backend.wrap` (root.zig:217-230): the first wrap of a host range uploads it
 * once; later wraps of the same start address return the same id and must ask
 * for the same length. The host range is only read during the first call. */
int nu_cuda_buffer_wrap(nu_cuda *h, const void *bytes, size_t len, uint32_t *id);
/* `Backend.unwrap` / `release` (root.zig:206-242): refused while recording. */
int nu_cuda_buffer_unwrap(nu_cuda *h, const void *bytes);
int nu_cuda_buffer_release(nu_cuda *h, uint32_t id);
/* Device address of a buffer, for callers that fill it with their own CUDA
 * code (tests, benchmarks). NULL for an unknown id. */
void *nu_cuda_buffer_device_ptr(nu_cuda *h, uint32_t id);
/* `Backend.created_bytes` (root.zig:113-116). */
uint64_t nu_cuda_created_bytes(const nu_cuda *h);

/* Re-lays a matrix once, at load time, into the form the specialized kernels read
 * (no reference analogue; the reference wraps the file bytes as they are,
 * root.zig:217-230). GGUF rows of some encodings start on 2-byte boundaries
 * (Q6_K blocks are 210 bytes, Q8_0 blocks 34, Q4_0 and IQ4_NL 18, Q5_0 22, Q5_1 24, Q3_K superblocks 110; IQ4_XS
 * and Q2_K superblocks, 136 and 84 bytes, on 8- and 4-byte ones), which no vector load or bulk copy can address;
 * the prepared form holds the same bytes in 16-byte aligned planes and decodes
 * to the same values bit for bit. `prepared` must be as long as the matrix and
 * must not overlap it; `layout` receives the value to put in `nu_matrix.layout`
 * (0 when the encoding needs no re-layout: the bytes are then copied as they
 * are). Refused while recording. Every operator that takes a matrix accepts
 * both forms, except the expert operators (GGUF form only). */
int nu_cuda_matrix_prepare(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix,
                           const nu_buffer *prepared, uint32_t *layout);

/* ---- recording (nu_metal_begin / commit / discard / gpu_seconds) --------- */

/* Opens a recording: operator calls between begin and commit are captured
 * into a CUDA graph, not run. */
int nu_cuda_begin(nu_cuda *h);
/* Instantiates the recorded graph, launches it and waits. */
int nu_cuda_commit(nu_cuda *h);
/* Drops the open recording; nothing of it runs. No-op when idle. */
int nu_cuda_discard(nu_cuda *h);
/* As commit, but keeps the instantiated graph for replay: a decode step
 * records the same operators every token, so it is recorded once. */
int nu_cuda_commit_retain(nu_cuda *h, uint32_t *graph);
/* Replays a retained graph `count` times back to back and waits; when
 * `elapsed_ms` is not NULL it receives the device time of the whole batch
 * (CUDA events on the handle's stream). */
int nu_cuda_graph_launch(nu_cuda *h, uint32_t graph, uint32_t count, float *elapsed_ms);
int nu_cuda_graph_release(nu_cuda *h, uint32_t graph);
/* Seconds of device time of everything committed so far (nu_metal_gpu_seconds). */
double nu_cuda_gpu_seconds(const nu_cuda *h);
/* Kernels recorded or launched by this handle so far. */
uint64_t nu_cuda_launch_count(const nu_cuda *h);
/* The CUDA stream (a `cudaStream_t`) of this handle, for callers that time
 * with their own events. */
void *nu_cuda_stream(nu_cuda *h);
/* Per-operator timing (nu_metal_profile_enable / nu_metal_profile_read):
 * once enabled, commit runs each recorded operator between its own pair of
 * events; `nu_cuda_profile_read` returns how many durations (seconds, in
 * recording order) the last commit produced and copies up to `cap` of them. */
int nu_cuda_profile_enable(nu_cuda *h, uint32_t max_ops);
uint32_t nu_cuda_profile_read(nu_cuda *h, double *seconds, uint32_t cap);

/* ---- operators ----------------------------------------------------------- */

/* `Backend.embed` (ops/rowwise.zig:15-25): decode row `token` of `matrix` to
 * F32, bit-identical to the CPU decoder. `out_dtype` NU_F32 or NU_BF16 (round
 * to nearest even of the F32 value; no reference analogue). */
int nu_cuda_embed(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix, uint32_t token,
                  const nu_buffer *output, uint32_t out_dtype);

/* `Backend.matvec` (ops/matvec.zig:32-34, 85-116): output[r] = sum_c W[r,c]*input[c]. */
int nu_cuda_matvec(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix,
                   const nu_buffer *input, const nu_buffer *output);

/* `Backend.matvecRows` (ops/matvec.zig:149-165): 2..8 token rows, strides in floats. */
int nu_cuda_matvec_rows(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix,
                        const nu_buffer *input, size_t in_stride,
                        const nu_buffer *output, size_t out_stride, size_t tokens);

/* `Backend.matmul` (ops/matmul.zig:62-108): out[t][r] = sum_c W[r,c]*in[t,c].
 * `in_dtype` NU_F32 (the reference's contract; strides in elements) or
 * NU_BF16 (prefill activations already rounded; no reference analogue).
 * Buffers hold `matmul_padded(tokens)` rows as in ops/matmul.zig:29-31. */
int nu_cuda_matmul(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix,
                   const nu_buffer *input, uint32_t in_dtype, size_t in_stride,
                   const nu_buffer *output, size_t out_stride, size_t tokens);
size_t nu_cuda_matmul_padded(size_t tokens);

/* `Backend.matvecSegments` (ops/matvec.zig:245-343): up to four projections of
 * one input in one launch; the pair modes write act(seg[0]) * seg[1] only. */
int nu_cuda_matvec_segments(nu_cuda *h, const nu_segment *segments, size_t count,
                            const nu_buffer *input, uint32_t mode);

/* `Backend.matvec` followed by the residual `Backend.add` of its output (ops/matvec.zig:85-116, then
 * ops/rowwise.zig:199-202; what a decoder layer does behind its O and down projections,
 * inference/src/models/qwen35_metal.zig:640) as one launch: output = residual + W x, the add folded into the
 * kernel's write. No single call of the reference does this. `output` may be `residual` itself; any other overlap
 * is refused. A matrix the specialized kernels do not serve takes the generic matvec and the add: the call never
 * declines. */
int nu_cuda_matvec_add(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix, const nu_buffer *input,
                       const nu_buffer *residual, const nu_buffer *output);

/* `Backend.addRmsNorm` followed by `Backend.matvecSegments` on its output (ops/rowwise.zig:76-93, then
 * ops/matvec.zig:245-343; the pair a decoder layer runs ahead of its projections,
 * inference/src/models/qwen35_metal.zig:635-640) as ONE launch: the kernel's staging pass, which reads the whole
 * input row in every block anyway, adds, takes the mean square and scales. No single call of the reference does
 * this. The rows the segments multiply are norm(residual + input) * weight with `eps` inside the root;
 * residual + input is written to `residual_out`, which must not overlap `residual` or `input` (every block reads
 * them while one writes the sum: keep two residual buffers and swap them). `input` and `residual_out` may both be
 * null: then it is `rmsNorm` + `matvecSegments`. One token row; buffers 16-byte aligned. Returns
 * NU_ERR_MERGE_DECLINED, with nothing recorded, when the specialized kernel does not serve the segments: the caller
 * then runs the two operators. */
int nu_cuda_matvec_segments_normed(nu_cuda *h, const nu_segment *segments, size_t count, const nu_buffer *residual,
                                   const nu_buffer *input, const nu_buffer *weight, const nu_buffer *residual_out,
                                   float eps, uint32_t mode);

/* `Backend.siluMul`, `Backend.geluMul` (ops/rowwise.zig:209, 230): gate[i] = act(gate[i]) * up[i]. */
int nu_cuda_silu_mul(nu_cuda *h, const nu_buffer *gate, const nu_buffer *up, size_t count);
int nu_cuda_gelu_mul(nu_cuda *h, const nu_buffer *gate, const nu_buffer *up, size_t count);

/* `Backend.route` (ops/experts.zig:29-34). */
int nu_cuda_route(nu_cuda *h, const nu_buffer *logits, size_t experts, size_t k, size_t rows, size_t in_stride,
                  const nu_buffer *indices, const nu_buffer *weights);

/* `Backend.expertLists` (ops/experts.zig:137-146): groups the rows * k slot rows of `indices` ([row][k], as
 * route writes them) by expert into `lists`, nu_cuda_expert_lists_words(rows * k, experts) 32-bit words in
 * the reference's layout: the tile count, n, experts + 1 exclusive prefix offsets, the tiles of at most 32
 * slot rows as (expert, first, count), and the n slot rows grouped by expert. At most 256 experts. */
size_t nu_cuda_expert_lists_words(size_t slot_rows, size_t experts);
int nu_cuda_expert_lists(nu_cuda *h, const nu_buffer *indices, size_t rows, size_t k, size_t experts, const nu_buffer *lists);
/* `Backend.matmulExperts` (ops/experts.zig:162-202): for each slot row s of the lists,
 * output[s * out_stride + r] = W[e_s][r] . input[(s / in_group) * in_stride]; weights are read once per
 * tile of an expert's slot rows; exactly rows * k output rows are written. Same shape rules as matmul
 * (columns % 64, rows % 8, 16-byte aligned input). */
int nu_cuda_matmul_experts(nu_cuda *h, const nu_buffer *weights, const nu_expert_matrix *tensor, const nu_buffer *lists, size_t rows, size_t k,
                           const nu_buffer *input, size_t in_stride, size_t in_group, const nu_buffer *output, size_t out_stride);

/* Expert parallelism (no counterpart in the reference, which is single-device): a rank that holds
 * experts [first_expert, first_expert + local_experts) turns the routed slots into its own view:
 * slots it owns keep their weight and get the expert's local index, the others get index 0 and
 * weight 0. The grouped operators then run unchanged on the rank's slice of the expert tensors and
 * the partial outputs of all ranks add up (nu_cuda_allreduce_sum_f32) to the full result. */
int nu_cuda_route_local(nu_cuda *h, const nu_buffer *indices, const nu_buffer *weights, size_t count, size_t first_expert, size_t local_experts,
                        const nu_buffer *local_indices, const nu_buffer *local_weights);

/* `Backend.matvecExperts` / `matvecExpertsGrouped` (ops/experts.zig:44-77). */
int nu_cuda_matvec_experts(nu_cuda *h, const nu_buffer *weights, const nu_expert_matrix *tensor,
                           const nu_buffer *indices, size_t slots,
                           const nu_buffer *input, size_t in_stride, size_t in_group,
                           const nu_buffer *output, size_t out_stride);

/* `Backend.matvecExpertsGrouped` on a gate_up tensor followed by `Backend.geluMulRows` on the two halves of its output
 * (ops/experts.zig:36-77, then 106-117) as one launch: output[slot][i] = act(gate row i . x) * (up row i . x) for
 * i < rows / 2, where `tensor` holds [gate rows][up rows] per expert. No single call of the reference does this.
 * `act`: 1 SiLU, 2 GELU. Tensors the specialized kernel does not serve take the GEMV and the activation pass as
 * two launches: the call never declines. */
int nu_cuda_matvec_experts_gated(nu_cuda *h, const nu_buffer *weights, const nu_expert_matrix *tensor, const nu_buffer *indices,
                                 size_t slots, const nu_buffer *input, size_t in_stride, size_t in_group,
                                 const nu_buffer *output, size_t out_stride, uint32_t act);

/* `Backend.geluMulRows` (ops/experts.zig:106-117). */
int nu_cuda_gelu_mul_rows(nu_cuda *h, const nu_buffer *gate, const nu_buffer *up, const nu_buffer *output,
                          size_t width, size_t rows, size_t gate_stride, size_t up_stride, size_t out_stride);

/* The steps on either side of a projection in a decoder layer (models/qwen35_metal.zig:630-640).
 * `Norm` of ops/rowwise.zig:24-35: `rows` rows of `width` floats, strides in floats, eps > 0. */
typedef struct nu_norm {
    size_t rows, width, in_stride, out_stride;
    float eps;
} nu_norm;
/* `Backend.rmsNorm` (ops/rowwise.zig:37-51): output = input * rsqrt(mean(input^2) + eps) * weight, per row.
 * `output` may alias `input` exactly. */
int nu_cuda_rms_norm(nu_cuda *h, const nu_buffer *input, const nu_buffer *weight, const nu_buffer *output, const nu_norm *spec);
/* `Backend.addRmsNorm` (ops/rowwise.zig:76-93): residual += input, then output = norm(residual) * weight, in
 * one pass over the row. `input` shares the residual's stride and overlaps neither it nor `output`. */
int nu_cuda_add_rms_norm(nu_cuda *h, const nu_buffer *residual, const nu_buffer *input, const nu_buffer *weight, const nu_buffer *output, const nu_norm *spec);
/* `Backend.add` (ops/rowwise.zig:199-202): x[0..count) += y[0..count). */
int nu_cuda_add(nu_cuda *h, const nu_buffer *x, const nu_buffer *y, size_t count);

/* `Backend.argmax` (ops/sampling.zig:73-86): greedy selection over the output head's logits. `result` receives one
 * uint32: the index of the largest of `count` F32 logits, the lowest index on ties, or 0xffffffff when any
 * logit is NaN or infinite. The scratch of the reference's two passes belongs to the handle here. */
int nu_cuda_argmax(nu_cuda *h, const nu_buffer *logits, size_t count, const nu_buffer *result);

/* `Backend.combineExperts` (ops/experts.zig:79-92); `scales` may be NULL. */
int nu_cuda_combine_experts(nu_cuda *h, const nu_buffer *values, const nu_buffer *weights, const nu_buffer *indices,
                            const nu_buffer *scales, const nu_buffer *output, const nu_combine_shape *shape);

/* Q4_K decode GEMV for callers that must not allocate. It has no counterpart in the
 * reference. Some hosts of this library run where device memory cannot be obtained at
 * call time: inside another runtime's memory plan that has handed out all of its arena,
 * in a plugin sandbox that forbids cudaMalloc, or in a real-time loop where an allocation's
 * latency and failure mode are unacceptable. `nu_cuda_create` allocates its scratch with
 * cudaMalloc; this entry point needs no handle and calls no cudaMalloc, cudaFree or
 * allocating library routine. The split-K partial sums and arrival counters of the kernel
 * live in an array inside the library image (about 1 MiB, held by every GPU that loads the
 * library until the process exits).
 *
 *   weights  device pointer, 16-byte aligned: `rows` contiguous GGUF Q4_K rows of `columns`
 *            values, `stride` = columns / 256 * 144 bytes apart
 *   input    device pointer, 16-byte aligned: `columns` floats
 *   output   device pointer: `rows` floats
 *   stream   a cudaStream_t (NULL for the default stream); the call only enqueues work
 *
 * Limits: at most 65,536 rows, 20,480 columns and 1 MiB of partial sums; beyond them the
 * call fails with NU_ERR_TOO_LARGE and a message in `err`, before anything is enqueued.
 * The first call on a device looks the array's device address up and configures the kernel:
 * make that first call outside any stream capture. All calls on a device share the one array,
 * which keeps the previous call's contents (the counters are cleared at the start of each
 * call): two calls whose kernels overlap on the GPU, on different streams, race on it.
 * Results are those of nu_cuda_matvec on the same data. */
int nu_cuda_matvec_q4k_static(const void *weights, size_t stride, uint32_t rows, uint32_t columns,
                              const float *input, float *output, void *stream, char *err, size_t err_cap);
/* Two helpers of the entry point above (no counterpart in the reference either; neither allocates).
 * `_plan` is host arithmetic only: how many K slices and blocks a call of that shape would use on a
 * GPU of `sm_count` multiprocessors (more than one slice means the built-in array is used), or
 * NU_ERR_TOO_LARGE when no way to cut the shape fits the array. `_status` waits for `stream` and
 * reads the word the kernel raises when one of its bounded waits ran out (0: all calls so far on
 * this device completed their copies); the entry point itself only enqueues and cannot report that. */
int nu_cuda_matvec_q4k_static_plan(uint32_t rows, uint32_t columns, uint32_t sm_count, uint32_t *slices, uint32_t *blocks);
int nu_cuda_matvec_q4k_static_status(void *stream, uint32_t *status);

/* ---- tensor-parallel collective (no reference analogue: the reference is
 * single-device) ---------------------------------------------------------- */

/* Size in bytes of the opaque rendezvous id below. */
enum { NU_COMM_ID_BYTES = 128 };
/* Rank 0 fills `id`; the caller carries it to the other ranks by any means. */
int nu_cuda_comm_unique_id(uint8_t id[NU_COMM_ID_BYTES]);
/* Joins this handle to a group of `ranks` handles (one per GPU). Collective. */
int nu_cuda_comm_init(nu_cuda *h, const uint8_t id[NU_COMM_ID_BYTES], int ranks, int rank);
/* In-place sum over the group of `count` floats at `buffer`; recorded like an operator. */
int nu_cuda_allreduce_sum_f32(nu_cuda *h, const nu_buffer *buffer, size_t count);
/* The same with the residual add behind a row-split projection folded in: residual[i] += sum over the group of
 * buffer[i]; `buffer` is left with this rank's partial values or the sums, depending on the transport. Every rank
 * adds the same sums in the same order, so identical residuals stay identical. `residual` must not overlap `buffer`. */
int nu_cuda_allreduce_sum_add_f32(nu_cuda *h, const nu_buffer *buffer, const nu_buffer *residual, size_t count);
/* One-shot allreduce over peer memory for short vectors (at most 65,536 floats): at 20 KB a
 * collective is pure latency, and this path costs one peer store and a local sum instead of
 * a library call. Each rank calls nu_cuda_comm_peer_handle (it allocates the rank's inbox and
 * returns a 64-byte interprocess handle), the handles travel to every rank by any means, ordered by
 * rank, and each rank calls nu_cuda_comm_attach_peers with all of them. From then on
 * nu_cuda_allreduce_sum_f32 uses this path for vectors that fit and NCCL (if a group was joined)
 * for longer ones. All ranks must make the same sequence of allreduce calls. One process per GPU. */
enum { NU_PEER_HANDLE_BYTES = 64 };
int nu_cuda_comm_peer_handle(nu_cuda *h, uint8_t handle[NU_PEER_HANDLE_BYTES]);
int nu_cuda_comm_attach_peers(nu_cuda *h, const uint8_t *handles, int ranks, int rank);
/* How long a rank's kernel polls its inbox for the peers' words before it gives up (default 2,000 ms;
 * 1..60,000). When the limit runs out the kernel returns, the next commit / graph_launch reports
 * NU_ERR_EXECUTION, and the peer-memory path of this handle stays closed (every later sum over it fails
 * at once) until the group is destroyed. Applies to operators recorded after the call. */
int nu_cuda_comm_set_wait_ms(nu_cuda *h, uint32_t ms);
/* Leaves the group. Every retained graph of the handle is released first (a graph
 * that holds a collective keeps the communicator alive). */
int nu_cuda_comm_destroy(nu_cuda *h);

#ifdef __cplusplus
}
#endif
#endif /* NUCLIS_CUDA_H */
