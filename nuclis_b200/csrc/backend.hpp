// Host side of the CUDA backend: the C++ mirror of `metal.Backend`
// (inference/src/backends/metal/root.zig:88-330 and ops/*.zig). Same method
// names, argument meaning and error behaviour; the C ABI in
// include/nuclis_cuda.h is a thin wrapper over this class.
//
// Ownership and threading follow the reference (root.zig:7-10): created
// buffers live until release or destruction, wrapped host ranges are uploaded
// once and cached by start address, one thread owns a backend, one recording
// is open at a time, and commit() waits.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/nuclis_cuda.h"

namespace nu {

struct FastJob;
struct FastJobBox;
struct FastChain;
struct FastJob;

using Buffer = nu_buffer;
using Matrix = nu_matrix;
using ExpertMatrix = nu_expert_matrix;
using Segment = nu_segment;

class Backend {
public:
    static Backend *create(int device, std::string &error);
    ~Backend();

    // ---- knobs (root.zig:99-114) ----
    bool generic_only = false;
    bool chaining = false;  // back-to-back one-token matvecs become one persistent launch (gemv_chain.cu); measured slower than
                            // kernels of their own with programmatic dependent launch, so off unless asked for

    // ---- buffers ----
    int createBuffer(size_t len, uint32_t *id);
    int upload(uint32_t id, size_t offset, const void *src, size_t len);
    int download(uint32_t id, size_t offset, void *dst, size_t len);
    int wrap(const void *bytes, size_t len, uint32_t *id);
    int unwrap(const void *bytes);
    int release(uint32_t id);
    void *devicePtr(uint32_t id);
    uint64_t createdBytes() const { return created_bytes_; }
    int prepare(const Buffer &weights, const Matrix &matrix, const Buffer &prepared, uint32_t *layout);

    // ---- recording ----
    int begin();
    int commit();
    int commitRetain(uint32_t *graph);
    int graphLaunch(uint32_t graph, uint32_t count, float *elapsed_ms);
    int graphRelease(uint32_t graph);
    int discard();
    double gpuSeconds() const { return gpu_seconds_; }
    uint64_t launchCount() const { return launches_; }
    cudaStream_t stream() const { return stream_; }
    int profileEnable(uint32_t max_ops);
    uint32_t profileRead(double *seconds, uint32_t cap);

    // ---- operators (ops/matvec.zig, ops/matmul.zig, ops/experts.zig, ops/rowwise.zig) ----
    int embed(const Buffer &weights, const Matrix &matrix, uint32_t token, const Buffer &output, uint32_t out_dtype);
    int matvec(const Buffer &weights, const Matrix &matrix, const Buffer &input, const Buffer &output);
    int matvecRows(const Buffer &weights, const Matrix &matrix, const Buffer &input, size_t in_stride,
                   const Buffer &output, size_t out_stride, size_t tokens);
    int matmul(const Buffer &weights, const Matrix &matrix, const Buffer &input, uint32_t in_dtype, size_t in_stride,
               const Buffer &output, size_t out_stride, size_t tokens);
    int matvecAdd(const Buffer &weights, const Matrix &m, const Buffer &input, const Buffer &residual, const Buffer &output);
    int matvecSegments(const Segment *segments, size_t count, const Buffer &input, uint32_t mode) { return segmentsJob(segments, count, input, mode, nullptr); }
    int matvecSegmentsNormed(const Segment *segments, size_t count, const Buffer &residual, const Buffer *input, const Buffer &weight, const Buffer *residual_out,
                             float eps, uint32_t mode);
    int actMul(uint32_t act, const Buffer &gate, const Buffer &up, size_t count);
    int rmsNorm(const Buffer &input, const Buffer &weight, const Buffer &output, const nu_norm &spec);
    int addRmsNorm(const Buffer &residual, const Buffer &input, const Buffer &weight, const Buffer &output, const nu_norm &spec);
    int add(const Buffer &x, const Buffer &y, size_t count);
    int argmax(const Buffer &logits, size_t count, const Buffer &result);
    int route(const Buffer &logits, size_t experts, size_t k, size_t rows, size_t in_stride, const Buffer &indices, const Buffer &weights);
    int routeLocal(const Buffer &indices, const Buffer &weights, size_t count, size_t first, size_t local, const Buffer &local_indices, const Buffer &local_weights);
    int matvecExpertsGrouped(const Buffer &weights, const ExpertMatrix &tensor, const Buffer &indices, size_t slots,
                             const Buffer &input, size_t in_stride, size_t in_group, const Buffer &output, size_t out_stride);
    int expertLists(const Buffer &indices, size_t rows, size_t k, size_t experts, const Buffer &lists);
    int matmulExperts(const Buffer &weights, const ExpertMatrix &tensor, const Buffer &lists, size_t rows, size_t k, const Buffer &input, size_t in_stride,
                      size_t in_group, const Buffer &output, size_t out_stride);
    int matvecExpertsGated(const Buffer &weights, const ExpertMatrix &t, const Buffer &indices, size_t slots, const Buffer &input, size_t in_stride, size_t in_group,
                           const Buffer &output, size_t out_stride, uint32_t act);
    int geluMulRows(const Buffer &gate, const Buffer &up, const Buffer &output, size_t width, size_t rows,
                    size_t gate_stride, size_t up_stride, size_t out_stride);
    int combineExperts(const Buffer &values, const Buffer &weights, const Buffer &indices, const Buffer *scales,
                       const Buffer &output, const nu_combine_shape &shape);

    // ---- collective ----
    int commInit(const uint8_t *id, int ranks, int rank);
    int allreduceSumF32(const Buffer &buffer, size_t count, const Buffer *add_to = nullptr);
    int commDestroy();
    int peerHandle(uint8_t *out);
    int attachPeers(const uint8_t *handles, int ranks, int rank);
    int setPeerWaitMs(uint32_t ms);

    const char *lastError() const { return error_.c_str(); }

    static size_t matmulPadded(size_t tokens) { return (tokens + 63) / 64 * 64; }

private:
    Backend() = default;
    struct Allocation {
        uint8_t *ptr = nullptr;
        size_t len = 0;
        bool wrapped = false;
    };
    int fail(int status, const char *what);
    int cuda(cudaError_t e, const char *what, int status = NU_ERR_EXECUTION);
    // Device address of a view after checking that `need` bytes fit in it and in its buffer.
    uint8_t *resolve(const Buffer &b, size_t need);
    static bool overlaps(const Buffer &a, size_t a_len, const Buffer &b, size_t b_len);
    int needRecording(bool keep_chain = false);
    void opBoundary();
    void wrote(const Buffer &b);
    bool written(const Buffer &b) const;
    int finishCapture(cudaGraphExec_t *exec);
    int runGraph(cudaGraphExec_t exec, uint32_t count, float *elapsed_ms);
    int checkKernelStatus();
    int flushPending();

    int device_ = 0;
    int sm_count_ = 0;
    cudaStream_t stream_ = nullptr;
    cudaEvent_t ev_start_ = nullptr, ev_stop_ = nullptr;
    std::vector<Allocation> buffers_;  // index = id; ids are never reused
    std::unordered_map<uintptr_t, std::pair<uint32_t, size_t>> wrapped_;
    std::unordered_map<uint32_t, cudaGraphExec_t> graphs_;
    uint32_t next_graph_ = 1;
    uint64_t created_bytes_ = 0;
    bool recording_ = false;
    std::vector<uint32_t> written_;  // ids of buffers written in the open recording
    double gpu_seconds_ = 0;
    uint64_t launches_ = 0;
    std::string error_;
    // scratch of the split-K kernels: partial sums, arrival counters and a status word
    float *partials_ = nullptr;
    size_t partials_floats_ = 0;
    uint32_t *counters_ = nullptr;
    float *argmax_records_ = nullptr;  // 128 x (value, index, non-finite) of the argmax blocks, then their arrival counter
    size_t counters_len_ = 0;
    // per-operator profile
    bool profiling_ = false;
    uint32_t profile_max_ = 0;
    std::vector<cudaEvent_t> profile_events_;
    uint32_t profile_ops_ = 0;
    std::vector<double> profile_last_;
    // collective
    void *comm_ = nullptr;  // ncclComm_t
    int ranks_ = 1, rank_ = 0;
    // one-shot allreduce over peer memory: this rank's inbox (floats, then flags, then sequence numbers)
    uint8_t *inbox_ = nullptr;
    void *peer_base_[8] = {};
    bool peers_attached_ = false;
    // a one-token plain matvec held back for one operator: if an allreduce of its output follows, the two are fused
    bool pending_ = false;
    FastJobBox *pending_job_ = nullptr;
    Buffer pending_out_{};
    int peer_ranks_ = 0, peer_rank_ = 0;
    // one-token integer-path matvecs recorded back to back, held until another operator (or the commit) ends the
    // run: two or more of them become one persistent launch (gemv_chain.cu)
    FastChain *chain_ = nullptr;
    int flushChain();
    int chainOrLaunch(const FastJob &job);
    // The add + RMS norm a merged launch folds into its staging pass: device pointers, resolved and checked.
    struct NormFuse {
        const float *weight, *input;
        float *residual_out;
        float eps;
        const Buffer *out_buffer;  // what residual_out belongs to (marked written), or null
    };
    int segmentsJob(const Segment *segments, size_t count, const Buffer &input, uint32_t mode, const NormFuse *norm);
    unsigned long long peer_wait_ns_ = 2000000000ull;
};

}  // namespace nu
