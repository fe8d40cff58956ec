// Backend: buffers, recording (CUDA graph capture) and the shape validation and
// kernel selection of every operator. The validation of each operator restates
// the checks of the reference's encoder for it, in the same order, so that the
// same bad call draws the same error before anything is recorded.
#include "backend.hpp"

#include <dlfcn.h>

#include <cstdio>
#include <cstring>

#include "kernels.hpp"
#include "nu_device.cuh"

namespace nu {

struct FastJobBox { FastJob job; };
struct FastChain { std::vector<FastJob> jobs; };

namespace {

constexpr size_t kPad = 256;                       // slack after every allocation: bulk copies may read up to 15 bytes past a row
constexpr size_t kPartialsFloats = 64u << 20;      // 256 MiB of scratch: split-K partial sums, the bf16 staging of F32 prefill activations,
                                                   // the gathered rows of the grouped (expert) prefill
constexpr size_t kCounters = 1u << 16;             // row-block arrival counters
constexpr size_t kPushCapacity = 8 * 8192;         // floats per inbox slot: 8 token rows of up to 8192 values
constexpr size_t kPushWordBytes = 2 * PUSH_MAX_RANKS * kPushCapacity * 8;   // (value, tag) words
constexpr size_t kPushBytes = kPushWordBytes + 64;                          // then sequence number, finished blocks, sticky failure

// quant.validateRow, inference/src/quant/decode.zig:108-120.
int validateRow(uint32_t enc, size_t byte_count, size_t element_count) {
    const Layout l = layout(enc);
    if (l.elements == 0) return NU_ERR_UNSUPPORTED_ENCODING;
    if (element_count == 0 || element_count % l.elements != 0) return NU_ERR_INVALID_ROW_LENGTH;
    if (byte_count % l.bytes != 0 || byte_count / l.bytes != element_count / l.elements) return NU_ERR_INVALID_BYTE_LENGTH;
    return NU_OK;
}

bool fits_u32(uint64_t v) { return v <= 0xffffffffull; }

// A matrix is in GGUF form (0) or in the form prepare gave it; anything else is a caller error.
bool layoutOk(const nu_matrix &m) {
    return m.layout == 0 || (fits_u32(m.rows) && fits_u32(m.columns) && m.layout == prepared_layout(m.encoding, (uint32_t)m.rows, (uint32_t)m.columns));
}

}  // namespace

// ---- lifecycle -------------------------------------------------------------------------

Backend *Backend::create(int device, std::string &error) {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || device < 0 || device >= count) {
        error = e != cudaSuccess ? std::string("no CUDA device: ") + cudaGetErrorString(e) : "device index out of range";
        return nullptr;
    }
    Backend *b = new Backend();
    b->device_ = device;
    bool ok = cudaSetDevice(device) == cudaSuccess;
    cudaDeviceProp prop{};
    ok = ok && cudaGetDeviceProperties(&prop, device) == cudaSuccess;
    if (ok && prop.major != 10) {
        error = "this library is built for sm_100a (B200) only; found compute capability " + std::to_string(prop.major) + "." + std::to_string(prop.minor);
        delete b;
        return nullptr;
    }
    b->sm_count_ = prop.multiProcessorCount;
    ok = ok && cudaStreamCreateWithFlags(&b->stream_, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaEventCreate(&b->ev_start_) == cudaSuccess && cudaEventCreate(&b->ev_stop_) == cudaSuccess;
    ok = ok && cudaMalloc(&b->partials_, kPartialsFloats * sizeof(float)) == cudaSuccess;
    ok = ok && cudaMalloc(&b->counters_, (kCounters + 3) * sizeof(uint32_t)) == cudaSuccess;
    ok = ok && cudaMemset(b->counters_, 0, (kCounters + 3) * sizeof(uint32_t)) == cudaSuccess;
    ok = ok && cudaMalloc(&b->argmax_records_, (128 * 4 + 4) * sizeof(float)) == cudaSuccess;
    ok = ok && cudaMemset(b->argmax_records_, 0, (128 * 4 + 4) * sizeof(float)) == cudaSuccess;
    if (!ok) {
        error = std::string("CUDA set-up failed: ") + cudaGetErrorString(cudaGetLastError());
        delete b;
        return nullptr;
    }
    if (!fast_configure()) {
        error = std::string("kernel set-up failed: ") + cudaGetErrorString(cudaGetLastError());
        delete b;
        return nullptr;
    }
    b->partials_floats_ = kPartialsFloats;
    b->counters_len_ = kCounters;
    b->buffers_.push_back({});  // id 0 is never handed out
    return b;
}

Backend::~Backend() {
    cudaSetDevice(device_);
    if (recording_) discard();
    if (stream_) cudaStreamSynchronize(stream_);
    commDestroy();
    for (auto &g : graphs_) cudaGraphExecDestroy(g.second);
    for (auto &a : buffers_) if (a.ptr) cudaFree(a.ptr);
    for (auto &ev : profile_events_) cudaEventDestroy(ev);
    delete pending_job_;
    delete chain_;
    if (inbox_) cudaFree(inbox_);
    if (partials_) cudaFree(partials_);
    if (counters_) cudaFree(counters_);
    if (argmax_records_) cudaFree(argmax_records_);
    if (ev_start_) cudaEventDestroy(ev_start_);
    if (ev_stop_) cudaEventDestroy(ev_stop_);
    if (stream_) cudaStreamDestroy(stream_);
}

int Backend::fail(int status, const char *what) {
    error_ = what;
    return status;
}

int Backend::cuda(cudaError_t e, const char *what, int status) {
    if (e == cudaSuccess) return NU_OK;
    error_ = std::string(what) + ": " + cudaGetErrorString(e);
    return status;
}

// ---- buffers ----------------------------------------------------------------------------

int Backend::createBuffer(size_t len, uint32_t *id) {
    if (len == 0 || !id) return fail(NU_ERR_INVALID_SHAPE, "create: empty buffer");
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "create: a recording is open");
    cudaSetDevice(device_);
    Allocation a;
    if (int rc = cuda(cudaMalloc(&a.ptr, len + kPad), "create: cudaMalloc", NU_ERR_BUFFER)) return rc;
    if (int rc = cuda(cudaMemsetAsync(a.ptr, 0, len + kPad, stream_), "create: memset", NU_ERR_BUFFER)) { cudaFree(a.ptr); return rc; }
    cudaStreamSynchronize(stream_);
    a.len = len;
    buffers_.push_back(a);
    created_bytes_ += len;
    *id = (uint32_t)(buffers_.size() - 1);
    return NU_OK;
}

int Backend::upload(uint32_t id, size_t offset, const void *src, size_t len) {
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "upload: a recording is open");
    if (id == 0 || id >= buffers_.size() || !buffers_[id].ptr) return fail(NU_ERR_BUFFER, "upload: unknown buffer");
    if (offset > buffers_[id].len || len > buffers_[id].len - offset || (!src && len)) return fail(NU_ERR_INVALID_SHAPE, "upload: range outside the buffer");
    cudaSetDevice(device_);
    if (int rc = cuda(cudaMemcpyAsync(buffers_[id].ptr + offset, src, len, cudaMemcpyHostToDevice, stream_), "upload")) return rc;
    return cuda(cudaStreamSynchronize(stream_), "upload: sync");
}

int Backend::download(uint32_t id, size_t offset, void *dst, size_t len) {
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "download: a recording is open");
    if (id == 0 || id >= buffers_.size() || !buffers_[id].ptr) return fail(NU_ERR_BUFFER, "download: unknown buffer");
    if (offset > buffers_[id].len || len > buffers_[id].len - offset || (!dst && len)) return fail(NU_ERR_INVALID_SHAPE, "download: range outside the buffer");
    cudaSetDevice(device_);
    if (int rc = cuda(cudaMemcpyAsync(dst, buffers_[id].ptr + offset, len, cudaMemcpyDeviceToHost, stream_), "download")) return rc;
    return cuda(cudaStreamSynchronize(stream_), "download: sync");
}

int Backend::wrap(const void *bytes, size_t len, uint32_t *id) {
    if (!bytes || len == 0 || !id) return fail(NU_ERR_INVALID_SHAPE, "wrap: empty range");
    auto it = wrapped_.find((uintptr_t)bytes);
    if (it != wrapped_.end()) {
        if (it->second.second != len) return fail(NU_ERR_INVALID_SHAPE, "wrap: same address wrapped at another length");
        *id = it->second.first;
        return NU_OK;
    }
    uint32_t fresh = 0;
    if (int rc = createBuffer(len, &fresh)) return rc;
    created_bytes_ -= len;  // wrapped ranges are accounted apart from created ones
    buffers_[fresh].wrapped = true;
    if (int rc = upload(fresh, 0, bytes, len)) { release(fresh); return rc; }
    wrapped_[(uintptr_t)bytes] = {fresh, len};
    *id = fresh;
    return NU_OK;
}

int Backend::unwrap(const void *bytes) {
    auto it = wrapped_.find((uintptr_t)bytes);
    if (it == wrapped_.end()) return NU_OK;
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "unwrap: a recording is open");
    const uint32_t id = it->second.first;
    wrapped_.erase(it);
    cudaFree(buffers_[id].ptr);
    buffers_[id] = {};
    return NU_OK;
}

int Backend::release(uint32_t id) {
    if (recording_) return fail(NU_ERR_INVALID_SHAPE, "release: a recording is open");
    if (id == 0 || id >= buffers_.size() || !buffers_[id].ptr) return fail(NU_ERR_BUFFER, "release: unknown buffer");
    cudaSetDevice(device_);
    cudaStreamSynchronize(stream_);
    cudaFree(buffers_[id].ptr);
    if (!buffers_[id].wrapped) created_bytes_ -= buffers_[id].len;
    else for (auto it = wrapped_.begin(); it != wrapped_.end(); ++it) if (it->second.first == id) { wrapped_.erase(it); break; }
    buffers_[id] = {};  // the id is never reused: a stale view fails instead of aliasing
    return NU_OK;
}

void *Backend::devicePtr(uint32_t id) {
    if (id == 0 || id >= buffers_.size()) return nullptr;
    return buffers_[id].ptr;
}

uint8_t *Backend::resolve(const Buffer &b, size_t need) {
    if (b.id == 0 || b.id >= buffers_.size() || !buffers_[b.id].ptr) return nullptr;
    const Allocation &a = buffers_[b.id];
    if (b.offset > a.len || b.len > a.len - b.offset || need > b.len) return nullptr;
    return a.ptr + b.offset;
}

bool Backend::overlaps(const Buffer &a, size_t a_len, const Buffer &b, size_t b_len) {
    if (a.id != b.id) return false;
    return a.offset <= b.offset ? b.offset - a.offset < a_len : a.offset - b.offset < b_len;
}

// No reference analogue: see nu_cuda_matrix_prepare in the header and prepare.cu.
int Backend::prepare(const Buffer &weights, const Matrix &m, const Buffer &prepared, uint32_t *layout_out) {
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "prepare: a recording is open");
    if (!layout_out || m.rows == 0 || m.columns == 0 || m.bytes % m.rows != 0 || m.layout != 0) return fail(NU_ERR_INVALID_SHAPE, "prepare: shape");
    if (int rc = validateRow(m.encoding, m.bytes / m.rows, m.columns)) return fail(rc, "prepare: row layout");
    if (!fits_u32(m.rows) || !fits_u32(m.columns)) return fail(NU_ERR_INVALID_SHAPE, "prepare: too large");
    const uint8_t *src = resolve(weights, m.bytes);
    uint8_t *dst = resolve(prepared, m.bytes);
    if (!src || !dst || overlaps(weights, m.bytes, prepared, m.bytes)) return fail(NU_ERR_INVALID_SHAPE, "prepare: buffers too short or overlapping");
    cudaSetDevice(device_);
    launches_ += launch_prepare(stream_, m.encoding, src, dst, (uint32_t)m.rows, (uint32_t)m.columns);
    if (int rc = cuda(cudaGetLastError(), "prepare: launch")) return rc;
    if (int rc = cuda(cudaStreamSynchronize(stream_), "prepare: wait")) return rc;
    *layout_out = prepared_layout(m.encoding, (uint32_t)m.rows, (uint32_t)m.columns);
    return NU_OK;
}

// ---- recording ----------------------------------------------------------------------------

int Backend::begin() {
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "begin: a recording is already open");
    cudaSetDevice(device_);
    if (profiling_) {
        profile_ops_ = 0;
        if (int rc = cuda(cudaEventRecord(profile_events_[0], stream_), "begin: event")) return rc;
    } else {
        if (int rc = cuda(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal), "begin: capture")) return rc;
    }
    recording_ = true;
    written_.clear();
    return NU_OK;
}

int Backend::needRecording(bool keep_chain) {
    if (!recording_) return fail(NU_ERR_NOT_RECORDING, "no recording is open (call begin first)");
    cudaSetDevice(device_);
    if (!keep_chain)
        if (int rc = flushChain()) return rc;  // every operator but another link ends a run of chained matvecs
    return flushPending();  // every operator but the allreduce that may fuse with it launches a held-back matvec first
}

// A one-token job on the specialized kernels: held as a link of the open chain if it can be one, else launched now.
int Backend::chainOrLaunch(const FastJob &job) {
    if (!chain_) chain_ = new FastChain;
    if (chaining && !profiling_ && !peers_attached_ && chain_supported(job)) {
        if (chain_->jobs.size() == (size_t)kChainMax)
            if (int rc = flushChain()) return rc;
        chain_->jobs.push_back(job);
        return NU_OK;
    }
    if (int rc = flushChain()) return rc;
    launches_ += launch_fast(stream_, job);
    return NU_OK;
}

// Launches the held run: one job as its own kernel, two or more as one persistent kernel.
int Backend::flushChain() {
    if (!chain_ || chain_->jobs.empty()) return NU_OK;
    std::vector<FastJob> &jobs = chain_->jobs;
    int launched = 0;
    if (jobs.size() >= 2) launched = launch_chain(stream_, jobs.data(), (uint32_t)jobs.size(), counters_ + counters_len_ + 1, sm_count_);
    if (launched) {
        launches_ += launched;
    } else {
        for (const FastJob &job : jobs) launches_ += launch_fast(stream_, job);
    }
    jobs.clear();
    return cuda(cudaGetLastError(), "matvec chain: launch");
}

// Launches the matvec that was held back to see whether an allreduce of its output follows.
int Backend::flushPending() {
    if (!pending_) return NU_OK;
    pending_ = false;
    launches_ += launch_fast(stream_, pending_job_->job);
    opBoundary();
    return cuda(cudaGetLastError(), "matvec: launch");
}

// Buffers an operator of the open recording has written. A decode kernel starts reading its
// weights before the kernel ahead of it has ended; that is only safe for weights nothing in the
// recording wrote (the normal case: weights are constants uploaded before the recording).
void Backend::wrote(const Buffer &b) {
    for (uint32_t id : written_) if (id == b.id) return;
    written_.push_back(b.id);
}
bool Backend::written(const Buffer &b) const {
    for (uint32_t id : written_) if (id == b.id) return true;
    return false;
}

// Called after each operator has enqueued its kernels.
void Backend::opBoundary() {
    if (profiling_ && profile_ops_ < profile_max_) {
        ++profile_ops_;
        cudaEventRecord(profile_events_[profile_ops_], stream_);
    }
}

int Backend::finishCapture(cudaGraphExec_t *exec) {
    cudaGraph_t graph = nullptr;
    recording_ = false;
    if (int rc = cuda(cudaStreamEndCapture(stream_, &graph), "commit: end capture")) return rc;
    if (!graph) return fail(NU_ERR_EXECUTION, "commit: the capture was invalidated");
    cudaError_t e = cudaGraphInstantiate(exec, graph, 0);
    cudaGraphDestroy(graph);
    return cuda(e, "commit: instantiate");
}

int Backend::checkKernelStatus() {
    uint32_t status = 0;
    if (int rc = cuda(cudaMemcpyAsync(&status, counters_ + counters_len_, sizeof status, cudaMemcpyDeviceToHost, stream_), "status read")) return rc;
    if (int rc = cuda(cudaStreamSynchronize(stream_), "status sync")) return rc;
    if (status != 0) {
        cudaMemsetAsync(counters_, 0, (counters_len_ + 3) * sizeof(uint32_t), stream_);  // counters, status word, the chain kernel's two arrival counts
        cudaStreamSynchronize(stream_);
        return fail(NU_ERR_EXECUTION, status == 2 ? "allreduce over peer memory: a rank never arrived (bounded wait ran out); the path stays closed" : "a kernel gave up a bounded wait (copy never completed)");
    }
    return NU_OK;
}

int Backend::runGraph(cudaGraphExec_t exec, uint32_t count, float *elapsed_ms) {
    if (int rc = cuda(cudaEventRecord(ev_start_, stream_), "launch: event")) return rc;
    for (uint32_t i = 0; i < count; ++i)
        if (int rc = cuda(cudaGraphLaunch(exec, stream_), "launch")) return rc;
    if (int rc = cuda(cudaEventRecord(ev_stop_, stream_), "launch: event")) return rc;
    if (int rc = cuda(cudaStreamSynchronize(stream_), "launch: wait")) return rc;
    float ms = 0;
    cudaEventElapsedTime(&ms, ev_start_, ev_stop_);
    gpu_seconds_ += ms * 1e-3;
    if (elapsed_ms) *elapsed_ms = ms;
    return checkKernelStatus();
}

int Backend::commit() {
    if (!recording_) return fail(NU_ERR_NOT_RECORDING, "commit: no recording is open");
    cudaSetDevice(device_);
    if (int rc = flushChain()) return rc;
    if (int rc = flushPending()) return rc;
    if (profiling_) {
        recording_ = false;
        if (int rc = cuda(cudaStreamSynchronize(stream_), "commit: wait")) return rc;
        profile_last_.assign(profile_ops_, 0.0);
        for (uint32_t i = 0; i < profile_ops_; ++i) {
            float ms = 0;
            cudaEventElapsedTime(&ms, profile_events_[i], profile_events_[i + 1]);
            profile_last_[i] = ms * 1e-3;
            gpu_seconds_ += ms * 1e-3;
        }
        return checkKernelStatus();
    }
    cudaGraphExec_t exec = nullptr;
    if (int rc = finishCapture(&exec)) return rc;
    const int rc = runGraph(exec, 1, nullptr);
    cudaGraphExecDestroy(exec);
    return rc;
}

int Backend::commitRetain(uint32_t *graph) {
    if (!graph) return fail(NU_ERR_INVALID_SHAPE, "commit_retain: null result");
    if (!recording_) return fail(NU_ERR_NOT_RECORDING, "commit_retain: no recording is open");
    if (profiling_) return fail(NU_ERR_INVALID_SHAPE, "commit_retain: not available while profiling");
    cudaSetDevice(device_);
    if (int rc = flushChain()) return rc;
    if (int rc = flushPending()) return rc;
    cudaGraphExec_t exec = nullptr;
    if (int rc = finishCapture(&exec)) return rc;
    if (int rc = runGraph(exec, 1, nullptr)) { cudaGraphExecDestroy(exec); return rc; }
    *graph = next_graph_++;
    graphs_[*graph] = exec;
    return NU_OK;
}

int Backend::graphLaunch(uint32_t graph, uint32_t count, float *elapsed_ms) {
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "graph_launch: a recording is open");
    auto it = graphs_.find(graph);
    if (it == graphs_.end() || count == 0) return fail(NU_ERR_INVALID_SHAPE, "graph_launch: unknown graph or zero count");
    cudaSetDevice(device_);
    return runGraph(it->second, count, elapsed_ms);
}

int Backend::graphRelease(uint32_t graph) {
    auto it = graphs_.find(graph);
    if (it == graphs_.end()) return fail(NU_ERR_INVALID_SHAPE, "graph_release: unknown graph");
    cudaGraphExecDestroy(it->second);
    graphs_.erase(it);
    return NU_OK;
}

int Backend::discard() {
    if (!recording_) return NU_OK;
    cudaSetDevice(device_);
    recording_ = false;
    pending_ = false;
    if (chain_) chain_->jobs.clear();
    if (profiling_) {
        // Profiling runs operators as they are recorded; there is nothing left to drop.
        cudaStreamSynchronize(stream_);
        return NU_OK;
    }
    cudaGraph_t graph = nullptr;
    cudaStreamEndCapture(stream_, &graph);
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    return NU_OK;
}

int Backend::profileEnable(uint32_t max_ops) {
    if (recording_ || profiling_ || max_ops == 0) return fail(NU_ERR_ALREADY_RECORDING, "profile_enable: once, while idle, with a positive capacity");
    cudaSetDevice(device_);
    profile_events_.resize((size_t)max_ops + 1);
    for (auto &ev : profile_events_)
        if (int rc = cuda(cudaEventCreate(&ev), "profile_enable: event")) return rc;
    profile_max_ = max_ops;
    profiling_ = true;
    return NU_OK;
}

uint32_t Backend::profileRead(double *seconds, uint32_t cap) {
    const uint32_t n = (uint32_t)profile_last_.size();
    for (uint32_t i = 0; i < n && i < cap && seconds; ++i) seconds[i] = profile_last_[i];
    return n;
}

// ---- operators -------------------------------------------------------------------------------

// ops/rowwise.zig:17-25.
int Backend::embed(const Buffer &weights, const Matrix &m, uint32_t token, const Buffer &output, uint32_t out_dtype) {
    if (m.rows == 0 || m.columns == 0 || m.columns % 16 != 0 || m.bytes % m.rows != 0 || token >= m.rows) return fail(NU_ERR_INVALID_SHAPE, "embed: shape");
    const size_t stride = m.bytes / m.rows;
    if (int rc = validateRow(m.encoding, stride, m.columns)) return fail(rc, "embed: row layout");
    if (out_dtype != NU_F32 && out_dtype != NU_BF16) return fail(NU_ERR_INVALID_SHAPE, "embed: output type");
    if (!layoutOk(m)) return fail(NU_ERR_INVALID_SHAPE, "embed: unknown matrix layout");
    if (!fits_u32(m.columns)) return fail(NU_ERR_INVALID_SHAPE, "embed: columns");
    const size_t out_bytes = m.columns * (out_dtype == NU_F32 ? 4 : 2);
    const uint8_t *w = resolve(weights, m.bytes);
    uint8_t *out = resolve(output, out_bytes);
    if (!w || !out || output.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "embed: buffer too short");
    if (int rc = needRecording()) return rc;
    launches_ += launch_dequant_row(stream_, m.encoding, m.layout, w, stride, (uint32_t)m.rows, token, (uint32_t)m.columns, out, out_dtype == NU_BF16);
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "embed: launch");
}

// ops/matvec.zig:85-116.
int Backend::matvec(const Buffer &weights, const Matrix &m, const Buffer &input, const Buffer &output) {
    if (m.rows == 0 || m.columns == 0 || m.columns % 16 != 0 || m.bytes % m.rows != 0) return fail(NU_ERR_INVALID_SHAPE, "matvec: shape");
    const size_t stride = m.bytes / m.rows;
    if (int rc = validateRow(m.encoding, stride, m.columns)) return fail(rc, "matvec: row layout");
    if (!fits_u32(m.rows) || !fits_u32(m.columns)) return fail(NU_ERR_INVALID_SHAPE, "matvec: too large");
    if (!layoutOk(m)) return fail(NU_ERR_INVALID_SHAPE, "matvec: unknown matrix layout");
    const uint8_t *w = resolve(weights, m.bytes);
    const float *in = (const float *)resolve(input, m.columns * 4);
    float *out = (float *)resolve(output, m.rows * 4);
    if (!w || !in || !out || input.offset % 4 != 0 || output.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "matvec: buffer too short");
    if (int rc = needRecording(true)) return rc;
    FastJob job{};
    job.enc = m.encoding; job.layout = m.layout; job.columns = (uint32_t)m.columns; job.tokens = 1; job.in = in; job.in_stride = m.columns;
    job.count = 1; job.mode = ACT_NONE;
    job.seg[0] = {w, stride, (uint32_t)m.rows, out, m.rows};
    job.serial = written(weights); job.partials = partials_; job.partials_floats = partials_floats_; job.counters = counters_; job.counters_len = counters_len_; job.sm_count = sm_count_;
    if (!generic_only && fast_supported(job)) {
        if (peers_attached_ && !profiling_ && m.rows <= kPushCapacity) {
            // held back: an allreduce of this output may follow and fuse with it (allreduceSumF32)
            if (!pending_job_) pending_job_ = new FastJobBox;
            pending_job_->job = job;
            pending_out_ = output;
            pending_ = true;
            wrote(output);
            return NU_OK;
        }
        if (int rc = chainOrLaunch(job)) return rc;
    } else {
        if (int rc = flushChain()) return rc;
        launches_ += launch_matmul_generic(stream_, m.encoding, m.layout, w, stride, (uint32_t)m.rows, (uint32_t)m.columns, in, false, m.columns, out, m.rows, 1);
    }
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "matvec: launch");
}

// No reference analogue as one call: `matvec` followed by the residual `add` of its output
// (ops/matvec.zig:85-116, ops/rowwise.zig:199-202; inference/src/models/qwen35_metal.zig:640): output = residual + W x,
// the add folded into the kernel's write. `output` may be `residual` itself. Matrices the specialized kernel does not
// serve take the generic matvec and the add as two launches: the call never declines.
int Backend::matvecAdd(const Buffer &weights, const Matrix &m, const Buffer &input, const Buffer &residual, const Buffer &output) {
    if (m.rows == 0 || m.columns == 0 || m.columns % 16 != 0 || m.bytes % m.rows != 0) return fail(NU_ERR_INVALID_SHAPE, "matvec_add: shape");
    const size_t stride = m.bytes / m.rows;
    if (int rc = validateRow(m.encoding, stride, m.columns)) return fail(rc, "matvec_add: row layout");
    if (!fits_u32(m.rows) || !fits_u32(m.columns)) return fail(NU_ERR_INVALID_SHAPE, "matvec_add: too large");
    if (!layoutOk(m)) return fail(NU_ERR_INVALID_SHAPE, "matvec_add: unknown matrix layout");
    const uint8_t *w = resolve(weights, m.bytes);
    const float *in = (const float *)resolve(input, m.columns * 4);
    const float *res = (const float *)resolve(residual, m.rows * 4);
    float *out = (float *)resolve(output, m.rows * 4);
    if (!w || !in || !res || !out || input.offset % 4 != 0 || output.offset % 4 != 0 || residual.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "matvec_add: buffer too short");
    const bool same = residual.id == output.id && residual.offset == output.offset;
    if (!same && overlaps(residual, m.rows * 4, output, m.rows * 4)) return fail(NU_ERR_INVALID_SHAPE, "matvec_add: output overlaps the residual");
    if (overlaps(output, m.rows * 4, input, m.columns * 4) || overlaps(output, m.rows * 4, weights, m.bytes)) return fail(NU_ERR_INVALID_SHAPE, "matvec_add: output overlaps an input");
    if (int rc = needRecording(true)) return rc;
    FastJob job{};
    job.enc = m.encoding; job.layout = m.layout; job.columns = (uint32_t)m.columns; job.tokens = 1; job.in = in; job.in_stride = m.columns;
    job.count = 1; job.mode = ACT_NONE;
    job.seg[0] = {w, stride, (uint32_t)m.rows, out, m.rows};
    job.add0 = res;
    job.serial = written(weights); job.partials = partials_; job.partials_floats = partials_floats_; job.counters = counters_; job.counters_len = counters_len_; job.sm_count = sm_count_;
    if (!generic_only && fast_supported(job)) {
        if (int rc = chainOrLaunch(job)) return rc;
    } else {
        if (int rc = flushChain()) return rc;
        // the products go to the handle's scratch (the generic kernel does not use it), then one pass adds them
        if (m.rows > partials_floats_) return fail(NU_ERR_TOO_LARGE, "matvec_add: rows beyond the scratch");
        launches_ += launch_matmul_generic(stream_, m.encoding, m.layout, w, stride, (uint32_t)m.rows, (uint32_t)m.columns, in, false, m.columns, partials_, m.rows, 1);
        if (!same && cudaMemcpyAsync(out, res, m.rows * 4, cudaMemcpyDeviceToDevice, stream_) != cudaSuccess) return fail(NU_ERR_EXECUTION, "matvec_add: copy");
        launches_ += launch_add(stream_, out, partials_, m.rows);
    }
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "matvec_add: launch");
}

// ops/matvec.zig:149-165.
int Backend::matvecRows(const Buffer &weights, const Matrix &m, const Buffer &input, size_t in_stride,
                        const Buffer &output, size_t out_stride, size_t tokens) {
    if (m.rows == 0 || m.columns == 0 || m.columns % 16 != 0 || m.bytes % m.rows != 0) return fail(NU_ERR_INVALID_SHAPE, "matvec_rows: shape");
    const size_t stride = m.bytes / m.rows;
    if (int rc = validateRow(m.encoding, stride, m.columns)) return fail(rc, "matvec_rows: row layout");
    if (tokens < 2 || tokens > 8) return fail(NU_ERR_INVALID_SHAPE, "matvec_rows: 2..8 tokens");
    if (in_stride < m.columns || out_stride < m.rows) return fail(NU_ERR_INVALID_SHAPE, "matvec_rows: strides");
    if (!fits_u32(m.rows) || !fits_u32(m.columns)) return fail(NU_ERR_INVALID_SHAPE, "matvec_rows: too large");
    if (!layoutOk(m)) return fail(NU_ERR_INVALID_SHAPE, "matvec_rows: unknown matrix layout");
    const uint8_t *w = resolve(weights, m.bytes);
    const float *in = (const float *)resolve(input, ((tokens - 1) * in_stride + m.columns) * 4);
    float *out = (float *)resolve(output, ((tokens - 1) * out_stride + m.rows) * 4);
    if (!w || !in || !out) return fail(NU_ERR_INVALID_SHAPE, "matvec_rows: buffer too short");
    if (input.offset % 16 != 0 || in_stride % 4 != 0 || output.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "matvec_rows: alignment");
    if (int rc = needRecording()) return rc;
    FastJob job{};
    job.enc = m.encoding; job.layout = m.layout; job.columns = (uint32_t)m.columns; job.tokens = (uint32_t)tokens; job.in = in; job.in_stride = in_stride;
    job.count = 1; job.mode = ACT_NONE;
    job.seg[0] = {w, stride, (uint32_t)m.rows, out, out_stride};
    job.serial = written(weights); job.partials = partials_; job.partials_floats = partials_floats_; job.counters = counters_; job.counters_len = counters_len_; job.sm_count = sm_count_;
    if (!generic_only && fast_supported(job)) launches_ += launch_fast(stream_, job);
    else launches_ += launch_matmul_generic(stream_, m.encoding, m.layout, w, stride, (uint32_t)m.rows, (uint32_t)m.columns, in, false, in_stride, out, out_stride, (uint32_t)tokens);
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "matvec_rows: launch");
}

// ops/matmul.zig:76-108.
int Backend::matmul(const Buffer &weights, const Matrix &m, const Buffer &input, uint32_t in_dtype, size_t in_stride,
                    const Buffer &output, size_t out_stride, size_t tokens) {
    if (m.rows == 0 || m.rows % 8 != 0 || m.columns == 0 || m.columns % 64 != 0 || m.bytes % m.rows != 0) return fail(NU_ERR_INVALID_SHAPE, "matmul: shape");
    if (tokens == 0 || in_stride < m.columns || out_stride < m.rows) return fail(NU_ERR_INVALID_SHAPE, "matmul: tokens or strides");
    const size_t stride = m.bytes / m.rows;
    if (int rc = validateRow(m.encoding, stride, m.columns)) return fail(rc, "matmul: row layout");
    if (in_dtype != NU_F32 && in_dtype != NU_BF16) return fail(NU_ERR_INVALID_SHAPE, "matmul: input type");
    if (!fits_u32(m.rows) || !fits_u32(m.columns) || !fits_u32(tokens)) return fail(NU_ERR_INVALID_SHAPE, "matmul: too large");
    if (!layoutOk(m)) return fail(NU_ERR_INVALID_SHAPE, "matmul: unknown matrix layout");
    const size_t padded = matmulPadded(tokens);
    const size_t esize = in_dtype == NU_F32 ? 4 : 2;
    const uint8_t *w = resolve(weights, m.bytes);
    const uint8_t *in = resolve(input, padded * in_stride * esize);
    float *out = (float *)resolve(output, padded * out_stride * 4);
    if (!w || !in || !out) return fail(NU_ERR_INVALID_SHAPE, "matmul: buffer too short");
    if (input.offset % 16 != 0 || in_stride % 4 != 0 || output.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "matmul: alignment");
    if (int rc = needRecording()) return rc;
    bool done = false;
    if (!generic_only && in_dtype == NU_F32 && tokens <= 32) {
        // Up to 8 tokens in one pass of the weights; a few more in passes of 8.
        FastJob job{};
        job.enc = m.encoding; job.layout = m.layout; job.columns = (uint32_t)m.columns; job.count = 1; job.mode = ACT_NONE; job.in_stride = in_stride;
        job.serial = written(weights); job.partials = partials_; job.partials_floats = partials_floats_; job.counters = counters_; job.counters_len = counters_len_; job.sm_count = sm_count_;
        job.tokens = (uint32_t)(tokens < 8 ? tokens : 8);
        job.in = (const float *)in;
        job.seg[0] = {w, stride, (uint32_t)m.rows, out, out_stride};
        if (fast_supported(job)) {
            for (size_t t0 = 0; t0 < tokens; t0 += 8) {
                job.tokens = (uint32_t)(tokens - t0 < 8 ? tokens - t0 : 8);
                job.in = (const float *)in + t0 * in_stride;
                job.seg[0].out = out + t0 * out_stride;
                launches_ += launch_fast(stream_, job);
            }
            done = true;
        }
    }
    if (!done && !generic_only && tokens > 8) {
        // Many token rows: the tensor-core prefill tile. F32 activations are first rounded to BF16 into
        // the handle's scratch when they fit there (the reference's tiles round them to half the same way).
        PrefillJob pj{};
        pj.enc = m.encoding; pj.layout = m.layout; pj.w = w; pj.stride = stride; pj.rows = (uint32_t)m.rows; pj.columns = (uint32_t)m.columns;
        pj.tokens = (uint32_t)tokens; pj.padded_tokens = (uint32_t)padded; pj.out = out; pj.out_stride = out_stride;
        pj.status = counters_ + counters_len_; pj.sm_count = sm_count_;
        if (in_dtype == NU_BF16) {
            pj.in = in; pj.in_stride = in_stride;
        } else if (padded * m.columns * 2 <= partials_floats_ * sizeof(float)) {
            pj.in = partials_; pj.in_stride = m.columns;
        }
        if (pj.in && prefill_supported(pj)) {
            if (in_dtype != NU_BF16) launches_ += launch_f32_to_bf16_rows(stream_, (const float *)in, in_stride, partials_, m.columns, (uint32_t)m.columns, (uint32_t)tokens);
            launches_ += launch_prefill(stream_, pj);
            done = true;
        }
    }
    if (!done)
        launches_ += launch_matmul_generic(stream_, m.encoding, m.layout, w, stride, (uint32_t)m.rows, (uint32_t)m.columns, in, in_dtype == NU_BF16, in_stride, out, out_stride, (uint32_t)tokens);
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "matmul: launch");
}

// ops/matvec.zig:268-343.
int Backend::segmentsJob(const Segment *segments, size_t count, const Buffer &input, uint32_t mode, const NormFuse *norm) {
    if (!segments || count == 0 || count > 4) return fail(NU_ERR_INVALID_SHAPE, "segments: 1..4 segments");
    if (mode > NU_SEGMENTS_GELU_MUL_PAIR) return fail(NU_ERR_INVALID_SHAPE, "segments: mode");
    const size_t columns = segments[0].matrix.columns;
    if (columns == 0 || columns > 0xffffffffull / 4 || columns % 16 != 0 || input.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "segments: columns");
    const float *in = (const float *)resolve(input, columns * 4);
    if (!in) return fail(NU_ERR_INVALID_SHAPE, "segments: input too short");
    if (mode != NU_SEGMENTS_PLAIN && (count != 2 || segments[0].matrix.rows != segments[1].matrix.rows ||
                                      segments[0].output.id != segments[1].output.id || segments[0].output.offset != segments[1].output.offset))
        return fail(NU_ERR_INVALID_SHAPE, "segments: a pair needs two equal segments naming one output");
    FastJob job{};
    job.enc = segments[0].matrix.encoding; job.layout = segments[0].matrix.layout; job.columns = (uint32_t)columns; job.tokens = 1; job.in = in; job.in_stride = columns;
    job.count = (uint32_t)count; job.mode = mode == NU_SEGMENTS_PLAIN ? ACT_NONE : (mode == NU_SEGMENTS_SILU_MUL_PAIR ? ACT_SILU : ACT_GELU);
    for (size_t i = 0; i < count; ++i) job.serial = job.serial || written(segments[i].weights); job.partials = partials_; job.partials_floats = partials_floats_; job.counters = counters_; job.counters_len = counters_len_; job.sm_count = sm_count_;
    bool same_encoding = true;
    uint64_t total_rows = 0;
    for (size_t i = 0; i < count; ++i) {
        const Segment &s = segments[i];
        const Matrix &m = s.matrix;
        if (m.rows == 0 || m.rows > 0xffffffffull / 4 || m.rows % 16 != 0 || m.columns != columns || m.bytes % m.rows != 0) return fail(NU_ERR_INVALID_SHAPE, "segments: segment shape");
        const size_t stride = m.bytes / m.rows;
        if (int rc = validateRow(m.encoding, stride, columns)) return fail(rc, "segments: row layout");
        const uint8_t *w = resolve(s.weights, m.bytes);
        float *out = (float *)resolve(s.output, m.rows * 4);
        if (!w || !out || s.output.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "segments: buffer too short");
        if (overlaps(s.output, m.rows * 4, input, columns * 4)) return fail(NU_ERR_INVALID_SHAPE, "segments: output overlaps input");
        for (size_t j = 0; j < count; ++j)
            if (overlaps(s.output, m.rows * 4, segments[j].weights, segments[j].matrix.bytes)) return fail(NU_ERR_INVALID_SHAPE, "segments: output overlaps weights");
        if (mode == NU_SEGMENTS_PLAIN)
            for (size_t j = 0; j < i; ++j)
                if (overlaps(s.output, m.rows * 4, segments[j].output, segments[j].matrix.rows * 4)) return fail(NU_ERR_INVALID_SHAPE, "segments: outputs overlap");
        total_rows += m.rows;
        if (total_rows > 0xffffffffull) return fail(NU_ERR_INVALID_SHAPE, "segments: too many rows");
        if (!layoutOk(m)) return fail(NU_ERR_INVALID_SHAPE, "segments: unknown matrix layout");
        same_encoding = same_encoding && m.encoding == job.enc && m.layout == job.layout;
        job.seg[i] = {w, stride, (uint32_t)m.rows, out, m.rows};
    }
    // One launch needs one unpacker: a merge of mixed encodings, or one the
    // specialized kernel does not serve, is declined before anything is
    // recorded and the caller runs the segments alone (ops/matvec.zig:245-257).
    if (norm) {
        job.norm_weight = norm->weight; job.norm_input = norm->input; job.residual_out = norm->residual_out; job.norm_eps = norm->eps;
    }
    if (generic_only || !same_encoding || !fast_supported(job)) return fail(NU_ERR_MERGE_DECLINED, "segments: merge declined");
    if (int rc = needRecording(true)) return rc;
    if (int rc = chainOrLaunch(job)) return rc;
    if (norm && norm->out_buffer) wrote(*norm->out_buffer);
    for (size_t i = 0; i < count; ++i) wrote(segments[i].output);
    opBoundary();
    return cuda(cudaGetLastError(), "segments: launch");
}

// No reference analogue as one call: `addRmsNorm` (ops/rowwise.zig:76-93) followed by `matvecSegments` on its output
// (inference/src/models/qwen35_metal.zig:635-640), as one launch. The rows the projections multiply are
// norm(residual + input) * weight; residual + input goes to residual_out, which must be a buffer of its own (every
// block of the launch reads residual and input while one of them writes the sum). Declined like a merge when the
// specialized kernel does not serve the segments: the caller then runs the two operators.
int Backend::matvecSegmentsNormed(const Segment *segments, size_t count, const Buffer &residual, const Buffer *input, const Buffer &weight, const Buffer *residual_out,
                                  float eps, uint32_t mode) {
    if (!segments || count == 0 || count > 4) return fail(NU_ERR_INVALID_SHAPE, "segments_normed: 1..4 segments");
    const size_t columns = segments[0].matrix.columns;
    if (columns == 0 || columns > 0xffffffffull / 4 || !(eps > 0)) return fail(NU_ERR_INVALID_SHAPE, "segments_normed: shape");
    if ((input != nullptr) != (residual_out != nullptr)) return fail(NU_ERR_INVALID_SHAPE, "segments_normed: input and residual_out go together");
    NormFuse norm{};
    norm.weight = (const float *)resolve(weight, columns * 4);
    norm.input = input ? (const float *)resolve(*input, columns * 4) : nullptr;
    norm.residual_out = residual_out ? (float *)resolve(*residual_out, columns * 4) : nullptr;
    norm.eps = eps;
    norm.out_buffer = residual_out;
    if (!norm.weight || weight.offset % 16 != 0 || residual.offset % 16 != 0) return fail(NU_ERR_INVALID_SHAPE, "segments_normed: weight too short or not 16-byte aligned");
    if (input) {
        if (!norm.input || !norm.residual_out || input->offset % 16 != 0 || residual_out->offset % 16 != 0) return fail(NU_ERR_INVALID_SHAPE, "segments_normed: buffer too short or not 16-byte aligned");
        if (overlaps(*residual_out, columns * 4, residual, columns * 4) || overlaps(*residual_out, columns * 4, *input, columns * 4) ||
            overlaps(*residual_out, columns * 4, weight, columns * 4))
            return fail(NU_ERR_INVALID_SHAPE, "segments_normed: residual_out overlaps an input");
        for (size_t i = 0; i < count; ++i)
            if (overlaps(*residual_out, columns * 4, segments[i].output, segments[i].matrix.rows * 4) || overlaps(*residual_out, columns * 4, segments[i].weights, segments[i].matrix.bytes))
                return fail(NU_ERR_INVALID_SHAPE, "segments_normed: residual_out overlaps a segment");
    }
    for (size_t i = 0; i < count; ++i)
        if (overlaps(segments[i].output, segments[i].matrix.rows * 4, weight, columns * 4) || (input && overlaps(segments[i].output, segments[i].matrix.rows * 4, *input, columns * 4)))
            return fail(NU_ERR_INVALID_SHAPE, "segments_normed: an output overlaps the norm's inputs");
    return segmentsJob(segments, count, residual, mode, &norm);
}

// ops/rowwise.zig:209-212, 230-233.
int Backend::actMul(uint32_t act, const Buffer &gate, const Buffer &up, size_t count) {
    if (count == 0 || !fits_u32(count)) return fail(NU_ERR_INVALID_SHAPE, "act_mul: count");
    float *g = (float *)resolve(gate, count * 4);
    const float *u = (const float *)resolve(up, count * 4);
    if (!g || !u || gate.offset % 4 != 0 || up.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "act_mul: buffer too short");
    if (int rc = needRecording()) return rc;
    launches_ += launch_act_mul_rows(stream_, act, g, u, g, (uint32_t)count, 1, count, count, count);
    wrote(gate);
    opBoundary();
    return cuda(cudaGetLastError(), "act_mul: launch");
}

// ops/rowwise.zig:37-51 (without the optional SiLU multiplier, which no caller on this path uses).
int Backend::rmsNorm(const Buffer &input, const Buffer &weight, const Buffer &output, const nu_norm &n) {
    if (n.rows == 0 || n.width == 0 || n.in_stride < n.width || n.out_stride < n.width || !(n.eps > 0) || !fits_u32(n.rows) || !fits_u32(n.width)) return fail(NU_ERR_INVALID_SHAPE, "rms_norm: shape");
    float *x = (float *)resolve(input, ((n.rows - 1) * n.in_stride + n.width) * 4);
    float *y = (float *)resolve(output, ((n.rows - 1) * n.out_stride + n.width) * 4);
    const float *w = (const float *)resolve(weight, n.width * 4);
    if (!x || !y || !w || input.offset % 4 != 0 || output.offset % 4 != 0 || weight.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "rms_norm: buffer too short");
    // input and output may alias exactly (the same rows at the same stride); any other overlap is refused
    const bool same = input.id == output.id && input.offset == output.offset && n.in_stride == n.out_stride;
    if (!same && overlaps(input, ((n.rows - 1) * n.in_stride + n.width) * 4, output, ((n.rows - 1) * n.out_stride + n.width) * 4)) return fail(NU_ERR_INVALID_SHAPE, "rms_norm: output overlaps input");
    if (int rc = needRecording()) return rc;
    launches_ += launch_norm_rows(stream_, x, nullptr, w, y, (uint32_t)n.width, (uint32_t)n.rows, n.in_stride, n.out_stride, n.eps);
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "rms_norm: launch");
}

// ops/rowwise.zig:76-93: residual += input, output = norm(residual) * weight, in one pass.
int Backend::addRmsNorm(const Buffer &residual, const Buffer &input, const Buffer &weight, const Buffer &output, const nu_norm &n) {
    if (n.rows == 0 || n.width == 0 || n.in_stride < n.width || n.out_stride < n.width || !(n.eps > 0) || !fits_u32(n.rows) || !fits_u32(n.width)) return fail(NU_ERR_INVALID_SHAPE, "add_rms_norm: shape");
    const size_t in_len = ((n.rows - 1) * n.in_stride + n.width) * 4, out_len = ((n.rows - 1) * n.out_stride + n.width) * 4;
    float *x = (float *)resolve(residual, in_len);
    const float *s = (const float *)resolve(input, in_len);
    float *y = (float *)resolve(output, out_len);
    const float *w = (const float *)resolve(weight, n.width * 4);
    if (!x || !s || !y || !w || residual.offset % 4 != 0 || input.offset % 4 != 0 || output.offset % 4 != 0 || weight.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "add_rms_norm: buffer too short");
    if (overlaps(input, in_len, output, out_len) || overlaps(input, in_len, residual, in_len)) return fail(NU_ERR_INVALID_SHAPE, "add_rms_norm: input overlaps the residual or the output");
    const bool same = residual.id == output.id && residual.offset == output.offset && n.in_stride == n.out_stride;
    if (!same && overlaps(residual, in_len, output, out_len)) return fail(NU_ERR_INVALID_SHAPE, "add_rms_norm: output overlaps the residual");
    if (int rc = needRecording()) return rc;
    launches_ += launch_norm_rows(stream_, x, s, w, y, (uint32_t)n.width, (uint32_t)n.rows, n.in_stride, n.out_stride, n.eps);
    wrote(residual); wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "add_rms_norm: launch");
}

// ops/rowwise.zig:199-202.
int Backend::add(const Buffer &xb, const Buffer &yb, size_t count) {
    if (count == 0) return fail(NU_ERR_INVALID_SHAPE, "add: count");
    float *x = (float *)resolve(xb, count * 4);
    const float *y = (const float *)resolve(yb, count * 4);
    if (!x || !y || xb.offset % 4 != 0 || yb.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "add: buffer too short");
    if (int rc = needRecording()) return rc;
    launches_ += launch_add(stream_, x, y, count);
    wrote(xb);
    opBoundary();
    return cuda(cudaGetLastError(), "add: launch");
}

// ops/sampling.zig:73-86: greedy selection over the head's logits; the scratch of the two passes is the handle's.
int Backend::argmax(const Buffer &logits, size_t count, const Buffer &result) {
    if (count == 0 || count >= 0xffffffffull) return fail(NU_ERR_INVALID_SHAPE, "argmax: count");
    const float *l = (const float *)resolve(logits, count * 4);
    uint32_t *r = (uint32_t *)resolve(result, 4);
    if (!l || !r || logits.offset % 4 != 0 || result.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "argmax: buffer too short");
    if (int rc = needRecording()) return rc;
    launches_ += launch_argmax(stream_, l, (uint32_t)count, argmax_records_, (uint32_t *)(argmax_records_ + 128 * 4), r);
    wrote(result);
    opBoundary();
    return cuda(cudaGetLastError(), "argmax: launch");
}

// ops/experts.zig:29-34.
int Backend::route(const Buffer &logits, size_t experts, size_t k, size_t rows, size_t in_stride, const Buffer &indices, const Buffer &weights) {
    if (experts == 0 || experts > 256 || k == 0 || k > experts || k > 64 || rows == 0 || in_stride < experts || !fits_u32(rows)) return fail(NU_ERR_INVALID_SHAPE, "route: shape");
    const float *l = (const float *)resolve(logits, ((rows - 1) * in_stride + experts) * 4);
    uint32_t *idx = (uint32_t *)resolve(indices, rows * k * 4);
    float *w = (float *)resolve(weights, rows * k * 4);
    if (!l || !idx || !w || logits.offset % 4 != 0 || indices.offset % 4 != 0 || weights.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "route: buffer too short");
    if (int rc = needRecording()) return rc;
    launches_ += launch_route(stream_, l, (uint32_t)experts, (uint32_t)k, (uint32_t)rows, in_stride, idx, w);
    wrote(indices); wrote(weights);
    opBoundary();
    return cuda(cudaGetLastError(), "route: launch");
}

// Expert parallelism (no reference analogue): the routed slots this rank owns, the others silenced.
int Backend::routeLocal(const Buffer &indices, const Buffer &weights, size_t count, size_t first, size_t local, const Buffer &local_indices,
                        const Buffer &local_weights) {
    if (count == 0 || local == 0 || !fits_u32(count) || !fits_u32(first) || !fits_u32(local)) return fail(NU_ERR_INVALID_SHAPE, "route_local: shape");
    const uint32_t *idx = (const uint32_t *)resolve(indices, count * 4);
    const float *w = (const float *)resolve(weights, count * 4);
    uint32_t *lidx = (uint32_t *)resolve(local_indices, count * 4);
    float *lw = (float *)resolve(local_weights, count * 4);
    if (!idx || !w || !lidx || !lw || indices.offset % 4 != 0 || weights.offset % 4 != 0 || local_indices.offset % 4 != 0 || local_weights.offset % 4 != 0)
        return fail(NU_ERR_INVALID_SHAPE, "route_local: buffer too short");
    if (int rc = needRecording()) return rc;
    launches_ += launch_route_local(stream_, idx, w, (uint32_t)count, (uint32_t)first, (uint32_t)local, lidx, lw);
    wrote(local_indices); wrote(local_weights);
    opBoundary();
    return cuda(cudaGetLastError(), "route_local: launch");
}

// ops/experts.zig:50-77 (expertBytes: backends/cpu/experts.zig:29-37).
int Backend::matvecExpertsGrouped(const Buffer &weights, const ExpertMatrix &t, const Buffer &indices, size_t slots,
                                  const Buffer &input, size_t in_stride, size_t in_group, const Buffer &output, size_t out_stride) {
    if (in_group == 0 || in_group > slots) return fail(NU_ERR_INVALID_SHAPE, "experts: in_group");
    if (t.experts == 0 || t.rows == 0 || t.columns == 0 || t.bytes % t.experts != 0 || (t.bytes / t.experts) % t.rows != 0) return fail(NU_ERR_INVALID_SHAPE, "experts: tensor shape");
    const size_t per_expert = t.bytes / t.experts;
    const size_t stride = per_expert / t.rows;
    if (validateRow(t.encoding, stride, t.columns) != NU_OK) return fail(NU_ERR_INVALID_SHAPE, "experts: row layout");
    if (t.columns % 16 != 0 || t.rows > 0xffffffffull / 4 || !fits_u32(t.experts) || !fits_u32(t.columns)) return fail(NU_ERR_INVALID_SHAPE, "experts: sizes");
    if (slots == 0 || slots > 0xffff || out_stride < t.rows || (in_stride != 0 && in_stride < t.columns) || in_stride % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "experts: slots or strides");
    const uint8_t *w = resolve(weights, t.bytes);
    const uint32_t *idx = (const uint32_t *)resolve(indices, slots * 4);
    const float *in = (const float *)resolve(input, ((slots - 1) / in_group * in_stride + t.columns) * 4);
    float *out = (float *)resolve(output, ((slots - 1) * out_stride + t.rows) * 4);
    if (!w || !idx || !in || !out || indices.offset % 4 != 0 || output.offset % 4 != 0 || input.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "experts: buffer too short");
    if (int rc = needRecording()) return rc;
    int launched = generic_only ? 0 : launch_matvec_experts_fast(stream_, t.encoding, w, stride, per_expert, (uint32_t)t.experts, (uint32_t)t.rows, (uint32_t)t.columns, idx,
                                              (uint32_t)slots, in, in_stride, (uint32_t)in_group, out, out_stride);
    if (!launched)
        launched = launch_matvec_experts_generic(stream_, t.encoding, w, stride, per_expert, (uint32_t)t.experts, (uint32_t)t.rows, (uint32_t)t.columns,
                                                 idx, (uint32_t)slots, in, in_stride, (uint32_t)in_group, out, out_stride);
    launches_ += launched;
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "experts: launch");
}

// No reference analogue as one call: `matvecExpertsGrouped` on a gate_up tensor followed by `geluMulRows` on its two halves
// (ops/experts.zig:36-77, 106-117; inference/src/models/gemma4.zig runs them back to back): output[slot][i] =
// act(gate row i . x) * (up row i . x) for i < rows / 2, one launch on the specialized Q4_K kernel; other tensors take the
// generic GEMV into the handle's scratch and the activation pass, so the call never declines. act: 1 SiLU, 2 GELU.
int Backend::matvecExpertsGated(const Buffer &weights, const ExpertMatrix &t, const Buffer &indices, size_t slots, const Buffer &input, size_t in_stride,
                                size_t in_group, const Buffer &output, size_t out_stride, uint32_t act) {
    if (act != ACT_SILU && act != ACT_GELU) return fail(NU_ERR_INVALID_SHAPE, "experts_gated: activation");
    if (in_group == 0 || in_group > slots) return fail(NU_ERR_INVALID_SHAPE, "experts_gated: in_group");
    if (t.experts == 0 || t.rows == 0 || t.rows % 2 != 0 || t.columns == 0 || t.bytes % t.experts != 0 || (t.bytes / t.experts) % t.rows != 0) return fail(NU_ERR_INVALID_SHAPE, "experts_gated: tensor shape");
    const size_t per_expert = t.bytes / t.experts, stride = per_expert / t.rows, width = t.rows / 2;
    if (validateRow(t.encoding, stride, t.columns) != NU_OK) return fail(NU_ERR_INVALID_SHAPE, "experts_gated: row layout");
    if (t.columns % 16 != 0 || t.rows > 0xffffffffull / 4 || !fits_u32(t.experts) || !fits_u32(t.columns)) return fail(NU_ERR_INVALID_SHAPE, "experts_gated: sizes");
    if (slots == 0 || slots > 0xffff || out_stride < width || (in_stride != 0 && in_stride < t.columns) || in_stride % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "experts_gated: slots or strides");
    const uint8_t *w = resolve(weights, t.bytes);
    const uint32_t *idx = (const uint32_t *)resolve(indices, slots * 4);
    const float *in = (const float *)resolve(input, ((slots - 1) / in_group * in_stride + t.columns) * 4);
    float *out = (float *)resolve(output, ((slots - 1) * out_stride + width) * 4);
    if (!w || !idx || !in || !out || indices.offset % 4 != 0 || output.offset % 4 != 0 || input.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "experts_gated: buffer too short");
    if (overlaps(output, ((slots - 1) * out_stride + width) * 4, input, ((slots - 1) / in_group * in_stride + t.columns) * 4)) return fail(NU_ERR_INVALID_SHAPE, "experts_gated: output overlaps input");
    if (int rc = needRecording()) return rc;
    int launched = generic_only ? 0 : launch_matvec_experts_gated_fast(stream_, act, t.encoding, w, stride, per_expert, (uint32_t)t.experts, (uint32_t)t.rows, (uint32_t)t.columns,
                                                                       idx, (uint32_t)slots, in, in_stride, (uint32_t)in_group, out, out_stride);
    if (!launched) {
        if (slots * t.rows > partials_floats_) return fail(NU_ERR_TOO_LARGE, "experts_gated: beyond the scratch");
        int n = generic_only ? 0 : launch_matvec_experts_fast(stream_, t.encoding, w, stride, per_expert, (uint32_t)t.experts, (uint32_t)t.rows, (uint32_t)t.columns, idx,
                                                              (uint32_t)slots, in, in_stride, (uint32_t)in_group, partials_, t.rows);
        if (!n)
            n = launch_matvec_experts_generic(stream_, t.encoding, w, stride, per_expert, (uint32_t)t.experts, (uint32_t)t.rows, (uint32_t)t.columns, idx, (uint32_t)slots, in,
                                              in_stride, (uint32_t)in_group, partials_, t.rows);
        launched = n + launch_act_mul_rows(stream_, act, partials_, partials_ + width, out, (uint32_t)width, (uint32_t)slots, t.rows, t.rows, out_stride);
    }
    launches_ += launched;
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "experts_gated: launch");
}

// ops/experts.zig:119-146: the lists buffer layout is the reference's (expertListsLayout).
static size_t expertTileBound(size_t n, size_t experts) { return (n + 31) / 32 + experts; }
static size_t expertListsWords(size_t n, size_t experts) { return experts + 3 + 3 * expertTileBound(n, experts) + n; }

int Backend::expertLists(const Buffer &indices, size_t rows, size_t k, size_t experts, const Buffer &lists) {
    if (rows == 0 || k == 0 || experts == 0 || experts > 256) return fail(NU_ERR_INVALID_SHAPE, "expert_lists: shape");
    if (rows > 0x3fffffffull / k) return fail(NU_ERR_INVALID_SHAPE, "expert_lists: too many slot rows");
    const size_t n = rows * k;
    const uint32_t *idx = (const uint32_t *)resolve(indices, n * 4);
    uint32_t *l = (uint32_t *)resolve(lists, expertListsWords(n, experts) * 4);
    if (!idx || !l || indices.offset % 4 != 0 || lists.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "expert_lists: buffer too short");
    if (int rc = needRecording()) return rc;
    launches_ += launch_expert_lists(stream_, idx, (uint32_t)n, (uint32_t)experts, (uint32_t)expertTileBound(n, experts), l);
    wrote(lists);
    opBoundary();
    return cuda(cudaGetLastError(), "expert_lists: launch");
}

// ops/experts.zig:148-202.
int Backend::matmulExperts(const Buffer &weights, const ExpertMatrix &t, const Buffer &lists, size_t rows, size_t k, const Buffer &input, size_t in_stride,
                           size_t in_group, const Buffer &output, size_t out_stride) {
    if (t.experts == 0 || t.experts > 256 || t.rows == 0 || t.columns == 0 || t.bytes % t.experts != 0 || (t.bytes / t.experts) % t.rows != 0)
        return fail(NU_ERR_INVALID_SHAPE, "matmul_experts: tensor shape");
    const size_t per_expert = t.bytes / t.experts;
    const size_t stride = per_expert / t.rows;
    if (validateRow(t.encoding, stride, t.columns) != NU_OK) return fail(NU_ERR_INVALID_SHAPE, "matmul_experts: row layout");
    if (t.rows % 8 != 0 || t.columns % 64 != 0 || t.rows > 0xffffffffull / 4 || !fits_u32(t.columns)) return fail(NU_ERR_INVALID_SHAPE, "matmul_experts: sizes");
    if (rows == 0 || k == 0 || in_group == 0 || in_stride < t.columns || out_stride < t.rows || in_stride % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "matmul_experts: rows or strides");
    if (rows > 0x3fffffffull / k) return fail(NU_ERR_INVALID_SHAPE, "matmul_experts: too many slot rows");
    const size_t n = rows * k, input_rows = (n + in_group - 1) / in_group;
    const uint8_t *w = resolve(weights, t.bytes);
    const uint32_t *l = (const uint32_t *)resolve(lists, expertListsWords(n, t.experts) * 4);
    const float *in = (const float *)resolve(input, ((input_rows - 1) * in_stride + t.columns) * 4);
    float *out = (float *)resolve(output, ((n - 1) * out_stride + t.rows) * 4);
    if (!w || !l || !in || !out || lists.offset % 4 != 0 || input.offset % 16 != 0 || output.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "matmul_experts: buffer too short");
    const size_t bound = expertTileBound(n, t.experts);
    if (bound > 65535) return fail(NU_ERR_TOO_LARGE, "matmul_experts: more than 65,535 tiles");
    if (int rc = needRecording()) return rc;
    // From two slot rows per expert on average: the tensor-core tiles (bf16 operands, as the prefill of a dense matrix). Their
    // cost is the decoding of every routed expert's matrix once, whatever the rows (measured, 128 experts: 0.6 ms for both
    // GEMMs at 512 slot rows, where the F32 kernel below takes 5.8 ms). Fewer rows stay on the F32 kernel, exact to 1e-5.
    int launched = 0;
    if (!generic_only && n >= 2 * t.experts && fits_u32(n))
        launched = launch_matmul_experts_fast(stream_, t.encoding, w, stride, per_expert, (uint32_t)t.experts, (uint32_t)t.rows, (uint32_t)t.columns, l, (uint32_t)bound,
                                              (uint32_t)n, in, in_stride, (uint32_t)in_group, out, out_stride, partials_, partials_floats_ * sizeof(float),
                                              counters_ + counters_len_);
    if (!launched)
        launched = launch_matmul_experts_generic(stream_, t.encoding, w, stride, per_expert, (uint32_t)t.experts, (uint32_t)t.rows, (uint32_t)t.columns, l,
                                                 (uint32_t)bound, in, in_stride, (uint32_t)in_group, out, out_stride);
    launches_ += launched;
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "matmul_experts: launch");
}

// ops/experts.zig:106-117.
int Backend::geluMulRows(const Buffer &gate, const Buffer &up, const Buffer &output, size_t width, size_t rows,
                         size_t gate_stride, size_t up_stride, size_t out_stride) {
    if (width == 0 || rows == 0 || gate_stride < width || up_stride < width || out_stride < width || !fits_u32(width) || !fits_u32(rows)) return fail(NU_ERR_INVALID_SHAPE, "gelu_mul_rows: shape");
    const size_t g_len = ((rows - 1) * gate_stride + width) * 4, u_len = ((rows - 1) * up_stride + width) * 4, o_len = ((rows - 1) * out_stride + width) * 4;
    const float *g = (const float *)resolve(gate, g_len);
    const float *u = (const float *)resolve(up, u_len);
    float *o = (float *)resolve(output, o_len);
    if (!g || !u || !o) return fail(NU_ERR_INVALID_SHAPE, "gelu_mul_rows: buffer too short");
    if (overlaps(output, o_len, gate, g_len) || overlaps(output, o_len, up, u_len)) return fail(NU_ERR_INVALID_SHAPE, "gelu_mul_rows: output overlaps an input");
    if (int rc = needRecording()) return rc;
    launches_ += launch_act_mul_rows(stream_, ACT_GELU, g, u, o, (uint32_t)width, (uint32_t)rows, gate_stride, up_stride, out_stride);
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "gelu_mul_rows: launch");
}

// ops/experts.zig:84-92.
int Backend::combineExperts(const Buffer &values, const Buffer &weights, const Buffer &indices, const Buffer *scales,
                            const Buffer &output, const nu_combine_shape &s) {
    if (s.columns == 0 || s.slots == 0 || s.rows == 0 || s.experts == 0 || s.in_stride < s.columns || s.out_stride < s.columns) return fail(NU_ERR_INVALID_SHAPE, "combine: shape");
    if (!fits_u32(s.columns) || !fits_u32(s.rows) || !fits_u32(s.slots) || !fits_u32(s.experts)) return fail(NU_ERR_INVALID_SHAPE, "combine: too large");
    if (s.rows > 65535) return fail(NU_ERR_TOO_LARGE, "combine: more than 65,535 token rows in one call");
    const size_t slot_rows = s.rows * s.slots;
    const float *v = (const float *)resolve(values, ((slot_rows - 1) * s.in_stride + s.columns) * 4);
    const float *w = (const float *)resolve(weights, slot_rows * 4);
    const uint32_t *idx = (const uint32_t *)resolve(indices, slot_rows * 4);
    float *out = (float *)resolve(output, ((s.rows - 1) * s.out_stride + s.columns) * 4);
    if (!v || !w || !idx || !out || indices.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "combine: buffer too short");
    const float *sc = nullptr;
    if (scales) {
        sc = (const float *)resolve(*scales, s.experts * 4);
        if (!sc) return fail(NU_ERR_INVALID_SHAPE, "combine: scales too short");
    }
    if (int rc = needRecording()) return rc;
    launches_ += launch_combine_experts(stream_, v, w, idx, sc, out, (uint32_t)s.columns, (uint32_t)s.slots, (uint32_t)s.rows, s.in_stride, s.out_stride, (uint32_t)s.experts);
    wrote(output);
    opBoundary();
    return cuda(cudaGetLastError(), "combine: launch");
}

// ---- collective: NCCL, loaded at run time so that single-GPU users need no NCCL at all ---------

namespace {
struct NcclId { char b[128]; };  // ncclUniqueId, passed by value
struct Nccl {
    void *lib = nullptr;
    int (*GetUniqueId)(void *) = nullptr;
    int (*CommInitRank)(void **, int, NcclId, int) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool load(std::string &why) {
        if (lib) return true;
        const char *env = getenv("NUCLIS_NCCL_LIB");
        const char *names[] = {env, "libnccl.so.2", "libnccl.so"};
        for (const char *n : names) {
            if (!n || !*n) continue;
            lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (lib) break;
        }
        if (!lib) { why = "cannot load libnccl.so.2 (set NUCLIS_NCCL_LIB to its path)"; return false; }
        GetUniqueId = (decltype(GetUniqueId))dlsym(lib, "ncclGetUniqueId");
        CommInitRank = (decltype(CommInitRank))dlsym(lib, "ncclCommInitRank");
        AllReduce = (decltype(AllReduce))dlsym(lib, "ncclAllReduce");
        CommDestroy = (decltype(CommDestroy))dlsym(lib, "ncclCommDestroy");
        GetErrorString = (decltype(GetErrorString))dlsym(lib, "ncclGetErrorString");
        if (!GetUniqueId || !CommInitRank || !AllReduce || !CommDestroy) { why = "libnccl lacks an expected symbol"; return false; }
        return true;
    }
};
Nccl g_nccl;
constexpr int kNcclFloat = 7, kNcclSum = 0;  // ncclFloat32, ncclSum
}  // namespace

int unique_id(uint8_t *id) {
    std::string why;
    if (!g_nccl.load(why)) return NU_ERR_COMM;
    return g_nccl.GetUniqueId(id) == 0 ? NU_OK : NU_ERR_COMM;
}

int Backend::commInit(const uint8_t *id, int ranks, int rank) {
    if (!id || ranks < 1 || rank < 0 || rank >= ranks) return fail(NU_ERR_INVALID_SHAPE, "comm_init: rank outside the group");
    if (comm_) return fail(NU_ERR_COMM, "comm_init: already joined");
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "comm_init: a recording is open");
    std::string why;
    if (!g_nccl.load(why)) return fail(NU_ERR_COMM, why.c_str());
    cudaSetDevice(device_);
    NcclId nid;
    memcpy(nid.b, id, 128);
    const int rc = g_nccl.CommInitRank(&comm_, ranks, nid, rank);
    if (rc != 0) {
        comm_ = nullptr;
        error_ = std::string("comm_init: ") + (g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "NCCL error");
        return NU_ERR_COMM;
    }
    ranks_ = ranks;
    rank_ = rank;
    // NCCL sets its channels up at the first collective (allocations, a host exchange with the peers).
    // That must not happen inside a stream capture: run one small allreduce here, on the scratch.
    const int warm = g_nccl.AllReduce(partials_, partials_, 256, kNcclFloat, kNcclSum, comm_, stream_);
    if (warm != 0 || cudaStreamSynchronize(stream_) != cudaSuccess) {
        error_ = "comm_init: the warm-up allreduce failed";
        return NU_ERR_COMM;
    }
    return NU_OK;
}

// The inbox of the one-shot allreduce, as an interprocess handle the other ranks open.
int Backend::peerHandle(uint8_t *out) {
    if (!out) return fail(NU_ERR_INVALID_SHAPE, "peer_handle: null result");
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "peer_handle: a recording is open");
    cudaSetDevice(device_);
    if (!inbox_) {
        if (int rc = cuda(cudaMalloc(&inbox_, kPushBytes), "peer_handle: cudaMalloc", NU_ERR_BUFFER)) return rc;
        if (int rc = cuda(cudaMemset(inbox_, 0, kPushBytes), "peer_handle: memset", NU_ERR_BUFFER)) return rc;
    }
    cudaIpcMemHandle_t h;
    if (int rc = cuda(cudaIpcGetMemHandle(&h, inbox_), "peer_handle: cudaIpcGetMemHandle", NU_ERR_COMM)) return rc;
    static_assert(sizeof(h) == 64, "interprocess memory handles are 64 bytes");
    memcpy(out, &h, 64);
    return NU_OK;
}

int Backend::attachPeers(const uint8_t *handles, int ranks, int rank) {
    if (!handles || ranks < 2 || ranks > PUSH_MAX_RANKS || rank < 0 || rank >= ranks) return fail(NU_ERR_INVALID_SHAPE, "attach_peers: 2..8 ranks");
    if (!inbox_ || peers_attached_) return fail(NU_ERR_COMM, "attach_peers: call peer_handle first, attach once");
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "attach_peers: a recording is open");
    cudaSetDevice(device_);
    for (int r = 0; r < ranks; ++r) {
        if (r == rank) { peer_base_[r] = inbox_; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * 64, 64);
        if (int rc = cuda(cudaIpcOpenMemHandle(&peer_base_[r], h, cudaIpcMemLazyEnablePeerAccess), "attach_peers: cudaIpcOpenMemHandle", NU_ERR_COMM)) {
            for (int q = 0; q < r; ++q) if (q != rank && peer_base_[q]) cudaIpcCloseMemHandle(peer_base_[q]);
            memset(peer_base_, 0, sizeof peer_base_);
            return rc;
        }
    }
    peer_ranks_ = ranks;
    peer_rank_ = rank;
    peers_attached_ = true;
    return NU_OK;
}

int Backend::setPeerWaitMs(uint32_t ms) {
    if (ms == 0 || ms > 60000) return fail(NU_ERR_INVALID_SHAPE, "comm_set_wait_ms: 1..60000 ms");
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "comm_set_wait_ms: a recording is open");
    peer_wait_ns_ = (unsigned long long)ms * 1000000ull;  // recorded graphs keep the limit they were recorded with
    return NU_OK;
}

// add_to: the sums are added to this vector (the residual behind a row-split projection) and `buffer` keeps this rank's
// partial values, or whatever the transport leaves there: the residual add folded into the sum's gather.
int Backend::allreduceSumF32(const Buffer &buffer, size_t count, const Buffer *add_to) {
    if (count == 0) return fail(NU_ERR_INVALID_SHAPE, "allreduce: empty");
    float *p = (float *)resolve(buffer, count * 4);
    if (!p || buffer.offset % 4 != 0) return fail(NU_ERR_INVALID_SHAPE, "allreduce: buffer too short");
    float *res = nullptr;
    if (add_to) {
        res = (float *)resolve(*add_to, count * 4);
        if (!res || add_to->offset % 4 != 0 || overlaps(*add_to, count * 4, buffer, count * 4)) return fail(NU_ERR_INVALID_SHAPE, "allreduce: residual too short or overlapping the vector");
    }
    if (peers_attached_ && count <= kPushCapacity) {
        // A one-token matvec whose whole output is this vector was held back: it becomes one kernel that
        // computes and pushes its rows into every rank's inbox, and the sum only gathers.
        const bool fuse = recording_ && pending_ && pending_out_.id == buffer.id && pending_out_.offset == buffer.offset &&
                          pending_job_->job.seg[0].rows == count;
        PushParams pp{};
        pp.buf = p; pp.count = (uint32_t)count; pp.ranks = (uint32_t)peer_ranks_; pp.rank = (uint32_t)peer_rank_; pp.capacity = (uint32_t)kPushCapacity;
        for (int r = 0; r < peer_ranks_; ++r) pp.inbox[r] = (uint2 *)peer_base_[r];
        pp.seq = (uint32_t *)(inbox_ + kPushWordBytes);
        pp.status = counters_ + counters_len_;
        pp.wait_ns = peer_wait_ns_;
        pp.add_to = res;
        if (fuse) {
            cudaSetDevice(device_);
            FastJob &job = pending_job_->job;
            job.push.ranks = pp.ranks; job.push.rank = pp.rank; job.push.capacity = pp.capacity; job.push.seq = pp.seq;
            for (int r = 0; r < peer_ranks_; ++r) job.push.inbox[r] = pp.inbox[r];
            if (fast_supported(job)) {
                pending_ = false;
                launches_ += launch_fast(stream_, job);
                opBoundary();
                launches_ += launch_gather_sum(stream_, pp);
                wrote(buffer);
                if (add_to) wrote(*add_to);
                opBoundary();
                return cuda(cudaGetLastError(), "allreduce: launch");
            }
            job.push.ranks = 0;
        }
        if (int rc = needRecording()) return rc;
        launches_ += launch_push_allreduce(stream_, pp);
        wrote(buffer);
        if (add_to) wrote(*add_to);
        opBoundary();
        return cuda(cudaGetLastError(), "allreduce: launch");
    }
    if (!comm_) return fail(NU_ERR_COMM, "allreduce: no group joined");
    if (int rc = needRecording()) return rc;
    const int rc = g_nccl.AllReduce(p, p, count, kNcclFloat, kNcclSum, comm_, stream_);
    if (rc != 0) {
        error_ = std::string("allreduce: ") + (g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "NCCL error");
        return NU_ERR_COMM;
    }
    wrote(buffer);
    opBoundary();  // a library collective: not counted among this library's own kernel launches
    if (add_to) {
        launches_ += launch_add(stream_, res, p, count);
        wrote(*add_to);
        opBoundary();
        return cuda(cudaGetLastError(), "allreduce: add");
    }
    return NU_OK;
}

int Backend::commDestroy() {
    if (!peers_attached_ && !comm_) return NU_OK;
    if (recording_) return fail(NU_ERR_ALREADY_RECORDING, "comm_destroy: a recording is open");
    // A retained graph may hold kernels with the peers' inbox addresses baked in, or a collective that
    // keeps the communicator busy. Retained graphs are therefore dropped with the group they may refer
    // to, before the peer mappings are closed: a later graph_launch finds no graph instead of storing
    // into unmapped memory.
    cudaSetDevice(device_);
    cudaStreamSynchronize(stream_);
    for (auto &g : graphs_) cudaGraphExecDestroy(g.second);
    graphs_.clear();
    pending_ = false;
    if (peers_attached_) {
        for (int r = 0; r < peer_ranks_; ++r)
            if (r != peer_rank_ && peer_base_[r]) cudaIpcCloseMemHandle(peer_base_[r]);
        memset(peer_base_, 0, sizeof peer_base_);
        peers_attached_ = false;
    }
    if (comm_) {
        g_nccl.CommDestroy(comm_);
        comm_ = nullptr;
    }
    ranks_ = 1;
    rank_ = 0;
    return NU_OK;
}

}  // namespace nu

// ---- C ABI --------------------------------------------------------------------------------------

struct nu_cuda {
    nu::Backend *b;
};

namespace nu { int unique_id(uint8_t *id); }

extern "C" {

nu_cuda *nu_cuda_create(int device, char *err, size_t err_cap) {
    std::string why;
    nu::Backend *b = nu::Backend::create(device, why);
    if (!b) {
        if (err && err_cap) snprintf(err, err_cap, "%s", why.c_str());
        return nullptr;
    }
    return new nu_cuda{b};
}

void nu_cuda_destroy(nu_cuda *h) {
    if (!h) return;
    delete h->b;
    delete h;
}

const char *nu_cuda_last_error(const nu_cuda *h) { return h ? h->b->lastError() : "null handle"; }

const char *nu_cuda_status_name(int status) {
    switch (status) {
    case NU_OK: return "Ok";
    case NU_ERR_UNSUPPORTED_ENCODING: return "UnsupportedTensorEncoding";
    case NU_ERR_INVALID_ROW_LENGTH: return "InvalidRowLength";
    case NU_ERR_INVALID_BYTE_LENGTH: return "InvalidByteLength";
    case NU_ERR_INVALID_SHAPE: return "InvalidShape";
    case NU_ERR_MERGE_DECLINED: return "MergeDeclined";
    case NU_ERR_NOT_RECORDING: return "NotRecording";
    case NU_ERR_ALREADY_RECORDING: return "AlreadyRecording";
    case NU_ERR_BUFFER: return "BufferFailed";
    case NU_ERR_EXECUTION: return "ExecutionFailed";
    case NU_ERR_INIT: return "InitializationFailed";
    case NU_ERR_COMM: return "CommFailed";
    case NU_ERR_TOO_LARGE: return "TooLarge";
    default: return "Unknown";
    }
}

#define NU_H(h) if (!(h)) return NU_ERR_INIT
#define NU_P(p) if (!(p)) return NU_ERR_INVALID_SHAPE

int nu_cuda_set_generic_only(nu_cuda *h, int on) { NU_H(h); h->b->generic_only = on != 0; return NU_OK; }
int nu_cuda_set_chaining(nu_cuda *h, int on) { NU_H(h); h->b->chaining = on != 0; return NU_OK; }
int nu_cuda_buffer_create(nu_cuda *h, size_t len, uint32_t *id) { NU_H(h); return h->b->createBuffer(len, id); }
int nu_cuda_buffer_upload(nu_cuda *h, uint32_t id, size_t offset, const void *src, size_t len) { NU_H(h); return h->b->upload(id, offset, src, len); }
int nu_cuda_buffer_download(nu_cuda *h, uint32_t id, size_t offset, void *dst, size_t len) { NU_H(h); return h->b->download(id, offset, dst, len); }
int nu_cuda_buffer_wrap(nu_cuda *h, const void *bytes, size_t len, uint32_t *id) { NU_H(h); return h->b->wrap(bytes, len, id); }
int nu_cuda_buffer_unwrap(nu_cuda *h, const void *bytes) { NU_H(h); return h->b->unwrap(bytes); }
int nu_cuda_buffer_release(nu_cuda *h, uint32_t id) { NU_H(h); return h->b->release(id); }
void *nu_cuda_buffer_device_ptr(nu_cuda *h, uint32_t id) { return h ? h->b->devicePtr(id) : nullptr; }
uint64_t nu_cuda_created_bytes(const nu_cuda *h) { return h ? h->b->createdBytes() : 0; }

int nu_cuda_matrix_prepare(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix, const nu_buffer *prepared, uint32_t *layout) {
    NU_H(h); NU_P(weights && matrix && prepared && layout);
    return h->b->prepare(*weights, *matrix, *prepared, layout);
}

int nu_cuda_begin(nu_cuda *h) { NU_H(h); return h->b->begin(); }
int nu_cuda_commit(nu_cuda *h) { NU_H(h); return h->b->commit(); }
int nu_cuda_discard(nu_cuda *h) { NU_H(h); return h->b->discard(); }
int nu_cuda_commit_retain(nu_cuda *h, uint32_t *graph) { NU_H(h); return h->b->commitRetain(graph); }
int nu_cuda_graph_launch(nu_cuda *h, uint32_t graph, uint32_t count, float *elapsed_ms) { NU_H(h); return h->b->graphLaunch(graph, count, elapsed_ms); }
int nu_cuda_graph_release(nu_cuda *h, uint32_t graph) { NU_H(h); return h->b->graphRelease(graph); }
double nu_cuda_gpu_seconds(const nu_cuda *h) { return h ? h->b->gpuSeconds() : 0.0; }
uint64_t nu_cuda_launch_count(const nu_cuda *h) { return h ? h->b->launchCount() : 0; }
void *nu_cuda_stream(nu_cuda *h) { return h ? (void *)h->b->stream() : nullptr; }
int nu_cuda_profile_enable(nu_cuda *h, uint32_t max_ops) { NU_H(h); return h->b->profileEnable(max_ops); }
uint32_t nu_cuda_profile_read(nu_cuda *h, double *seconds, uint32_t cap) { return h ? h->b->profileRead(seconds, cap) : 0; }

int nu_cuda_embed(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix, uint32_t token, const nu_buffer *output, uint32_t out_dtype) {
    NU_H(h); NU_P(weights && matrix && output);
    return h->b->embed(*weights, *matrix, token, *output, out_dtype);
}
int nu_cuda_matvec(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix, const nu_buffer *input, const nu_buffer *output) {
    NU_H(h); NU_P(weights && matrix && input && output);
    return h->b->matvec(*weights, *matrix, *input, *output);
}
int nu_cuda_matvec_rows(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix, const nu_buffer *input, size_t in_stride,
                        const nu_buffer *output, size_t out_stride, size_t tokens) {
    NU_H(h); NU_P(weights && matrix && input && output);
    return h->b->matvecRows(*weights, *matrix, *input, in_stride, *output, out_stride, tokens);
}
int nu_cuda_matmul(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix, const nu_buffer *input, uint32_t in_dtype, size_t in_stride,
                   const nu_buffer *output, size_t out_stride, size_t tokens) {
    NU_H(h); NU_P(weights && matrix && input && output);
    return h->b->matmul(*weights, *matrix, *input, in_dtype, in_stride, *output, out_stride, tokens);
}
size_t nu_cuda_matmul_padded(size_t tokens) { return nu::Backend::matmulPadded(tokens); }
int nu_cuda_matvec_add(nu_cuda *h, const nu_buffer *weights, const nu_matrix *matrix, const nu_buffer *input, const nu_buffer *residual, const nu_buffer *output) {
    NU_H(h); NU_P(weights && matrix && input && residual && output);
    return h->b->matvecAdd(*weights, *matrix, *input, *residual, *output);
}
int nu_cuda_matvec_segments(nu_cuda *h, const nu_segment *segments, size_t count, const nu_buffer *input, uint32_t mode) {
    NU_H(h); NU_P(input);
    return h->b->matvecSegments(segments, count, *input, mode);
}
int nu_cuda_matvec_segments_normed(nu_cuda *h, const nu_segment *segments, size_t count, const nu_buffer *residual, const nu_buffer *input, const nu_buffer *weight,
                                   const nu_buffer *residual_out, float eps, uint32_t mode) {
    NU_H(h); NU_P(segments && residual && weight);
    return h->b->matvecSegmentsNormed(segments, count, *residual, input, *weight, residual_out, eps, mode);
}
int nu_cuda_silu_mul(nu_cuda *h, const nu_buffer *gate, const nu_buffer *up, size_t count) {
    NU_H(h); NU_P(gate && up);
    return h->b->actMul(nu::ACT_SILU, *gate, *up, count);
}
int nu_cuda_gelu_mul(nu_cuda *h, const nu_buffer *gate, const nu_buffer *up, size_t count) {
    NU_H(h); NU_P(gate && up);
    return h->b->actMul(nu::ACT_GELU, *gate, *up, count);
}
int nu_cuda_expert_lists(nu_cuda *h, const nu_buffer *indices, size_t rows, size_t k, size_t experts, const nu_buffer *lists) {
    NU_H(h);
    if (!indices || !lists) return NU_ERR_INVALID_SHAPE;
    return h->b->expertLists(*indices, rows, k, experts, *lists);
}
size_t nu_cuda_expert_lists_words(size_t slot_rows, size_t experts) { return experts + 3 + 3 * ((slot_rows + 31) / 32 + experts) + slot_rows; }
int nu_cuda_matmul_experts(nu_cuda *h, const nu_buffer *weights, const nu_expert_matrix *tensor, const nu_buffer *lists, size_t rows, size_t k,
                           const nu_buffer *input, size_t in_stride, size_t in_group, const nu_buffer *output, size_t out_stride) {
    NU_H(h);
    if (!weights || !tensor || !lists || !input || !output) return NU_ERR_INVALID_SHAPE;
    return h->b->matmulExperts(*weights, *tensor, *lists, rows, k, *input, in_stride, in_group, *output, out_stride);
}
int nu_cuda_rms_norm(nu_cuda *h, const nu_buffer *input, const nu_buffer *weight, const nu_buffer *output, const nu_norm *spec) {
    NU_H(h); NU_P(input && weight && output && spec);
    return h->b->rmsNorm(*input, *weight, *output, *spec);
}
int nu_cuda_add_rms_norm(nu_cuda *h, const nu_buffer *residual, const nu_buffer *input, const nu_buffer *weight, const nu_buffer *output, const nu_norm *spec) {
    NU_H(h); NU_P(residual && input && weight && output && spec);
    return h->b->addRmsNorm(*residual, *input, *weight, *output, *spec);
}
int nu_cuda_add(nu_cuda *h, const nu_buffer *x, const nu_buffer *y, size_t count) {
    NU_H(h); NU_P(x && y);
    return h->b->add(*x, *y, count);
}
int nu_cuda_argmax(nu_cuda *h, const nu_buffer *logits, size_t count, const nu_buffer *result) {
    NU_H(h); NU_P(logits && result);
    return h->b->argmax(*logits, count, *result);
}
int nu_cuda_route_local(nu_cuda *h, const nu_buffer *indices, const nu_buffer *weights, size_t count, size_t first_expert, size_t local_experts,
                        const nu_buffer *local_indices, const nu_buffer *local_weights) {
    NU_H(h);
    if (!indices || !weights || !local_indices || !local_weights) return NU_ERR_INVALID_SHAPE;
    return h->b->routeLocal(*indices, *weights, count, first_expert, local_experts, *local_indices, *local_weights);
}
int nu_cuda_route(nu_cuda *h, const nu_buffer *logits, size_t experts, size_t k, size_t rows, size_t in_stride,
                  const nu_buffer *indices, const nu_buffer *weights) {
    NU_H(h); NU_P(logits && indices && weights);
    return h->b->route(*logits, experts, k, rows, in_stride, *indices, *weights);
}
int nu_cuda_matvec_experts(nu_cuda *h, const nu_buffer *weights, const nu_expert_matrix *tensor, const nu_buffer *indices, size_t slots,
                           const nu_buffer *input, size_t in_stride, size_t in_group, const nu_buffer *output, size_t out_stride) {
    NU_H(h); NU_P(weights && tensor && indices && input && output);
    return h->b->matvecExpertsGrouped(*weights, *tensor, *indices, slots, *input, in_stride, in_group, *output, out_stride);
}
int nu_cuda_matvec_experts_gated(nu_cuda *h, const nu_buffer *weights, const nu_expert_matrix *tensor, const nu_buffer *indices, size_t slots, const nu_buffer *input,
                                 size_t in_stride, size_t in_group, const nu_buffer *output, size_t out_stride, uint32_t act) {
    NU_H(h);
    if (!weights || !tensor || !indices || !input || !output) return NU_ERR_INVALID_SHAPE;
    return h->b->matvecExpertsGated(*weights, *tensor, *indices, slots, *input, in_stride, in_group, *output, out_stride, act);
}
int nu_cuda_gelu_mul_rows(nu_cuda *h, const nu_buffer *gate, const nu_buffer *up, const nu_buffer *output,
                          size_t width, size_t rows, size_t gate_stride, size_t up_stride, size_t out_stride) {
    NU_H(h); NU_P(gate && up && output);
    return h->b->geluMulRows(*gate, *up, *output, width, rows, gate_stride, up_stride, out_stride);
}
int nu_cuda_combine_experts(nu_cuda *h, const nu_buffer *values, const nu_buffer *weights, const nu_buffer *indices,
                            const nu_buffer *scales, const nu_buffer *output, const nu_combine_shape *shape) {
    NU_H(h); NU_P(values && weights && indices && output && shape);
    return h->b->combineExperts(*values, *weights, *indices, scales, *output, *shape);
}

int nu_cuda_comm_unique_id(uint8_t id[NU_COMM_ID_BYTES]) { return id ? nu::unique_id(id) : NU_ERR_INVALID_SHAPE; }
int nu_cuda_comm_init(nu_cuda *h, const uint8_t id[NU_COMM_ID_BYTES], int ranks, int rank) { NU_H(h); return h->b->commInit(id, ranks, rank); }
int nu_cuda_allreduce_sum_f32(nu_cuda *h, const nu_buffer *buffer, size_t count) { NU_H(h); NU_P(buffer); return h->b->allreduceSumF32(*buffer, count); }
int nu_cuda_allreduce_sum_add_f32(nu_cuda *h, const nu_buffer *buffer, const nu_buffer *residual, size_t count) { NU_H(h); NU_P(buffer && residual); return h->b->allreduceSumF32(*buffer, count, residual); }
int nu_cuda_comm_destroy(nu_cuda *h) { NU_H(h); return h->b->commDestroy(); }
int nu_cuda_comm_peer_handle(nu_cuda *h, uint8_t handle[NU_PEER_HANDLE_BYTES]) { NU_H(h); return h->b->peerHandle(handle); }
int nu_cuda_comm_attach_peers(nu_cuda *h, const uint8_t *handles, int ranks, int rank) { NU_H(h); return h->b->attachPeers(handles, ranks, rank); }
int nu_cuda_comm_set_wait_ms(nu_cuda *h, uint32_t ms) { NU_H(h); return h->b->setPeerWaitMs(ms); }

}  // extern "C"
