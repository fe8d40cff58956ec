"""Python host side: the operator interface of the engine's ``metal.Backend``
(inference/src/backends/metal/root.zig:88-330, ops/{matvec,matmul,experts,rowwise}.zig)
over the C ABI of ``libnuclis_cuda.so``.

Method names, argument order and error behaviour follow the reference so that
a test written against ``metal.Backend`` reads the same here:

    backend = Backend()                       # Backend.init
    w = backend.wrap(weight_bytes)            # upload once, cached by address
    x = backend.create(columns * 4)           # zero-filled
    y = backend.create(rows * 4)
    x.write(values)
    backend.begin()
    backend.matvec(w, Matrix(Q4_K, rows, columns, len(weight_bytes)), x, y)
    backend.commit()                          # submits and waits
    out = y.floats()

Every failed call raises ``NuclisError`` whose ``name`` is the reference's
error name; shape errors are raised before anything is recorded.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from enum import IntEnum

import numpy as np

from . import _lib
from .errors import NuclisError


@dataclass(frozen=True)
class Matrix:
    """``cpu.Matrix`` (inference/src/backends/cpu/root.zig:31-36); ``bytes`` is the byte length."""
    encoding: int
    rows: int
    columns: int
    bytes: int
    layout: int = 0  # 0: GGUF rows; otherwise what Backend.prepare returned

    def _c(self) -> _lib.CMatrix:
        return _lib.CMatrix(self.encoding, self.layout, self.rows, self.columns, self.bytes)


@dataclass(frozen=True)
class ExpertMatrix:
    """``cpu.ExpertMatrix`` (inference/src/backends/cpu/experts.zig:20-43)."""
    encoding: int
    experts: int
    rows: int
    columns: int
    bytes: int

    def _c(self) -> _lib.CExpertMatrix:
        return _lib.CExpertMatrix(self.encoding, 0, self.experts, self.rows, self.columns, self.bytes)


class SegmentMode(IntEnum):
    """``SegmentMode`` (ops/matvec.zig:224)."""
    plain = 0
    silu_mul_pair = 1
    gelu_mul_pair = 2


@dataclass(frozen=True)
class CombineShape:
    """``CombineShape`` (ops/experts.zig:80)."""
    columns: int
    slots: int
    experts: int
    in_stride: int
    out_stride: int
    rows: int = 1


class Buffer:
    """``Buffer`` (root.zig:62-86): a byte range of a device buffer; ``slice`` derives sub-ranges."""

    def __init__(self, backend: "Backend", id: int, offset: int, len: int):
        self.backend, self.id, self.offset, self.len = backend, id, offset, len

    def slice(self, byte_offset: int, len: int) -> "Buffer":
        assert byte_offset + len <= self.len
        return Buffer(self.backend, self.id, self.offset + byte_offset, len)

    def _c(self) -> _lib.CBuffer:
        return _lib.CBuffer(self.id, 0, self.offset, self.len)

    # Device memory has no host pointer: these replace `Buffer.host` / `floats()`.
    def write(self, data) -> None:
        a = np.ascontiguousarray(data)
        raw = a.view(np.uint8).reshape(-1)
        if raw.size > self.len:
            raise NuclisError(4, "write: data longer than the view")
        self.backend._check(self.backend._lib.nu_cuda_buffer_upload(self.backend._h, self.id, self.offset, raw.ctypes.data, raw.size))

    def read(self, dtype=np.uint8, count: int | None = None) -> np.ndarray:
        dtype = np.dtype(dtype)
        n = self.len // dtype.itemsize if count is None else count
        out = np.empty(n, dtype=dtype)
        self.backend._check(self.backend._lib.nu_cuda_buffer_download(self.backend._h, self.id, self.offset, out.ctypes.data, out.nbytes))
        return out

    def floats(self) -> np.ndarray:
        return self.read(np.float32)

    @property
    def device_ptr(self) -> int:
        base = self.backend._lib.nu_cuda_buffer_device_ptr(self.backend._h, self.id)
        return (base or 0) + self.offset


@dataclass(frozen=True)
class Segment:
    """``Segment`` (ops/matvec.zig:223)."""
    weights: Buffer
    matrix: Matrix
    output: Buffer


class Backend:
    """One CUDA device context. Not thread-safe: one thread owns it (root.zig:7-10)."""

    matvec_rows_max = 8  # ops/matvec.zig:140-143
    matmul_tile = 64     # ops/matmul.zig:19-21

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        err = ctypes.create_string_buffer(512)
        self._h = self._lib.nu_cuda_create(device, err, len(err))
        if not self._h:
            raise NuclisError(10, err.value.decode() or "nu_cuda_create failed")
        self.device = device
        self._keep = {}  # host arrays handed to wrap(), kept alive like the borrowed ranges of the reference

    # ---- lifecycle ----
    def deinit(self) -> None:
        if getattr(self, "_h", None):
            self._lib.nu_cuda_destroy(self._h)
            self._h = None

    close = deinit

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.deinit()

    def __del__(self):
        try:
            self.deinit()
        except Exception:
            pass

    def _check(self, status: int) -> None:
        if status != 0:
            raise NuclisError(status, self._lib.nu_cuda_last_error(self._h).decode())

    @property
    def generic_only(self) -> bool:
        return self._generic_only if hasattr(self, "_generic_only") else False

    @generic_only.setter
    def generic_only(self, on: bool) -> None:
        self._check(self._lib.nu_cuda_set_generic_only(self._h, int(bool(on))))
        self._generic_only = bool(on)

    @property
    def chaining(self) -> bool:
        """Back-to-back one-token matvecs run as one persistent kernel (off by default: measured slower than kernels of
        their own; no counterpart in the reference)."""
        return self._chaining if hasattr(self, "_chaining") else False

    @chaining.setter
    def chaining(self, on: bool) -> None:
        self._check(self._lib.nu_cuda_set_chaining(self._h, int(bool(on))))
        self._chaining = bool(on)

    # ---- buffers ----
    def create(self, len: int) -> Buffer:
        id = ctypes.c_uint32()
        self._check(self._lib.nu_cuda_buffer_create(self._h, len, ctypes.byref(id)))
        return Buffer(self, id.value, 0, len)

    def release(self, buffer: Buffer) -> None:
        if buffer.offset != 0:
            raise NuclisError(4, "release: whole buffers only")
        self._check(self._lib.nu_cuda_buffer_release(self._h, buffer.id))

    def wrap(self, data: np.ndarray) -> Buffer:
        """Uploads a host range once; later wraps of the same start address return the same buffer."""
        a = np.ascontiguousarray(data)
        raw = a.view(np.uint8).reshape(-1)
        id = ctypes.c_uint32()
        self._check(self._lib.nu_cuda_buffer_wrap(self._h, raw.ctypes.data, raw.size, ctypes.byref(id)))
        self._keep[raw.ctypes.data] = raw
        return Buffer(self, id.value, 0, raw.size)

    def unwrap(self, data: np.ndarray) -> None:
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        self._check(self._lib.nu_cuda_buffer_unwrap(self._h, raw.ctypes.data))
        self._keep.pop(raw.ctypes.data, None)

    def prepare(self, weights: Buffer, matrix: Matrix, prepared: Buffer | None = None) -> tuple[Buffer, Matrix]:
        """Re-lays a matrix once, at load time, into the form the specialized kernels read (same bytes,
        same values; see nu_cuda_matrix_prepare). Returns the prepared buffer and its descriptor."""
        out = prepared if prepared is not None else self.create(matrix.bytes)
        layout = ctypes.c_uint32()
        self._check(self._lib.nu_cuda_matrix_prepare(self._h, weights._c(), matrix._c(), out._c(), ctypes.byref(layout)))
        return out, Matrix(matrix.encoding, matrix.rows, matrix.columns, matrix.bytes, layout.value)

    @property
    def created_bytes(self) -> int:
        return self._lib.nu_cuda_created_bytes(self._h)

    # ---- recording ----
    def begin(self) -> None:
        self._check(self._lib.nu_cuda_begin(self._h))

    def commit(self) -> None:
        self._check(self._lib.nu_cuda_commit(self._h))

    def discard(self) -> None:
        self._check(self._lib.nu_cuda_discard(self._h))

    def commit_retain(self) -> int:
        g = ctypes.c_uint32()
        self._check(self._lib.nu_cuda_commit_retain(self._h, ctypes.byref(g)))
        return g.value

    def graph_launch(self, graph: int, count: int = 1) -> float:
        """Replays a retained recording ``count`` times; returns the device milliseconds of the batch."""
        ms = ctypes.c_float()
        self._check(self._lib.nu_cuda_graph_launch(self._h, graph, count, ctypes.byref(ms)))
        return ms.value

    def graph_release(self, graph: int) -> None:
        self._check(self._lib.nu_cuda_graph_release(self._h, graph))

    def gpu_seconds(self) -> float:
        return self._lib.nu_cuda_gpu_seconds(self._h)

    @property
    def launch_count(self) -> int:
        return self._lib.nu_cuda_launch_count(self._h)

    @property
    def stream(self) -> int:
        return self._lib.nu_cuda_stream(self._h) or 0

    def enable_profiling(self, max_ops: int) -> None:
        self._check(self._lib.nu_cuda_profile_enable(self._h, max_ops))

    def profile_read(self) -> np.ndarray:
        n = self._lib.nu_cuda_profile_read(self._h, None, 0)
        out = np.zeros(n, dtype=np.float64)
        if n:
            self._lib.nu_cuda_profile_read(self._h, out.ctypes.data_as(ctypes.POINTER(ctypes.c_double)), n)
        return out

    # ---- operators ----
    def embed(self, weights: Buffer, matrix: Matrix, token: int, output: Buffer, out_dtype: int = 0) -> None:
        self._check(self._lib.nu_cuda_embed(self._h, weights._c(), matrix._c(), token, output._c(), out_dtype))

    def matvec(self, weights: Buffer, matrix: Matrix, input: Buffer, output: Buffer) -> None:
        self._check(self._lib.nu_cuda_matvec(self._h, weights._c(), matrix._c(), input._c(), output._c()))

    def matvec_add(self, weights: Buffer, matrix: Matrix, input: Buffer, residual: Buffer, output: Buffer) -> None:
        """``matvec`` and the residual ``add`` of its output (ops/matvec.zig:85-116, ops/rowwise.zig:199-202) as one launch:
        output = residual + W x; ``output`` may be ``residual``."""
        self._check(self._lib.nu_cuda_matvec_add(self._h, weights._c(), matrix._c(), input._c(), residual._c(), output._c()))

    def matvec_rows(self, weights: Buffer, matrix: Matrix, input: Buffer, in_stride: int, output: Buffer, out_stride: int, tokens: int) -> None:
        self._check(self._lib.nu_cuda_matvec_rows(self._h, weights._c(), matrix._c(), input._c(), in_stride, output._c(), out_stride, tokens))

    def matmul(self, weights: Buffer, matrix: Matrix, input: Buffer, in_stride: int, output: Buffer, out_stride: int, tokens: int,
               in_dtype: int = 0) -> None:
        self._check(self._lib.nu_cuda_matmul(self._h, weights._c(), matrix._c(), input._c(), in_dtype, in_stride, output._c(), out_stride, tokens))

    @staticmethod
    def matmul_padded(tokens: int) -> int:
        return (tokens + 63) // 64 * 64

    def matvec_segments(self, segments: list[Segment], input: Buffer, mode: SegmentMode = SegmentMode.plain) -> None:
        arr = (_lib.CSegment * max(len(segments), 1))()
        for i, s in enumerate(segments):
            arr[i] = _lib.CSegment(s.weights._c(), s.matrix._c(), s.output._c())
        self._check(self._lib.nu_cuda_matvec_segments(self._h, arr, len(segments), input._c(), int(mode)))

    def matvec_segments_normed(self, segments: list[Segment], residual: Buffer, weight: Buffer, input: Buffer | None = None,
                               residual_out: Buffer | None = None, eps: float = 1e-6, mode: SegmentMode = SegmentMode.plain) -> None:
        """``addRmsNorm`` (ops/rowwise.zig:76-93) and ``matvecSegments`` on its output as one launch: the segments multiply
        norm(residual + input) * weight, and residual + input goes to ``residual_out`` (a buffer of its own). Without
        ``input`` / ``residual_out``: ``rmsNorm`` + ``matvecSegments``. Raises MergeDeclined when the specialized kernel
        does not serve the segments."""
        arr = (_lib.CSegment * max(len(segments), 1))()
        for i, s in enumerate(segments):
            arr[i] = _lib.CSegment(s.weights._c(), s.matrix._c(), s.output._c())
        self._check(self._lib.nu_cuda_matvec_segments_normed(self._h, arr, len(segments), residual._c(), input._c() if input is not None else None, weight._c(),
                                                             residual_out._c() if residual_out is not None else None, eps, int(mode)))

    def silu_mul(self, gate: Buffer, up: Buffer, count: int) -> None:
        self._check(self._lib.nu_cuda_silu_mul(self._h, gate._c(), up._c(), count))

    def gelu_mul(self, gate: Buffer, up: Buffer, count: int) -> None:
        self._check(self._lib.nu_cuda_gelu_mul(self._h, gate._c(), up._c(), count))

    def rms_norm(self, input: Buffer, weight: Buffer, output: Buffer, rows: int, width: int, in_stride: int | None = None, out_stride: int | None = None,
                 eps: float = 1e-6) -> None:
        """``rmsNorm`` (ops/rowwise.zig:37-51): output = input * rsqrt(mean(input^2) + eps) * weight per row."""
        n = _lib.CNorm(rows, width, in_stride or width, out_stride or width, eps)
        self._check(self._lib.nu_cuda_rms_norm(self._h, input._c(), weight._c(), output._c(), ctypes.byref(n)))

    def add_rms_norm(self, residual: Buffer, input: Buffer, weight: Buffer, output: Buffer, rows: int, width: int, in_stride: int | None = None,
                     out_stride: int | None = None, eps: float = 1e-6) -> None:
        """``addRmsNorm`` (ops/rowwise.zig:76-93): residual += input, output = norm(residual) * weight."""
        n = _lib.CNorm(rows, width, in_stride or width, out_stride or width, eps)
        self._check(self._lib.nu_cuda_add_rms_norm(self._h, residual._c(), input._c(), weight._c(), output._c(), ctypes.byref(n)))

    def add(self, x: Buffer, y: Buffer, count: int) -> None:
        """``add`` (ops/rowwise.zig:199-202): x += y."""
        self._check(self._lib.nu_cuda_add(self._h, x._c(), y._c(), count))

    def argmax(self, logits: Buffer, count: int, result: Buffer) -> None:
        """Index of the largest logit into `result` (one uint32; 0xffffffff if a logit is not finite)."""
        self._check(self._lib.nu_cuda_argmax(self._h, logits._c(), count, result._c()))

    def route(self, logits: Buffer, experts: int, k: int, rows: int, in_stride: int, indices: Buffer, weights: Buffer) -> None:
        self._check(self._lib.nu_cuda_route(self._h, logits._c(), experts, k, rows, in_stride, indices._c(), weights._c()))

    @staticmethod
    def expert_lists_words(slot_rows: int, experts: int) -> int:
        """32-bit words of the lists buffer `expert_lists` fills (the reference's `expertListsLayout`)."""
        return _lib.load().nu_cuda_expert_lists_words(slot_rows, experts)

    def expert_lists(self, indices: Buffer, rows: int, k: int, experts: int, lists: Buffer) -> None:
        self._check(self._lib.nu_cuda_expert_lists(self._h, indices._c(), rows, k, experts, lists._c()))

    def matmul_experts(self, weights: Buffer, tensor: ExpertMatrix, lists: Buffer, rows: int, k: int, input: Buffer, in_stride: int, in_group: int,
                       output: Buffer, out_stride: int) -> None:
        self._check(self._lib.nu_cuda_matmul_experts(self._h, weights._c(), tensor._c(), lists._c(), rows, k, input._c(), in_stride, in_group,
                                                     output._c(), out_stride))

    def route_local(self, indices: Buffer, weights: Buffer, count: int, first_expert: int, local_experts: int, local_indices: Buffer,
                    local_weights: Buffer) -> None:
        """Expert parallelism: the routed slots this rank owns (local index, same weight), the others silenced (index 0, weight 0)."""
        self._check(self._lib.nu_cuda_route_local(self._h, indices._c(), weights._c(), count, first_expert, local_experts, local_indices._c(),
                                                  local_weights._c()))

    def matvec_experts(self, weights: Buffer, tensor: ExpertMatrix, indices: Buffer, slots: int, input: Buffer, in_stride: int,
                       output: Buffer, out_stride: int) -> None:
        self.matvec_experts_grouped(weights, tensor, indices, slots, input, in_stride, 1, output, out_stride)

    def matvec_experts_grouped(self, weights: Buffer, tensor: ExpertMatrix, indices: Buffer, slots: int, input: Buffer, in_stride: int,
                               in_group: int, output: Buffer, out_stride: int) -> None:
        self._check(self._lib.nu_cuda_matvec_experts(self._h, weights._c(), tensor._c(), indices._c(), slots, input._c(), in_stride, in_group,
                                                     output._c(), out_stride))

    def matvec_experts_gated(self, weights: Buffer, tensor: ExpertMatrix, indices: Buffer, slots: int, input: Buffer, in_stride: int, in_group: int,
                             output: Buffer, out_stride: int, act: int = 2) -> None:
        """``matvecExpertsGrouped`` on a gate_up tensor and ``geluMulRows`` on its halves (ops/experts.zig:36-77, 106-117) as one
        launch: output[slot][i] = act(gate row i . x) * (up row i . x); ``act``: 1 SiLU, 2 GELU."""
        self._check(self._lib.nu_cuda_matvec_experts_gated(self._h, weights._c(), tensor._c(), indices._c(), slots, input._c(), in_stride, in_group,
                                                           output._c(), out_stride, act))

    def gelu_mul_rows(self, gate: Buffer, up: Buffer, output: Buffer, width: int, rows: int, gate_stride: int, up_stride: int, out_stride: int) -> None:
        self._check(self._lib.nu_cuda_gelu_mul_rows(self._h, gate._c(), up._c(), output._c(), width, rows, gate_stride, up_stride, out_stride))

    def combine_experts(self, values: Buffer, weights: Buffer, indices: Buffer, scales: Buffer | None, output: Buffer, s: CombineShape) -> None:
        shape = _lib.CCombineShape(s.columns, s.slots, s.rows, s.experts, s.in_stride, s.out_stride)
        self._check(self._lib.nu_cuda_combine_experts(self._h, values._c(), weights._c(), indices._c(), scales._c() if scales is not None else None,
                                                      output._c(), ctypes.byref(shape)))

    # ---- collective ----
    @staticmethod
    def comm_unique_id() -> bytes:
        lib = _lib.load()
        buf = (ctypes.c_uint8 * 128)()
        rc = lib.nu_cuda_comm_unique_id(buf)
        if rc != 0:
            raise NuclisError(rc, "nu_cuda_comm_unique_id")
        return bytes(buf)

    def comm_init(self, unique_id: bytes, ranks: int, rank: int) -> None:
        buf = (ctypes.c_uint8 * 128).from_buffer_copy(unique_id)
        self._check(self._lib.nu_cuda_comm_init(self._h, buf, ranks, rank))

    def allreduce_sum_f32(self, buffer: Buffer, count: int) -> None:
        self._check(self._lib.nu_cuda_allreduce_sum_f32(self._h, buffer._c(), count))

    def allreduce_sum_add_f32(self, buffer: Buffer, residual: Buffer, count: int) -> None:
        """residual += the sum over the group of ``buffer``: the residual add behind a row-split projection, in the sum's gather."""
        self._check(self._lib.nu_cuda_allreduce_sum_add_f32(self._h, buffer._c(), residual._c(), count))

    def comm_peer_handle(self) -> bytes:
        """This rank's inbox for the one-shot allreduce, as a 64-byte interprocess handle."""
        buf = (ctypes.c_uint8 * 64)()
        self._check(self._lib.nu_cuda_comm_peer_handle(self._h, buf))
        return bytes(buf)

    def comm_attach_peers(self, handles: list[bytes], rank: int) -> None:
        """Opens every rank's inbox (handles ordered by rank); short allreduces then bypass NCCL."""
        flat = (ctypes.c_uint8 * (64 * len(handles))).from_buffer_copy(b"".join(handles))
        self._check(self._lib.nu_cuda_comm_attach_peers(self._h, flat, len(handles), rank))

    def comm_set_wait_ms(self, ms: int) -> None:
        """How long a kernel of the peer-memory allreduce waits for the peers' words before it gives up."""
        self._check(self._lib.nu_cuda_comm_set_wait_ms(self._h, ms))

    def comm_destroy(self) -> None:
        self._check(self._lib.nu_cuda_comm_destroy(self._h))
