"""ctypes binding of the C oracle in ``nu_oracle.c``.

Each wrapper mirrors one function of the reference's CPU path (cited in the C
source) with numpy arrays in place of Zig slices. Errors come back as
``OracleError`` carrying the reference's error name.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libnu_oracle.so")

OK, UNSUPPORTED_ENCODING, INVALID_ROW_LENGTH, INVALID_BYTE_LENGTH, INVALID_SHAPE, SCRATCH_TOO_SMALL, INVALID_EXPERT, NON_FINITE = range(8)
_NAMES = {
    UNSUPPORTED_ENCODING: "UnsupportedTensorEncoding",
    INVALID_ROW_LENGTH: "InvalidRowLength",
    INVALID_BYTE_LENGTH: "InvalidByteLength",
    INVALID_SHAPE: "InvalidShape",
    SCRATCH_TOO_SMALL: "ScratchTooSmall",
    INVALID_EXPERT: "InvalidExpert",
    NON_FINITE: "NonFiniteInput",
}


class OracleError(Exception):
    def __init__(self, code: int):
        self.code = code
        self.name = _NAMES.get(code, f"error {code}")
        super().__init__(self.name)


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc, -ffp-contract=off)."""
    src = os.path.join(_HERE, "nu_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libnu_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def _load():
    global _lib
    if _lib is None:
        build()  # compiles when the library is missing or older than its source
        lib = ctypes.CDLL(_SO)
        sz, u32, vp, f32 = ctypes.c_size_t, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_float
        lib.nu_ref_layout.argtypes = [u32, ctypes.POINTER(u32), ctypes.POINTER(u32)]
        lib.nu_ref_validate_row.argtypes = [u32, sz, sz]
        lib.nu_ref_row.argtypes = [u32, vp, sz, vp, sz]
        lib.nu_ref_matvec.argtypes = [u32, sz, sz, vp, sz, vp, sz, vp, sz, vp, sz, ctypes.c_uint]
        lib.nu_ref_matvec_abs.argtypes = [u32, sz, sz, vp, sz, vp, vp]
        lib.nu_ref_gelu.argtypes = [f32]
        lib.nu_ref_gelu.restype = f32
        lib.nu_ref_silu.argtypes = [f32]
        lib.nu_ref_silu.restype = f32
        lib.nu_ref_route.argtypes = [vp, sz, vp, vp, sz]
        lib.nu_ref_ffn.argtypes = [u32, sz, sz, sz, vp, sz, u32, sz, sz, sz, vp, sz, vp, sz, vp, sz, vp, vp, sz, vp, sz, ctypes.c_uint]
        _lib = lib
    return _lib


def _check(rc: int) -> None:
    if rc != OK:
        raise OracleError(rc)


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def _bytes(a) -> np.ndarray:
    a = np.frombuffer(a, dtype=np.uint8) if isinstance(a, (bytes, bytearray, memoryview)) else np.asarray(a)
    if a.dtype != np.uint8:
        raise TypeError("weights must be uint8")
    return np.ascontiguousarray(a)


def cores() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def layout(encoding: int) -> tuple[int, int]:
    e, b = ctypes.c_uint32(), ctypes.c_uint32()
    _check(_load().nu_ref_layout(encoding, ctypes.byref(e), ctypes.byref(b)))
    return e.value, b.value


def validate_row(encoding: int, byte_count: int, element_count: int) -> None:
    _check(_load().nu_ref_validate_row(encoding, byte_count, element_count))


def row(encoding: int, data, elements: int, out: np.ndarray | None = None) -> np.ndarray:
    """quant.row: decode one row of ``elements`` values. ``out`` is left untouched on error."""
    data = _bytes(data)
    if out is None:
        out = np.empty(elements, dtype=np.float32)
    _check(_load().nu_ref_row(encoding, _ptr(data), data.size, _ptr(out), elements))
    return out


def matvec(encoding: int, rows: int, columns: int, data, x: np.ndarray, tasks: int | None = None,
           out: np.ndarray | None = None, scratch_len: int | None = None) -> np.ndarray:
    """cpu.matvec: F64 accumulation in column order, one rounding to F32."""
    data = _bytes(data)
    x = np.ascontiguousarray(x, dtype=np.float32)
    if out is None:
        out = np.empty(rows, dtype=np.float32)
    tasks = cores() if tasks is None else tasks
    if scratch_len is None:
        scratch_len = max(1, tasks) * columns
    scratch = np.empty(max(scratch_len, 1), dtype=np.float32)
    _check(_load().nu_ref_matvec(encoding, rows, columns, _ptr(data), data.size, _ptr(x), x.size, _ptr(out), out.size,
                                 _ptr(scratch), scratch_len, tasks))
    return out


def matmul(encoding: int, rows: int, columns: int, data, x: np.ndarray, tasks: int | None = None) -> np.ndarray:
    """Batched expectation: ``cpu.matvec`` once per token row, as the reference's checks build it
    (inference/metal-check.zig:4414-4416). ``x`` is [tokens][columns]; returns [tokens][rows]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    return np.stack([matvec(encoding, rows, columns, data, x[t], tasks) for t in range(x.shape[0])])


def matvec_abs(encoding: int, rows: int, columns: int, data, x: np.ndarray) -> np.ndarray:
    """sum_c |w[r,c]*x[c]| per row in F64: the scale of the acceptance formula."""
    data = _bytes(data)
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(rows, dtype=np.float64)
    _check(_load().nu_ref_matvec_abs(encoding, rows, columns, _ptr(data), data.size, _ptr(x), _ptr(out)))
    return out


def gelu(x) -> np.ndarray:
    f = _load().nu_ref_gelu
    return np.array([f(float(v)) for v in np.asarray(x, dtype=np.float32).ravel()], dtype=np.float32).reshape(np.shape(x))


def silu(x) -> np.ndarray:
    f = _load().nu_ref_silu
    return np.array([f(float(v)) for v in np.asarray(x, dtype=np.float32).ravel()], dtype=np.float32).reshape(np.shape(x))


def rms_norm(x: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    """cpu rmsNorm (vector.zig:53-64): x / sqrt(mean(x^2) + eps), the sum of squares in F64; no weight."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    f = _load().nu_ref_rms_norm
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float]
    _check(f(_ptr(x), _ptr(out), x.size, eps))
    return out


def route(logits: np.ndarray, k: int) -> tuple[np.ndarray, np.ndarray]:
    """cpu.experts.route for one token: (indices u32[k], weights f32[k])."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    idx = np.zeros(max(k, 1), dtype=np.uint32)
    w = np.zeros(max(k, 1), dtype=np.float32)
    _check(_load().nu_ref_route(_ptr(logits), logits.size, _ptr(idx), _ptr(w), k))
    return idx[:k], w[:k]


def ffn(gate_up: tuple, down: tuple, x: np.ndarray, indices: np.ndarray, weights: np.ndarray,
        down_scale: np.ndarray | None = None, tasks: int | None = None) -> np.ndarray:
    """cpu.experts.ffn. ``gate_up`` and ``down`` are (encoding, experts, rows, columns, bytes)."""
    ge, gx, gr, gc, gb = gate_up
    de, dx, dr, dc, db = down
    gb, db = _bytes(gb), _bytes(db)
    x = np.ascontiguousarray(x, dtype=np.float32)
    indices = np.ascontiguousarray(indices, dtype=np.uint32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    out = np.empty(dr, dtype=np.float32)
    if down_scale is not None:
        down_scale = np.ascontiguousarray(down_scale, dtype=np.float32)
    _check(_load().nu_ref_ffn(ge, gx, gr, gc, _ptr(gb), gb.size, de, dx, dr, dc, _ptr(db), db.size,
                              _ptr(down_scale) if down_scale is not None else None,
                              down_scale.size if down_scale is not None else 0,
                              _ptr(x), x.size, _ptr(indices), _ptr(weights), indices.size, _ptr(out), out.size,
                              cores() if tasks is None else tasks))
    return out
