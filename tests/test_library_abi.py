"""CPU-side checks of the boundary: the library builds, loads and exports every symbol the
header declares; the Python mirror declares every one of them; host-side layout arithmetic."""
import ctypes
import os
import re

import numpy as np
import pytest

from nuclis_b200 import _lib, build, encoding as enc, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nuclis_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nu_cuda_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    lib = ctypes.CDLL(path)
    names = declared_symbols()
    assert len(names) >= 35
    for name in names:
        assert hasattr(lib, name), f"{name} declared in nuclis_cuda.h but not exported"


def test_python_mirror_covers_the_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_status_names_need_no_device():
    lib = _lib.load()
    assert lib.nu_cuda_status_name(4) == b"InvalidShape"
    assert lib.nu_cuda_status_name(5) == b"MergeDeclined"
    assert lib.nu_cuda_matmul_padded(1) == 64 and lib.nu_cuda_matmul_padded(65) == 128


def test_layout_arithmetic():
    assert enc.row_bytes(enc.Q4_K, 4096) == 2304
    assert enc.matrix_bytes(enc.Q4_K, 4096, 4096) == 9437184
    assert enc.matrix_bytes(enc.Q6_K, 5120, 17408) == 5120 * 14280
    assert enc.row_bytes(enc.Q8_0, 704) == 748
    with pytest.raises(ValueError):
        enc.row_bytes(enc.Q6_K, 704)
    assert enc.bits_per_weight(enc.Q4_K) == 4.5 and enc.bits_per_weight(enc.Q8_0) == 8.5


def test_synthetic_blocks_decode_to_finite_values_and_are_seeded():
    import oracle
    for e in (enc.Q4_K, enc.Q6_K, enc.Q8_0):
        a = synth.matrix(e, 3, 512, seed=5)
        b = synth.matrix(e, 3, 512, seed=5)
        c = synth.matrix(e, 3, 512, seed=6)
        assert np.array_equal(a, b) and not np.array_equal(a, c)
        assert a.size == enc.matrix_bytes(e, 3, 512)
        stride = a.size // 3
        vals = oracle.row(e, a[:stride], 512)
        assert np.all(np.isfinite(vals)) and np.any(vals != 0)
    # Q6_K sub-scales stay in [-32, 31]; Q8_0 codes never take -128
    q6 = synth.matrix(enc.Q6_K, 4, 256, seed=1).reshape(-1, 210)
    sub = q6[:, 192:208].view(np.int8)
    assert sub.min() >= -32 and sub.max() <= 31
    q8 = synth.matrix(enc.Q8_0, 4, 256, seed=1).reshape(-1, 34)
    assert q8[:, 2:].view(np.int8).min() >= -127


def test_static_entry_point_plans_its_whole_documented_range():
    """The planner (host arithmetic) finds a cut that fits the built-in array up to the documented limits."""
    lib = _lib.load()
    slices, blocks = ctypes.c_uint32(), ctypes.c_uint32()
    for rows, columns in ((65536, 20480), (50000, 20480), (65536, 256), (16, 20480), (5120, 17408)):
        assert lib.nu_cuda_matvec_q4k_static_plan(rows, columns, 148, ctypes.byref(slices), ctypes.byref(blocks)) == 0, (rows, columns)
        assert 1 <= slices.value <= 32 and 1 <= blocks.value <= 148
        # partial sums of a cut: slices x 16-row tiles x 32 floats, inside 256 Ki floats
        assert slices.value == 1 or slices.value * ((rows + 15) // 16) * 32 <= 256 * 1024
    assert lib.nu_cuda_matvec_q4k_static_plan(65537, 256, 148, ctypes.byref(slices), ctypes.byref(blocks)) == 12
    assert lib.nu_cuda_matvec_q4k_static_plan(16, 20736, 148, ctypes.byref(slices), ctypes.byref(blocks)) == 12
    assert lib.nu_cuda_matvec_q4k_static_plan(16, 100, 148, ctypes.byref(slices), ctypes.byref(blocks)) == 4
