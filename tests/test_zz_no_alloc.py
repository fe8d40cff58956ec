"""The entry point for callers that cannot allocate device memory (nu_cuda_matvec_q4k_static).

A host embedded in another runtime's memory plan, a sandbox without cudaMalloc, or a real-time
loop gets a Q4_K decode GEMV whose scratch is an array inside the library image. This test calls
it through the C ABI with caller-owned device pointers, twice in a row (the array keeps the last
call's contents), and checks the output against the ordinary entry point on the same data.
The file sorts last so that a run that stops at the first failure has run every other test.
"""
import ctypes

import numpy as np
import pytest

from nuclis_b200 import Backend, Matrix, encoding as enc
from parity import assert_matvec_close, expect, make_case

pytestmark = pytest.mark.gpu


def call_static(b, wb, m, xb, yb):
    err = ctypes.create_string_buffer(256)
    stride = m.bytes // m.rows
    return b._lib.nu_cuda_matvec_q4k_static(wb.device_ptr, stride, m.rows, m.columns, xb.device_ptr, yb.device_ptr, b.stream, err, len(err)), err.value.decode()


def planned_slices(b, rows, columns):
    """K slices the entry point will cut this shape into on this GPU (more than one: the built-in array is used)."""
    import torch
    slices, blocks = ctypes.c_uint32(), ctypes.c_uint32()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert b._lib.nu_cuda_matvec_q4k_static_plan(rows, columns, sms, ctypes.byref(slices), ctypes.byref(blocks)) == 0
    return slices.value


# (5120, 17408) and (2048, 20480) are cut along K, so their partial sums and arrival counters go through the
# built-in array; the others fit one slice and never touch it.
@pytest.mark.parametrize("shape,split", [((5120, 17408), True), ((2048, 20480), True), ((5120, 5120), False), ((1024, 2048), False), ((80, 256), False)])
def test_static_scratch_matvec_matches_the_ordinary_entry_point(shape, split):
    rows, columns = shape
    b = Backend(0)
    try:
        assert (planned_slices(b, rows, columns) > 1) == split
        w, x, m = make_case(enc.Q4_K, rows, columns, 1, seed=41)
        want, mag = expect(enc.Q4_K, rows, columns, w, x)
        wb = b.wrap(w)
        xb = b.create(columns * 4)
        y_ref = b.create(rows * 4)
        y_new = b.create(rows * 4)
        xb.write(x)
        b.begin()
        b.matvec(wb, m, xb, y_ref)
        b.commit()
        ref = y_ref.floats()
        for call in range(2):  # the second call meets the scratch as the first left it
            y_new.write(np.full(rows, np.nan, dtype=np.float32))
            status, message = call_static(b, wb, m, xb, y_new)
            assert status == 0, message
            got = y_new.floats()  # the download waits for the backend's stream, on which the kernel ran
            assert_matvec_close(got, want[0], mag[0], f"static scratch {shape} call {call}")
            assert np.allclose(got, ref, rtol=1e-5, atol=1e-6), f"call {call} differs from nu_cuda_matvec"
            word = ctypes.c_uint32(7)
            assert b._lib.nu_cuda_matvec_q4k_static_status(b.stream, ctypes.byref(word)) == 0 and word.value == 0
    finally:
        b.deinit()


def test_static_scratch_rejects_what_it_cannot_hold():
    b = Backend(0)
    try:
        xb = b.create(32768 * 4)
        yb = b.create(64 * 4)
        wb = b.create(64 * (32768 // 256) * 144)
        status, message = call_static(b, wb, Matrix(enc.Q4_K, 64, 32768, wb.len), xb, yb)  # more columns than the limit
        assert status == 12 and "beyond" in message
        status, message = b._lib.nu_cuda_matvec_q4k_static(wb.device_ptr, 100, 64, 256, xb.device_ptr, yb.device_ptr, b.stream, None, 0), ""
        assert status == 4  # a stride that is not the row length
    finally:
        b.deinit()
