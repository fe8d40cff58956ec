"""GPU parity of the encodings served by the generic kernels: Q4_0, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, IQ4_NL, IQ4_XS.

The reference decodes them in inference/src/quant/decode.zig:46-56, 125-143, 147-196, 260-275 and pins
them with the rows of its fixtures simple, five-bit, codebook, k-affine and k-signed.json, which
tests/golden/quant_rows.json carries; the golden-row tests of test_gpu_matvec.py decode those on the
device bit for bit. Here: random matrices through every operator entry point (row decode, one-token
GEMV, 2..8 token rows, prefill tiles) against the CPU oracle, all through the C ABI.
"""
import numpy as np
import pytest

import oracle
from nuclis_b200 import Backend, Matrix, encoding as enc, synth
from parity import assert_matvec_close, expect, make_case, rel_l2

pytestmark = pytest.mark.gpu

ENCODINGS = [enc.Q4_0, enc.Q5_0, enc.Q5_1, enc.Q2_K, enc.Q3_K, enc.Q5_K, enc.IQ4_NL, enc.IQ4_XS]


@pytest.fixture(scope="module")
def backend():
    b = Backend(0)
    yield b
    b.deinit()


@pytest.mark.parametrize("encoding", ENCODINGS)
def test_rows_decode_bit_for_bit(backend, encoding):
    rows, columns = 5, 1280
    w, _, m = make_case(encoding, rows, columns, 1, seed=300 + encoding)
    stride = w.size // rows
    # behind a 2-byte offset: the decoder must not assume alignment
    host = np.zeros(w.size + 2, dtype=np.uint8)
    host[2:] = w
    wb = backend.wrap(host)
    out = backend.create(columns * 4)
    for token in (0, 2, 4):
        backend.begin()
        backend.embed(wb.slice(2, w.size), m, token, out)
        backend.commit()
        want = oracle.row(encoding, w[token * stride:(token + 1) * stride], columns)
        assert np.array_equal(out.floats().view(np.uint32), want.view(np.uint32))
    backend.unwrap(host)
    backend.release(out)


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("tokens", [1, 4, 8])
def test_gemv_and_token_rows_match_oracle(backend, encoding, tokens):
    rows, columns = 77, 2304
    w, x, m = make_case(encoding, rows, columns, tokens, seed=320 + encoding + tokens)
    want, mag = expect(encoding, rows, columns, w, x)
    wb = backend.wrap(w)
    xb = backend.create(x.nbytes); xb.write(x)
    yb = backend.create(tokens * rows * 4)
    backend.begin()
    if tokens == 1:
        backend.matvec(wb, m, xb, yb)
    else:
        backend.matvec_rows(wb, m, xb, columns, yb, rows, tokens)
    backend.commit()
    got = yb.floats().reshape(tokens, rows)
    for t in range(tokens):
        assert_matvec_close(got[t], want[t], mag[t], f"enc {encoding} token {t}")
    backend.unwrap(w)
    for buf in (xb, yb):
        backend.release(buf)


@pytest.mark.parametrize("encoding", ENCODINGS)
def test_prefill_tiles_match_oracle(backend, encoding):
    rows, columns, tokens = 136, 1280, 37
    w = synth.matrix(encoding, rows, columns, seed=340 + encoding)
    x = synth.activations(tokens, columns, seed=341 + encoding)
    m = Matrix(encoding, rows, columns, w.size)
    padded = Backend.matmul_padded(tokens)
    wb = backend.wrap(w)
    xb = backend.create(padded * columns * 4)
    yb = backend.create(padded * rows * 4)
    xin = np.zeros((padded, columns), dtype=np.float32)
    xin[:tokens] = x
    xb.write(xin)
    backend.begin()
    backend.matmul(wb, m, xb, columns, yb, rows, tokens, in_dtype=enc.F32)
    backend.commit()
    got = yb.floats().reshape(padded, rows)[:tokens]
    # the prefill path multiplies bf16(x) by bf16(w) and accumulates in F32: 2e-2 covers both roundings
    for t in (0, 17, 36):
        want = oracle.matvec(encoding, rows, columns, w, x[t])
        assert np.all(np.isfinite(got[t]))
        assert rel_l2(got[t], want) <= 2e-2, (encoding, t)
    backend.unwrap(w)
    for buf in (xb, yb):
        backend.release(buf)
