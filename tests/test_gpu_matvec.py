"""GPU parity of the decode GEMV and the 2..8-row multi-row GEMV against the CPU oracle.

Mirrors the reference's GPU kernel checks (inference/metal-check.zig): every golden row
decoded on the device bit for bit (:4228-4236), one-hot inputs selecting golden columns
(:4218-4226), randomized wide rows for the specialized and the forced-generic kernels
(:3934-3989), multi-row batches (:4540-4594), and contract violations refused before
anything is recorded (:4470-4480). All device calls go through the C ABI.
"""
import numpy as np
import pytest

import oracle
from nuclis_b200 import Backend, Matrix, NuclisError, encoding as enc
from parity import assert_matvec_close, expect, make_case, tiled_fixture_matrix

pytestmark = pytest.mark.gpu

ENCODINGS = [enc.Q4_K, enc.Q5_K, enc.Q6_K, enc.Q8_0]


@pytest.fixture(scope="module")
def backend():
    b = Backend(0)
    yield b
    b.deinit()


def run_matvec(b, w, m, x, generic=False):
    b.generic_only = generic
    try:
        wb = b.wrap(w)
        xb = b.create(x.size * 4)
        yb = b.create(m.rows * 4)
        xb.write(x)
        yb.write(np.full(m.rows, np.nan, dtype=np.float32))  # a row the kernel skips stays NaN
        b.begin()
        b.matvec(wb, m, xb, yb)
        b.commit()
        out = yb.floats()
        b.unwrap(w)
        b.release(xb)
        b.release(yb)
        return out
    finally:
        b.generic_only = False


def run_rows(b, w, m, x, generic=False, in_stride=None, out_stride=None):
    tokens = x.shape[0]
    in_stride = in_stride or m.columns
    out_stride = out_stride or m.rows
    b.generic_only = generic
    try:
        wb = b.wrap(w)
        xb = b.create(tokens * in_stride * 4)
        yb = b.create(tokens * out_stride * 4)
        xin = np.zeros((tokens, in_stride), dtype=np.float32)
        xin[:, : m.columns] = x
        xb.write(xin)
        yb.write(np.full(tokens * out_stride, np.nan, dtype=np.float32))
        b.begin()
        b.matvec_rows(wb, m, xb, in_stride, yb, out_stride, tokens)
        b.commit()
        out = yb.floats().reshape(tokens, out_stride)[:, : m.rows]
        b.unwrap(w)
        b.release(xb)
        b.release(yb)
        return out
    finally:
        b.generic_only = False


def test_embed_decodes_golden_rows_bit_for_bit(backend, golden_rows):
    for r in golden_rows:
        n = r["values"].size
        m = Matrix(r["encoding"], 1, n, r["bytes"].size)
        # behind a 2-byte offset: the decoder must not assume alignment
        host = np.zeros(r["bytes"].size + 2, dtype=np.uint8)
        host[2:] = r["bytes"]
        wb = backend.wrap(host)
        out = backend.create(n * 4)
        backend.begin()
        backend.embed(wb.slice(2, r["bytes"].size), m, 0, out)
        backend.commit()
        got = out.floats()
        assert np.array_equal(got.view(np.uint32), r["values"].view(np.uint32)), r["name"]
        backend.unwrap(host)
        backend.release(out)


@pytest.mark.parametrize("encoding", ENCODINGS)
def test_embed_random_rows_bit_for_bit(backend, encoding):
    rows, columns = 7, 1280
    w, _, m = make_case(encoding, rows, columns, 1, seed=100 + encoding)
    wb = backend.wrap(w)
    out = backend.create(columns * 4)
    stride = w.size // rows
    for token in (0, 3, 6):
        backend.begin()
        backend.embed(wb, m, token, out)
        backend.commit()
        want = oracle.row(encoding, w[token * stride:(token + 1) * stride], columns)
        assert np.array_equal(out.floats().view(np.uint32), want.view(np.uint32))
    backend.unwrap(w)
    backend.release(out)


@pytest.mark.parametrize("generic", [False, True])
def test_one_hot_inputs_select_golden_columns(backend, golden_rows, generic):
    for r in golden_rows:
        _, columns, _ = enc.layout(r["encoding"])
        rows = r["values"].size // columns
        m = Matrix(r["encoding"], rows, columns, r["bytes"].size)
        for column in (0, columns // 2 + 1, columns - 1):
            x = np.zeros((1, columns), dtype=np.float32)
            x[0, column] = 1
            got = run_matvec(backend, r["bytes"], m, x, generic=generic)
            want = r["values"].reshape(rows, columns)[:, column]
            assert np.allclose(got, want, rtol=1e-5, atol=0), (r["name"], column)


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("columns", [256, 1280, 5120])
@pytest.mark.parametrize("generic", [False, True])
def test_wide_rows_of_tiled_golden_blocks(backend, golden_rows, encoding, columns, generic):
    row = next(r for r in golden_rows if r["encoding"] == encoding)
    rows = 35
    w = tiled_fixture_matrix(row, rows, columns)
    m = Matrix(encoding, rows, columns, w.size)
    x = np.random.default_rng(columns).standard_normal((1, columns), dtype=np.float32)
    want, mag = expect(encoding, rows, columns, w, x)
    got = run_matvec(backend, w, m, x, generic=generic)
    # golden blocks hold extreme scales (largest finite f16): the element formula is the right scale
    assert_matvec_close(got, want[0], mag[0], f"enc {encoding} cols {columns} generic {generic}", rel=1e-4)


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("shape", [(80, 1280), (4096, 4096), (17408, 5120), (5120, 17408)])
def test_matvec_matches_oracle(backend, encoding, shape):
    rows, columns = shape
    w, x, m = make_case(encoding, rows, columns, 1, seed=7 + encoding)
    want, mag = expect(encoding, rows, columns, w, x)
    got = run_matvec(backend, w, m, x)
    assert_matvec_close(got, want[0], mag[0], f"enc {encoding} {shape}")


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("tokens", [2, 3, 4, 5, 8])
def test_matvec_rows_matches_oracle(backend, encoding, tokens):
    rows, columns = 1056, 2304
    w, x, m = make_case(encoding, rows, columns, tokens, seed=31 + tokens)
    want, mag = expect(encoding, rows, columns, w, x)
    got = run_rows(backend, w, m, x, in_stride=columns + 64, out_stride=rows + 8)
    assert_matvec_close(got, want, mag, f"enc {encoding} tokens {tokens}")
    got = run_rows(backend, w, m, x, generic=True)
    assert_matvec_close(got, want, mag, f"generic enc {encoding} tokens {tokens}")


@pytest.mark.parametrize("encoding", ENCODINGS)
@pytest.mark.parametrize("shape", [(17408, 5120), (5120, 17408)])
@pytest.mark.parametrize("tokens", [2, 4, 8])
def test_verify_batch_shapes_match_oracle(backend, encoding, shape, tokens):
    rows, columns = shape
    w, x, m = make_case(encoding, rows, columns, tokens, seed=500 + tokens)
    # the oracle costs ~0.2 s per token row at this size: check two of the token rows in full
    got = run_rows(backend, w, m, x)
    for t in (0, tokens - 1):
        want = oracle.matvec(encoding, rows, columns, w, x[t])
        mag = oracle.matvec_abs(encoding, rows, columns, w, x[t])
        assert_matvec_close(got[t], want, mag, f"enc {encoding} {shape} tokens {tokens} row {t}")


def test_scale_extremes_do_not_overflow(backend):
    # activations far outside fp16 range: the kernel rescales per slice, the CPU path does not care
    rows, columns = 64, 1024
    w, x, m = make_case(enc.Q4_K, rows, columns, 1, seed=3)
    for factor in (1e-20, 1e-6, 1e6, 1e20):
        xs = (x * np.float32(factor)).astype(np.float32)
        want, mag = expect(enc.Q4_K, rows, columns, w, xs)
        got = run_matvec(backend, w, m, xs)
        assert np.all(np.isfinite(got))
        assert np.max(np.abs(got - want[0]) / (4e-6 * mag[0] + 1e-30)) <= 1.0, factor


def test_contract_violations_are_refused_before_recording(backend):
    rows, columns = 32, 512
    w, x, m = make_case(enc.Q4_K, rows, columns, 1, seed=1)
    wb = backend.wrap(w)
    xb = backend.create(columns * 4)
    yb = backend.create(rows * 4)
    sentinel = np.full(rows, 123, dtype=np.float32)
    yb.write(sentinel)

    def refused(name, fn):
        backend.begin()
        with pytest.raises(NuclisError) as e:
            fn()
        assert e.value.name == name, e.value
        backend.commit()  # an empty recording: nothing may have run

    refused("InvalidShape", lambda: backend.matvec(wb, Matrix(enc.Q4_K, 0, columns, w.size), xb, yb))
    refused("InvalidShape", lambda: backend.matvec(wb, Matrix(enc.Q4_K, rows, 0, w.size), xb, yb))
    refused("InvalidShape", lambda: backend.matvec(wb, m, xb.slice(0, columns * 4 - 4), yb))
    refused("InvalidShape", lambda: backend.matvec(wb, m, xb, yb.slice(0, rows * 4 - 4)))
    refused("InvalidShape", lambda: backend.matvec(wb.slice(0, w.size - 1), m, xb, yb))
    refused("InvalidByteLength", lambda: backend.matvec(wb, Matrix(enc.Q4_K, rows, columns, w.size - rows), xb, yb))
    refused("InvalidRowLength", lambda: backend.matvec(wb, Matrix(enc.Q6_K, 3, 704, 3 * 210 * 3), xb, yb))
    refused("UnsupportedTensorEncoding", lambda: backend.matvec(wb, Matrix(999, rows, columns, w.size), xb, yb))
    refused("InvalidShape", lambda: backend.matvec_rows(wb, m, xb, columns, yb, rows, 1))
    refused("InvalidShape", lambda: backend.matvec_rows(wb, m, xb, columns, yb, rows, 9))
    assert np.array_equal(yb.floats(), sentinel)
    # outside a recording every operator is refused
    with pytest.raises(NuclisError) as e:
        backend.matvec(wb, m, xb, yb)
    assert e.value.name == "NotRecording"
    backend.unwrap(w)
    backend.release(xb)
    backend.release(yb)


def test_discard_drops_the_recording(backend):
    rows, columns = 32, 512
    w, x, m = make_case(enc.Q4_K, rows, columns, 1, seed=2)
    wb = backend.wrap(w)
    xb = backend.create(columns * 4)
    yb = backend.create(rows * 4)
    xb.write(x)
    sentinel = np.full(rows, 7, dtype=np.float32)
    yb.write(sentinel)
    backend.begin()
    backend.matvec(wb, m, xb, yb)
    backend.discard()
    assert np.array_equal(yb.floats(), sentinel)
    with pytest.raises(NuclisError):
        backend.commit()
    backend.begin()  # and the backend can begin again
    backend.matvec(wb, m, xb, yb)
    backend.commit()
    assert not np.array_equal(yb.floats(), sentinel)
    backend.unwrap(w)
    backend.release(xb)
    backend.release(yb)


def test_wrap_caches_by_address_and_ids_are_not_reused(backend):
    a = np.arange(4096, dtype=np.uint8)
    first = backend.wrap(a)
    again = backend.wrap(a)
    assert first.id == again.id
    with pytest.raises(NuclisError):
        backend.wrap(a[:100])  # same start address at another length
    backend.unwrap(a)
    fresh = backend.create(16)
    assert fresh.id != first.id
    with pytest.raises(NuclisError):
        first.read()
    backend.release(fresh)


# ---- the planar form of nu_cuda_matrix_prepare (Q6_K) ---------------------------------------------

PLANAR = {enc.Q6_K: 1, enc.Q8_0: 2, enc.Q5_0: 3, enc.Q5_1: 4, enc.Q4_0: 5, enc.IQ4_NL: 5, enc.IQ4_XS: 6, enc.Q2_K: 7, enc.Q3_K: 8}
PREPARED = [enc.Q6_K, enc.Q8_0, enc.Q5_0, enc.Q5_1, enc.Q4_0, enc.IQ4_NL, enc.IQ4_XS, enc.Q2_K, enc.Q3_K]


@pytest.mark.parametrize("encoding", PREPARED)
def test_prepared_form_decodes_bit_for_bit(backend, golden_rows, encoding):
    # golden blocks tiled into 16 rows, then random rows: every row of the prepared form decodes to
    # the bits the CPU decoder gives for the GGUF form
    row = next(r for r in golden_rows if r["encoding"] == encoding)
    for w, rows, columns in [(tiled_fixture_matrix(row, 16, 1280), 16, 1280), (make_case(encoding, 48, 2304, 1, seed=77)[0], 48, 2304)]:
        m = Matrix(encoding, rows, columns, w.size)
        wb = backend.wrap(w)
        pb, pm = backend.prepare(wb, m)
        assert pm.layout == PLANAR[encoding] and pm.bytes == m.bytes
        out = backend.create(columns * 4)
        stride = w.size // rows
        for token in (0, 1, rows // 2, rows - 1):
            backend.begin()
            backend.embed(pb, pm, token, out)
            backend.commit()
            want = oracle.row(encoding, w[token * stride:(token + 1) * stride], columns)
            assert np.array_equal(out.floats().view(np.uint32), want.view(np.uint32)), (rows, token)
        backend.unwrap(w)
        backend.release(pb)
        backend.release(out)


@pytest.mark.parametrize("encoding", PREPARED)
def test_prepare_writes_the_bytes_of_the_host_mirror(backend, encoding):
    # the device's re-layout against nuclis_b200.planar (numpy): the same bytes, so a loader may re-lay on either side
    from nuclis_b200 import planar
    rows, columns = 48, 1280
    w, _, m = make_case(encoding, rows, columns, 1, seed=123)
    wb = backend.wrap(w)
    pb, pm = backend.prepare(wb, m)
    want, layout = planar.relay(encoding, w, rows, columns)
    assert pm.layout == layout and np.array_equal(pb.read(), want)
    backend.unwrap(w)
    backend.release(pb)


@pytest.mark.parametrize("encoding", PREPARED)
@pytest.mark.parametrize("shape", [(80, 1280), (4096, 4096), (17408, 5120), (5120, 17408)])
@pytest.mark.parametrize("generic", [False, True])
def test_prepared_matvec_matches_oracle(backend, encoding, shape, generic):
    rows, columns = shape
    w, x, m = make_case(encoding, rows, columns, 1, seed=21)
    want, mag = expect(encoding, rows, columns, w, x)
    wb = backend.wrap(w)
    pb, pm = backend.prepare(wb, m)
    xb = backend.create(columns * 4)
    yb = backend.create(rows * 4)
    xb.write(x)
    yb.write(np.full(rows, np.nan, dtype=np.float32))
    backend.generic_only = generic
    try:
        backend.begin()
        backend.matvec(pb, pm, xb, yb)
        backend.commit()
    finally:
        backend.generic_only = False
    assert_matvec_close(yb.floats(), want[0], mag[0], f"prepared enc {encoding} {shape} generic {generic}")
    backend.unwrap(w)
    for buf in (pb, xb, yb):
        backend.release(buf)


def test_prepare_contract(backend):
    w, _, m = make_case(enc.Q6_K, 20, 512, 1, seed=5)  # 20 rows: not a multiple of 16, stays in GGUF form
    wb = backend.wrap(w)
    pb, pm = backend.prepare(wb, m)
    assert pm.layout == 0 and np.array_equal(pb.read(), w)
    w4, _, m4 = make_case(enc.Q4_K, 32, 512, 1, seed=5)  # Q4_K needs no re-layout
    w4b = backend.wrap(w4)
    p4b, p4m = backend.prepare(w4b, m4)
    assert p4m.layout == 0 and np.array_equal(p4b.read(), w4)
    with pytest.raises(NuclisError):
        backend.prepare(wb, m, prepared=wb)  # overlapping
    with pytest.raises(NuclisError):
        backend.prepare(wb, Matrix(enc.Q6_K, 20, 512, w.size, layout=1))  # already prepared
    xb, yb = backend.create(512 * 4), backend.create(20 * 4)
    backend.begin()
    with pytest.raises(NuclisError) as e:
        backend.matvec(wb, Matrix(enc.Q6_K, 20, 512, w.size, layout=7), xb, yb)
    assert e.value.name == "InvalidShape"
    backend.discard()
    backend.unwrap(w)
    backend.unwrap(w4)


@pytest.mark.parametrize("encoding", PREPARED)
@pytest.mark.parametrize("tokens", [2, 3, 8])
def test_prepared_matvec_rows_match_oracle(backend, encoding, tokens):
    rows, columns = 1056, 2304
    w, x, m = make_case(encoding, rows, columns, tokens, seed=91 + tokens)
    want, mag = expect(encoding, rows, columns, w, x)
    wb = backend.wrap(w)
    pb, pm = backend.prepare(wb, m)
    xb = backend.create(x.nbytes)
    yb = backend.create(tokens * rows * 4)
    xb.write(x)
    backend.begin()
    backend.matvec_rows(pb, pm, xb, columns, yb, rows, tokens)
    backend.commit()
    assert_matvec_close(yb.floats().reshape(tokens, rows), want, mag, f"prepared rows enc {encoding} tokens {tokens}")
    backend.unwrap(w)
    for buf in (pb, xb, yb):
        backend.release(buf)
