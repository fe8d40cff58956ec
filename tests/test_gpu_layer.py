"""GPU parity of the operators a decode layer is built from, at the shapes of the 27B-shape stack:
merged projections (`matvecSegments`: plain, SiLU pair, GELU pair; inference/metal-check.zig:4596-4680
checks the reference's merged matvec the same way), the verify batch on the planar forms at both
config-1 shapes, and one whole layer (QKV -> O -> gate/up -> down) for one and eight tokens against
the CPU oracle."""
import numpy as np
import pytest

import oracle
from nuclis_b200 import Backend, Matrix, NuclisError, Segment, SegmentMode, encoding as enc, synth
from parity import assert_matvec_close, expect, make_case, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    b = Backend(0)
    yield b
    b.deinit()


def upload(b, data):
    buf = b.create(data.nbytes)
    buf.write(data)
    return buf


def weights_from(b, w, m, prepare):
    """The GGUF bytes `w` on the device (planar when `prepare`) and the descriptor to use with them."""
    wb = upload(b, w)
    if prepare:
        pb, m = b.prepare(wb, m)
        b.release(wb)
        wb = pb
    return wb, m, w


def weights(b, encoding, rows, columns, seed, prepare):
    """A matrix on the device (planar when `prepare`), its descriptor and its GGUF bytes on the host."""
    w = synth.matrix(encoding, rows, columns, seed)
    m = Matrix(encoding, rows, columns, w.size)
    wb = upload(b, w)
    if prepare:
        pb, m = b.prepare(wb, m)
        b.release(wb)
        wb = pb
    return wb, m, w


EVERY = [(enc.Q4_K, False), (enc.Q5_K, False), (enc.Q6_K, True), (enc.Q8_0, True), (enc.Q4_0, True), (enc.Q5_0, True), (enc.Q5_1, True),
         (enc.IQ4_NL, True), (enc.IQ4_XS, True), (enc.Q2_K, True), (enc.Q3_K, True)]


@pytest.mark.parametrize("encoding,prepare", EVERY)
def test_plain_segments_share_one_input(backend, encoding, prepare):
    b = backend
    columns, rows = 1280, [512, 256, 272]
    x = synth.activations(1, columns, 7)[0]
    xb = upload(b, x)
    segs, wants, bufs = [], [], [xb]
    for i, r in enumerate(rows):
        wb, m, w = weights(b, encoding, r, columns, 20 + i, prepare)
        out = b.create(r * 4)
        segs.append(Segment(wb, m, out))
        wants.append((oracle.matvec(encoding, r, columns, w, x), oracle.matvec_abs(encoding, r, columns, w, x)))
        bufs += [wb, out]
    b.begin()
    b.matvec_segments(segs, xb, SegmentMode.plain)
    b.commit()
    for seg, (want, mag) in zip(segs, wants):
        assert_matvec_close(seg.output.floats()[: seg.matrix.rows], want, mag, f"segment of {seg.matrix.rows} rows, enc {encoding}")
    for buf in bufs:
        b.release(buf)


@pytest.mark.parametrize("mode", [SegmentMode.silu_mul_pair, SegmentMode.gelu_mul_pair])
@pytest.mark.parametrize("shape", [(1056, 1280), (17408, 5120)])
def test_gate_up_pair_writes_the_activated_product(backend, mode, shape):
    b = backend
    rows, columns = shape
    x = synth.activations(1, columns, 11)[0]
    xb = upload(b, x)
    gb, m, wg = weights(b, enc.Q4_K, rows, columns, 31, False)
    ub, _, wu = weights(b, enc.Q4_K, rows, columns, 32, False)
    out = b.create(rows * 4)
    b.begin()
    b.matvec_segments([Segment(gb, m, out), Segment(ub, m, out)], xb, mode)
    b.commit()
    g = oracle.matvec(enc.Q4_K, rows, columns, wg, x)
    u = oracle.matvec(enc.Q4_K, rows, columns, wu, x)
    act = oracle.silu(g) if mode == SegmentMode.silu_mul_pair else oracle.gelu(g)
    want = act.astype(np.float64) * u.astype(np.float64)
    got = out.floats()[:rows]
    # the product of two sums each within the matvec bound: compare on the whole vector
    assert rel_l2(got, want) <= 1e-5
    for buf in (xb, gb, ub, out):
        b.release(buf)


@pytest.mark.parametrize("encoding,prepare", EVERY[1:])
def test_gate_up_pair_on_the_other_encodings(backend, encoding, prepare):
    b = backend
    rows, columns = 1056, 1280
    x = synth.activations(1, columns, 12)[0]
    xb = upload(b, x)
    gb, m, wg = weights(b, encoding, rows, columns, 33, prepare)
    ub, _, wu = weights(b, encoding, rows, columns, 34, prepare)
    out = b.create(rows * 4)
    b.begin()
    b.matvec_segments([Segment(gb, m, out), Segment(ub, m, out)], xb, SegmentMode.silu_mul_pair)
    b.commit()
    g = oracle.matvec(encoding, rows, columns, wg, x)
    u = oracle.matvec(encoding, rows, columns, wu, x)
    want = oracle.silu(g).astype(np.float64) * u.astype(np.float64)
    assert rel_l2(out.floats()[:rows], want) <= 1e-5
    for buf in (xb, gb, ub, out):
        b.release(buf)


def test_merge_is_declined_before_anything_is_recorded(backend):
    b = backend
    columns = 1280
    xb = upload(b, synth.activations(1, columns, 3)[0])
    a, ma, _ = weights(b, enc.Q4_K, 256, columns, 41, False)
    c, mc, _ = weights(b, enc.Q6_K, 256, columns, 42, True)
    o1, o2 = b.create(256 * 4), b.create(256 * 4)
    b.begin()
    try:
        with pytest.raises(NuclisError) as e:
            b.matvec_segments([Segment(a, ma, o1), Segment(c, mc, o2)], xb, SegmentMode.plain)  # two encodings
        assert e.value.status == 5  # MergeDeclined: the caller falls back to separate matvecs
        with pytest.raises(NuclisError):
            b.matvec_segments([Segment(a, ma, o1), Segment(a, ma, o2)], xb, SegmentMode.silu_mul_pair)  # a pair names one output
    finally:
        b.discard()
    for buf in (xb, a, c, o1, o2):
        b.release(buf)


@pytest.mark.parametrize("encoding", [enc.Q6_K, enc.Q8_0])
@pytest.mark.parametrize("shape", [(17408, 5120), (5120, 17408)])
@pytest.mark.parametrize("tokens", [2, 4, 8])
def test_verify_batch_on_the_planar_forms(backend, encoding, shape, tokens):
    b = backend
    rows, columns = shape
    w, x, m = make_case(encoding, rows, columns, tokens, seed=300 + tokens)
    want, mag = expect(encoding, rows, columns, w, x)
    wb = upload(b, w)
    pb, pm = b.prepare(wb, m)
    xb = upload(b, x)
    yb = b.create(tokens * rows * 4)
    b.begin()
    b.matvec_rows(pb, pm, xb, columns, yb, rows, tokens)
    b.commit()
    assert_matvec_close(yb.floats().reshape(tokens, rows), want, mag, f"planar enc {encoding} {rows}x{columns} tokens {tokens}")
    for buf in (wb, pb, xb, yb):
        b.release(buf)


@pytest.mark.parametrize("tokens", [1, 8])
def test_one_layer_of_the_stack_matches_the_oracle(backend, tokens):
    """QKV (three merged projections) -> O -> gate/up -> down at the 27B shapes, the way the benchmark records a layer."""
    b = backend
    hidden, kv, ffn = 5120, 1024, 17408
    h = synth.activations(tokens, hidden, 5)
    wq, mq, hq = weights(b, enc.Q4_K, hidden, hidden, 51, False)
    wk, mk, hk = weights(b, enc.Q4_K, kv, hidden, 52, False)
    wv, mv, hv = weights(b, enc.Q4_K, kv, hidden, 53, False)
    wo, mo, ho = weights(b, enc.Q4_K, hidden, hidden, 54, False)
    wg, mg, hg = weights(b, enc.Q4_K, ffn, hidden, 55, False)
    wu, mu, hu = weights(b, enc.Q4_K, ffn, hidden, 56, False)
    wd, md, hd = weights(b, enc.Q6_K, hidden, ffn, 57, True)
    hb = upload(b, h)
    q = b.create(tokens * hidden * 4); k = b.create(tokens * kv * 4); v = b.create(tokens * kv * 4)
    o = b.create(tokens * hidden * 4); g = b.create(tokens * ffn * 4); u = b.create(tokens * ffn * 4); d = b.create(tokens * hidden * 4)
    b.begin()
    if tokens == 1:
        b.matvec_segments([Segment(wq, mq, q), Segment(wk, mk, k), Segment(wv, mv, v)], hb, SegmentMode.plain)
        b.matvec(wo, mo, q, o)
        b.matvec_segments([Segment(wg, mg, g), Segment(wu, mg, g)], o, SegmentMode.silu_mul_pair)
        b.matvec(wd, md, g, d)
    else:
        b.matvec_rows(wq, mq, hb, hidden, q, hidden, tokens)
        b.matvec_rows(wk, mk, hb, hidden, k, kv, tokens)
        b.matvec_rows(wo, mo, q, hidden, o, hidden, tokens)
        b.matvec_rows(wg, mg, o, hidden, g, ffn, tokens)
        b.matvec_rows(wu, mu, o, hidden, u, ffn, tokens)
        b.silu_mul(g, u, tokens * ffn)
        b.matvec_rows(wd, md, g, ffn, d, hidden, tokens)
    b.commit()
    got = d.floats()[: tokens * hidden].reshape(tokens, hidden)
    for t in range(tokens):
        qq = oracle.matvec(enc.Q4_K, hidden, hidden, hq, h[t])
        oo = oracle.matvec(enc.Q4_K, hidden, hidden, ho, qq)
        act = (oracle.silu(oracle.matvec(enc.Q4_K, ffn, hidden, hg, oo)) * oracle.matvec(enc.Q4_K, ffn, hidden, hu, oo)).astype(np.float32)
        want = oracle.matvec(enc.Q6_K, hidden, ffn, hd, act)
        # four chained products: each within 1e-5, their errors add up
        assert rel_l2(got[t], want) <= 4e-5, (t, rel_l2(got[t], want))
    if tokens == 1:
        assert_matvec_close(k.floats()[:kv], oracle.matvec(enc.Q4_K, kv, hidden, hk, h[0]), oracle.matvec_abs(enc.Q4_K, kv, hidden, hk, h[0]), "K rows")
        assert_matvec_close(v.floats()[:kv], oracle.matvec(enc.Q4_K, kv, hidden, hv, h[0]), oracle.matvec_abs(enc.Q4_K, kv, hidden, hv, h[0]), "V rows")
    for buf in (wq, wk, wv, wo, wg, wu, wd, hb, q, k, v, o, g, u, d):
        b.release(buf)


@pytest.mark.parametrize("name", ["silu_mul", "gelu_mul"])
@pytest.mark.parametrize("count", [1, 33, 704, 17408])
def test_gate_activations_match_the_oracle(backend, name, count):
    """`siluMul` / `geluMul` alone (ops/rowwise.zig:209-233): gate[i] = act(gate[i]) * up[i] in place, against the
    CPU forms (vector.zig:94-98, 178-181: evaluated in F64, rounded once). F32 `exp` / `tanh` on the device:
    1 + tanh(u) cancels for negative gates, so the bound is absolute in the gate's size:
    |error| <= 1e-6 * max(1, |gate|) * |up| + 1e-7; large |gate| values take the saturated branches."""
    b = backend
    rng = np.random.default_rng(count)
    gate = (rng.standard_normal(count) * 4).astype(np.float32)
    gate[:1] = 0.0
    if count > 8:
        gate[1:7] = [30.0, -30.0, 88.0, -88.0, 1e-8, -1e-8]
    up = rng.standard_normal(count).astype(np.float32)
    gb, ub = upload(b, gate), upload(b, up)
    b.begin()
    getattr(b, name)(gb, ub, count)
    b.commit()
    got = gb.floats()
    act = oracle.silu(gate) if name == "silu_mul" else oracle.gelu(gate)
    want = act.astype(np.float64) * up.astype(np.float64)
    assert np.all(np.isfinite(got))
    bound = 1e-6 * np.maximum(1.0, np.abs(gate)) * np.abs(up) + 1e-7
    assert np.all(np.abs(got - want) <= bound), float(np.max(np.abs(got - want) / bound))
    assert np.array_equal(ub.floats(), up)  # `up` is only read
    b.release(gb); b.release(ub)


def test_gate_activations_refuse_bad_calls(backend):
    b = backend
    gb, ub = b.create(64), b.create(64)
    b.begin()
    with pytest.raises(NuclisError):
        b.gelu_mul(gb, ub, 17)   # 17 floats do not fit 64 bytes
    with pytest.raises(NuclisError):
        b.silu_mul(gb, ub, 0)
    b.discard()
    b.release(gb); b.release(ub)


@pytest.mark.parametrize("rows,width,pad", [(1, 5120, 0), (8, 5120, 64), (3, 2816, 0), (2, 17408, 0), (4, 100, 3), (1, 16, 0)])
def test_norms_around_the_projections_match_the_oracle(backend, rows, width, pad):
    """`rmsNorm`, `addRmsNorm` and `add` (ops/rowwise.zig:37-51, 76-93, 199-202) against the CPU forms (vector.zig:53-64:
    F64 sum of squares, one division per element) times the weight: within 4e-6 relative + 1e-7. `addRmsNorm` also
    leaves residual + input in the residual, bit for bit what `add` gives; rows wider than a thread keeps in
    registers (17408), odd widths and padded strides take the other paths of the kernel."""
    b = backend
    rng = np.random.default_rng(rows * 1000 + width)
    stride = width + pad
    x = (rng.standard_normal((rows, stride)) * 3).astype(np.float32)
    s = rng.standard_normal((rows, stride)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    xb, sb, wb, yb = upload(b, x), upload(b, s), upload(b, w), b.create(rows * stride * 4)
    x2 = upload(b, x)
    b.begin()
    b.rms_norm(xb, wb, yb, rows, width, stride, stride)
    b.commit()
    got = yb.floats().reshape(rows, stride)[:, :width]
    for r in range(rows):
        want = oracle.rms_norm(x[r, :width]).astype(np.float64) * w
        assert np.all(np.abs(got[r] - want) <= 4e-6 * np.abs(want) + 1e-7), (r, float(np.max(np.abs(got[r] - want))))
    b.begin()
    b.add_rms_norm(xb, sb, wb, yb, rows, width, stride, stride)
    b.add(x2, sb, rows * stride)
    b.commit()
    got = yb.floats().reshape(rows, stride)[:, :width]
    summed = xb.floats().reshape(rows, stride)
    assert np.array_equal(summed[:, :width], (x + s)[:, :width]) and np.array_equal(x2.floats().reshape(rows, stride), x + s)
    assert np.array_equal(summed[:, width:], x[:, width:])          # the padding between rows is not touched
    for r in range(rows):
        want = oracle.rms_norm((x + s)[r, :width]).astype(np.float64) * w
        assert np.all(np.abs(got[r] - want) <= 4e-6 * np.abs(want) + 1e-7), r
    # in place, and the refusals
    b.begin()
    b.rms_norm(xb, wb, xb, rows, width, stride, stride)
    with pytest.raises(NuclisError):
        b.rms_norm(xb, wb, yb, rows, width, width - 1 if width > 1 else 0, stride)
    with pytest.raises(NuclisError):
        b.add_rms_norm(xb, xb, wb, yb, rows, width, stride, stride)   # input is the residual
    with pytest.raises(NuclisError):
        b.rms_norm(xb, wb, yb, rows, width, stride, stride, eps=0.0)
    b.commit()
    inplace = xb.floats().reshape(rows, stride)[:, :width]
    assert np.array_equal(inplace, got)
    for buf in (xb, sb, wb, yb, x2):
        b.release(buf)


@pytest.mark.parametrize("encoding,prepare", [(enc.Q4_K, False), (enc.Q5_K, False), (enc.Q6_K, True), (enc.Q8_0, True), (enc.Q5_0, True)])
@pytest.mark.parametrize("shape", [(1056, 1280), (17408, 5120), (2048, 17408)])   # 17408 columns: K cut into slices, the rows read in a pass of their own
@pytest.mark.parametrize("with_add", [True, False])
def test_add_rms_norm_folded_into_the_projections(backend, encoding, prepare, shape, with_add):
    """`matvec_segments_normed`: `addRmsNorm` (ops/rowwise.zig:76-93) and the gate/up pair on its output
    (inference/src/models/qwen35_metal.zig:635-640) as one launch. The product against the oracle on the CPU norm's
    output (vector.zig:53-64: F64 sum of squares); residual + input bit for bit in the second residual buffer; and the
    two separate operators agree with the one launch to the accuracy of the fixed-point staging."""
    b = backend
    rows, columns = shape
    rng = np.random.default_rng(rows + columns)
    res = (rng.standard_normal(columns) * 3).astype(np.float32)
    inp = rng.standard_normal(columns).astype(np.float32)
    wn = (1.0 + 0.1 * rng.standard_normal(columns)).astype(np.float32)
    rb, ib, wnb, ob, yb = upload(b, res), upload(b, inp), upload(b, wn), b.create(columns * 4), b.create(columns * 4)
    gb, m, wg = weights(b, encoding, rows, columns, 51, prepare)
    ub, _, wu = weights(b, encoding, rows, columns, 52, prepare)
    out, out2 = b.create(rows * 4), b.create(rows * 4)
    ob.write(np.full(columns, np.nan, dtype=np.float32))
    before = b.launch_count
    b.begin()
    b.matvec_segments_normed([Segment(gb, m, out), Segment(ub, m, out)], rb, wnb, input=ib if with_add else None, residual_out=ob if with_add else None,
                             mode=SegmentMode.silu_mul_pair)
    b.commit()
    assert b.launch_count - before == 1
    summed = res + inp if with_add else res
    if with_add:
        assert np.array_equal(ob.floats(), summed)
    assert np.array_equal(rb.floats(), res)          # the residual that came in is not touched
    xn = (oracle.rms_norm(summed).astype(np.float64) * wn).astype(np.float32)
    g = oracle.matvec(encoding, rows, columns, wg, xn)
    u = oracle.matvec(encoding, rows, columns, wu, xn)
    want = oracle.silu(g).astype(np.float64) * u.astype(np.float64)
    got = out.floats()[:rows]
    assert rel_l2(got, want) <= 1e-5
    # the two operators on their own
    b.begin()
    if with_add:
        b.add_rms_norm(rb, ib, wnb, yb, 1, columns)
    else:
        b.rms_norm(rb, wnb, yb, 1, columns)
    b.matvec_segments([Segment(gb, m, out2), Segment(ub, m, out2)], yb, SegmentMode.silu_mul_pair)
    b.commit()
    assert rel_l2(got, out2.floats()[:rows].astype(np.float64)) <= 2e-6
    for buf in (rb, ib, wnb, ob, yb, gb, ub, out, out2):
        b.release(buf)


def test_folded_norm_contract(backend):
    b = backend
    columns, rows = 1280, 256
    x = synth.activations(1, columns, 3)[0]
    rb, ib, wnb, ob = upload(b, x), upload(b, x), upload(b, np.ones(columns, dtype=np.float32)), b.create(columns * 4)
    a, ma, _ = weights(b, enc.Q4_K, rows, columns, 61, False)
    c, mc, _ = weights(b, enc.Q6_K, rows, columns, 62, False)   # GGUF-form Q6_K: not served by the specialized kernel
    o1 = b.create(rows * 4)
    b.begin()
    try:
        with pytest.raises(NuclisError):
            b.matvec_segments_normed([Segment(a, ma, o1)], rb, wnb, input=ib, residual_out=rb)        # the sum would land on the residual being read
        with pytest.raises(NuclisError):
            b.matvec_segments_normed([Segment(a, ma, o1)], rb, wnb, input=ib)                         # input without a place for the sum
        with pytest.raises(NuclisError):
            b.matvec_segments_normed([Segment(a, ma, o1)], rb, wnb, input=ib, residual_out=ob, eps=0.0)
        with pytest.raises(NuclisError) as e:
            b.matvec_segments_normed([Segment(c, mc, o1)], rb, wnb, input=ib, residual_out=ob)
        assert e.value.status == 5   # MergeDeclined: the caller runs addRmsNorm and the matvec
    finally:
        b.discard()
    for buf in (rb, ib, wnb, ob, a, c, o1):
        b.release(buf)


@pytest.mark.parametrize("encoding,prepare", [(enc.Q4_K, False), (enc.Q6_K, True), (enc.Q8_0, True), (enc.Q5_1, True), (enc.Q6_K, False)])
@pytest.mark.parametrize("shape", [(80, 1280), (5120, 17408)])
@pytest.mark.parametrize("in_place", [True, False])
def test_residual_add_folded_into_the_projection(backend, encoding, prepare, shape, in_place):
    """`matvec_add`: the down (or O) projection and the residual `add` behind it (inference/src/models/qwen35_metal.zig:640)
    as one launch on the specialized kernels (5120 x 17408 runs split over K: the last block to arrive for a unit adds),
    two on the generic one (GGUF-form Q6_K here). residual + W x against the oracle within the matvec bound."""
    b = backend
    rows, columns = shape
    w, x, m = make_case(encoding, rows, columns, 1, seed=77 + rows)
    want, mag = expect(encoding, rows, columns, w, x)
    res = (np.random.default_rng(rows).standard_normal(rows) * 0.1).astype(np.float32)
    wb, mm, _ = weights_from(b, w, m, prepare)
    xb, rb = upload(b, x[0]), upload(b, res)
    ob = rb if in_place else b.create(rows * 4)
    fast = prepare or encoding == enc.Q4_K
    before = b.launch_count
    b.begin()
    b.matvec_add(wb, mm, xb, rb, ob)
    b.commit()
    assert b.launch_count - before == (1 if fast and rows % 16 == 0 else 2)
    got = ob.floats()[:rows]
    assert_matvec_close(got - res, want[0], mag[0] + np.abs(res), f"matvec_add enc {encoding} {shape}")
    if not in_place:
        assert np.array_equal(rb.floats(), res)
        b.begin()
        with pytest.raises(NuclisError):
            b.matvec_add(wb, mm, xb, rb, rb.slice(4, rb.len - 4))   # a shifted overlap of residual and output
        b.discard()
    for buf in {id(v): v for v in (wb, xb, rb, ob)}.values():
        b.release(buf)


def test_pre_norm_layer_on_the_folded_operators_matches_the_oracle(backend):
    """One layer of the stack as a pre-norm decoder runs it (`Stack.record_with_norms`): x += O(Q(norm(x))), then
    x += down(silu(gate(norm(x))) * up(norm(x))), four launches; against the CPU oracle's norms, matvecs and adds."""
    from nuclis_b200.shard import LayerShapes
    from nuclis_b200.stack import Stack, make_stack
    b = backend
    shapes = LayerShapes(hidden=1280, ffn=2816, kv=256)
    st = make_stack(b, 1, 1, shapes=shapes, seed=5, prepare=False)
    w = st.layers[0]
    host = {k: getattr(w, k).read() for k in ("qkv", "o", "gate", "up", "down")}
    st.prepare_layer(w)
    st.enable_norms(3)
    before = b.launch_count
    b.begin()
    assert st.record() == 4
    b.commit()
    assert b.launch_count - before == 4
    l = st.local
    x = st.residual0.copy()
    xn = (oracle.rms_norm(x).astype(np.float64) * st.norm_attn_host).astype(np.float32)
    qkv = oracle.matvec(shapes.qkv_encoding, l.qkv_rows, shapes.hidden, host["qkv"], xn)
    x = x + oracle.matvec(shapes.o_encoding, shapes.hidden, l.q_rows, host["o"], qkv[: l.q_rows])
    xn = (oracle.rms_norm(x).astype(np.float64) * st.norm_ffn_host).astype(np.float32)
    g = oracle.matvec(shapes.gate_up_encoding, l.ffn_rows, shapes.hidden, host["gate"], xn)
    u = oracle.matvec(shapes.gate_up_encoding, l.ffn_rows, shapes.hidden, host["up"], xn)
    act = (oracle.silu(g).astype(np.float64) * u).astype(np.float32)
    x = x + oracle.matvec(shapes.down_encoding, shapes.hidden, l.ffn_rows, host["down"], act)
    assert rel_l2(st.residual.floats(), x) <= 1e-5
