"""GPU parity of the mixture-of-experts operators against the CPU oracle.

Follows the reference's expert checks (inference/metal-check.zig:1594-1648 router with ties,
:1711-1727 gathered matvec with poisoned unselected experts, :1760-1831 decode chain against
cpu.experts.ffn at 2e-5 * (1 + max|y|)). Shapes: the 26B-A4B-style config (128 experts, top-8,
hidden 2816, expert intermediate 704; gate_up fused as [experts][2*ff][hidden] Q4_K, down as
[experts][hidden][ff] in Q8_0, the block size a 704-wide row is stored in).
"""
import numpy as np
import pytest

import oracle
from nuclis_b200 import Backend, CombineShape, ExpertMatrix, NuclisError, encoding as enc, shard, synth
from parity import rel_l2

pytestmark = pytest.mark.gpu

EXPERTS, K, HIDDEN, FF = 128, 8, 2816, 704


@pytest.fixture(scope="module")
def backend():
    b = Backend(0)
    yield b
    b.deinit()


@pytest.fixture(scope="module")
def tensors():
    gate_up = synth.matrix(enc.Q4_K, EXPERTS * 2 * FF, HIDDEN, seed=901)
    down = synth.matrix(enc.Q8_0, EXPERTS * HIDDEN, FF, seed=902)
    return gate_up, down


def test_router_indices_exact_and_weights_close(backend):
    rng = np.random.default_rng(5)
    rows = 9
    logits = rng.standard_normal((rows, EXPERTS)).astype(np.float32)
    logits[0, 3] = logits[0, 77] = logits[0].max() + 1.0   # a tie at the top: lowest index first
    logits[1, :] = 0.25                                     # all equal
    logits[2, 5] = -800.0
    lb = backend.create(logits.nbytes)
    ib = backend.create(rows * K * 4)
    wb = backend.create(rows * K * 4)
    lb.write(logits)
    backend.begin()
    backend.route(lb, EXPERTS, K, rows, EXPERTS, ib, wb)
    backend.commit()
    idx = ib.read(np.uint32).reshape(rows, K)
    w = wb.floats().reshape(rows, K)
    for r in range(rows):
        want_idx, want_w = oracle.route(logits[r], K)
        assert np.array_equal(idx[r], want_idx), r
        assert np.max(np.abs(w[r] - want_w)) <= 1e-6, r
    with pytest.raises(NuclisError):
        backend.begin()
        try:
            backend.route(lb, EXPERTS, EXPERTS + 1, rows, EXPERTS, ib, wb)
        finally:
            backend.discard()
    for buf in (lb, ib, wb):
        backend.release(buf)


@pytest.mark.parametrize("tokens", [1, 8])
def test_expert_chain_matches_cpu_ffn(backend, tensors, tokens):
    gate_up, down = tensors
    rng = np.random.default_rng(17 + tokens)
    x = rng.standard_normal((tokens, HIDDEN)).astype(np.float32)
    logits = rng.standard_normal((tokens, EXPERTS)).astype(np.float32)
    scales = (0.5 + rng.random(EXPERTS)).astype(np.float32)
    gu_t = ExpertMatrix(enc.Q4_K, EXPERTS, 2 * FF, HIDDEN, gate_up.size)
    dn_t = ExpertMatrix(enc.Q8_0, EXPERTS, HIDDEN, FF, down.size)
    slots = tokens * K
    gub, dnb = backend.wrap(gate_up), backend.wrap(down)
    xb = backend.create(x.nbytes)
    lb = backend.create(logits.nbytes)
    sb = backend.create(scales.nbytes)
    ib = backend.create(slots * 4)
    wb = backend.create(slots * 4)
    gu_out = backend.create(slots * 2 * FF * 4)
    hid = backend.create(slots * FF * 4)
    y = backend.create(slots * HIDDEN * 4)
    out = backend.create(tokens * HIDDEN * 4)
    xb.write(x); lb.write(logits); sb.write(scales)
    backend.begin()
    backend.route(lb, EXPERTS, K, tokens, EXPERTS, ib, wb)
    # gate-up: the k slots of a token share its input row (in_group = k); one token: in_stride 0 shares the row
    backend.matvec_experts_grouped(gub, gu_t, ib, slots, xb, HIDDEN if tokens > 1 else 0, K if tokens > 1 else 1, gu_out, 2 * FF)
    backend.gelu_mul_rows(gu_out, gu_out.slice(FF * 4, gu_out.len - FF * 4), hid, FF, slots, 2 * FF, 2 * FF, FF)
    backend.matvec_experts(dnb, dn_t, ib, slots, hid, FF, y, HIDDEN)
    backend.combine_experts(y, wb, ib, sb, out, CombineShape(columns=HIDDEN, slots=K, experts=EXPERTS, in_stride=HIDDEN, out_stride=HIDDEN, rows=tokens))
    backend.commit()
    got = out.floats().reshape(tokens, HIDDEN)
    for t in range(tokens):
        idx, w = oracle.route(logits[t], K)
        want = oracle.ffn((enc.Q4_K, EXPERTS, 2 * FF, HIDDEN, gate_up), (enc.Q8_0, EXPERTS, HIDDEN, FF, down), x[t], idx, w, down_scale=scales)
        bound = 2e-5 * (1 + np.max(np.abs(want)))
        assert np.max(np.abs(got[t] - want)) <= bound, (t, np.max(np.abs(got[t] - want)), bound)
    backend.unwrap(gate_up); backend.unwrap(down)
    for buf in (xb, lb, sb, ib, wb, gu_out, hid, y, out):
        backend.release(buf)


@pytest.mark.parametrize("tokens", [1, 8])
def test_expert_parallel_partials_add_up_to_the_full_result(backend, tensors, tokens):
    """Eight ranks of 16 experts each, run one after the other on this GPU: every rank sees only its slice of
    the expert tensors and its own view of the routing (route_local); the partial outputs add up to the
    CPU oracle's full result (what the allreduce over the ranks would hold)."""
    gate_up, down = tensors
    ranks = 8
    rng = np.random.default_rng(31 + tokens)
    x = rng.standard_normal((tokens, HIDDEN)).astype(np.float32)
    logits = rng.standard_normal((tokens, EXPERTS)).astype(np.float32)
    scales = (0.5 + rng.random(EXPERTS)).astype(np.float32)
    slots = tokens * K
    gu_bytes, dn_bytes = gate_up.size // EXPERTS, down.size // EXPERTS
    xb = backend.create(x.nbytes); lb = backend.create(logits.nbytes)
    ib = backend.create(slots * 4); wb = backend.create(slots * 4)
    lib_ = backend.create(slots * 4); lwb = backend.create(slots * 4)
    gu_out = backend.create(slots * 2 * FF * 4); hid = backend.create(slots * FF * 4)
    y = backend.create(slots * HIDDEN * 4); out = backend.create(tokens * HIDDEN * 4)
    xb.write(x); lb.write(logits)
    total = np.zeros((tokens, HIDDEN), dtype=np.float64)
    owners = 0
    for r in range(ranks):
        e0, e1 = shard.expert_range(EXPERTS, ranks, r)
        n = e1 - e0
        gub = backend.create(n * gu_bytes); gub.write(gate_up[e0 * gu_bytes:e1 * gu_bytes])
        dnb = backend.create(n * dn_bytes); dnb.write(down[e0 * dn_bytes:e1 * dn_bytes])
        sb = backend.create(n * 4); sb.write(scales[e0:e1])
        gu_t = ExpertMatrix(enc.Q4_K, n, 2 * FF, HIDDEN, n * gu_bytes)
        dn_t = ExpertMatrix(enc.Q8_0, n, HIDDEN, FF, n * dn_bytes)
        backend.begin()
        backend.route(lb, EXPERTS, K, tokens, EXPERTS, ib, wb)
        backend.route_local(ib, wb, slots, e0, n, lib_, lwb)
        backend.matvec_experts_grouped(gub, gu_t, lib_, slots, xb, HIDDEN if tokens > 1 else 0, K if tokens > 1 else 1, gu_out, 2 * FF)
        backend.gelu_mul_rows(gu_out, gu_out.slice(FF * 4, gu_out.len - FF * 4), hid, FF, slots, 2 * FF, 2 * FF, FF)
        backend.matvec_experts(dnb, dn_t, lib_, slots, hid, FF, y, HIDDEN)
        backend.combine_experts(y, lwb, lib_, sb, out, CombineShape(columns=HIDDEN, slots=K, experts=n, in_stride=HIDDEN, out_stride=HIDDEN, rows=tokens))
        backend.commit()
        total += out.floats().reshape(tokens, HIDDEN).astype(np.float64)
        owners += int(np.count_nonzero(lwb.floats()[:slots]))
        idx = ib.read(np.uint32)[:slots]
        assert np.array_equal(lib_.read(np.uint32)[:slots], np.where((idx >= e0) & (idx < e1), idx - e0, 0))
        for buf in (gub, dnb, sb):
            backend.release(buf)
    assert owners == slots  # every routed slot has exactly one owner (weights are positive)
    for t in range(tokens):
        idx, w = oracle.route(logits[t], K)
        want = oracle.ffn((enc.Q4_K, EXPERTS, 2 * FF, HIDDEN, gate_up), (enc.Q8_0, EXPERTS, HIDDEN, FF, down), x[t], idx, w, down_scale=scales)
        bound = 2e-5 * (1 + np.max(np.abs(want)))
        assert np.max(np.abs(total[t] - want)) <= bound, (t, np.max(np.abs(total[t] - want)), bound)
    for buf in (xb, lb, ib, wb, lib_, lwb, gu_out, hid, y, out):
        backend.release(buf)


def test_expert_lists_group_slot_rows_by_expert(backend):
    rows, experts = 37, 128
    rng = np.random.default_rng(77)
    idx = np.stack([rng.choice(experts, K, replace=False) for _ in range(rows)]).astype(np.uint32)
    idx[0, 0] = 4000  # a corrupt index is clamped to the last expert, as in the other expert operators
    n = rows * K
    words = Backend.expert_lists_words(n, experts)
    bound = (n + 31) // 32 + experts
    assert words == experts + 3 + 3 * bound + n
    ib = backend.create(idx.nbytes); lb = backend.create(words * 4)
    ib.write(idx)
    backend.begin(); backend.expert_lists(ib, rows, K, experts, lb); backend.commit()
    lists = lb.read(np.uint32)[:words]
    flat = np.minimum(idx.reshape(-1), experts - 1)
    counts = np.bincount(flat, minlength=experts)
    assert lists[1] == n
    assert np.array_equal(lists[2:2 + experts + 1], np.concatenate([[0], np.cumsum(counts)]))
    tiles = lists[experts + 3:experts + 3 + 3 * lists[0]].reshape(-1, 3)
    assert lists[0] == sum((c + 31) // 32 for c in counts)
    slot_rows = lists[experts + 3 + 3 * bound:]
    order = np.argsort(flat, kind="stable")
    assert np.array_equal(slot_rows, order)
    at = 0
    for e, first, count in tiles:
        assert first == at and 1 <= count <= 32 and np.all(flat[slot_rows[first:first + count]] == e)
        at += count
    assert at == n
    with pytest.raises(NuclisError):
        backend.begin()
        try:
            backend.expert_lists(ib, rows, K, 300, lb)
        finally:
            backend.discard()
    backend.release(ib); backend.release(lb)


def test_gathered_matmul_over_expert_lists_matches_cpu_ffn(backend, tensors):
    """The prefill form of the expert chain (rows > 8): slot rows grouped by expert, weights read once per
    tile of an expert's rows, against the CPU oracle token by token."""
    gate_up, down = tensors
    tokens = 24
    rng = np.random.default_rng(41)
    x = rng.standard_normal((tokens, HIDDEN)).astype(np.float32)
    logits = rng.standard_normal((tokens, EXPERTS)).astype(np.float32)
    scales = (0.5 + rng.random(EXPERTS)).astype(np.float32)
    gu_t = ExpertMatrix(enc.Q4_K, EXPERTS, 2 * FF, HIDDEN, gate_up.size)
    dn_t = ExpertMatrix(enc.Q8_0, EXPERTS, HIDDEN, FF, down.size)
    slots = tokens * K
    gub, dnb = backend.wrap(gate_up), backend.wrap(down)
    xb = backend.create(x.nbytes); lb = backend.create(logits.nbytes); sb = backend.create(scales.nbytes)
    ib = backend.create(slots * 4); wb = backend.create(slots * 4)
    lists = backend.create(Backend.expert_lists_words(slots, EXPERTS) * 4)
    gu_out = backend.create(slots * 2 * FF * 4); hid = backend.create(slots * FF * 4)
    y = backend.create(slots * HIDDEN * 4); out = backend.create(tokens * HIDDEN * 4)
    xb.write(x); lb.write(logits); sb.write(scales)
    backend.begin()
    backend.route(lb, EXPERTS, K, tokens, EXPERTS, ib, wb)
    backend.expert_lists(ib, tokens, K, EXPERTS, lists)
    backend.matmul_experts(gub, gu_t, lists, tokens, K, xb, HIDDEN, K, gu_out, 2 * FF)
    backend.gelu_mul_rows(gu_out, gu_out.slice(FF * 4, gu_out.len - FF * 4), hid, FF, slots, 2 * FF, 2 * FF, FF)
    backend.matmul_experts(dnb, dn_t, lists, tokens, K, hid, FF, 1, y, HIDDEN)
    backend.combine_experts(y, wb, ib, sb, out, CombineShape(columns=HIDDEN, slots=K, experts=EXPERTS, in_stride=HIDDEN, out_stride=HIDDEN, rows=tokens))
    backend.commit()
    got = out.floats().reshape(tokens, HIDDEN)
    for t in range(tokens):
        idx, w = oracle.route(logits[t], K)
        want = oracle.ffn((enc.Q4_K, EXPERTS, 2 * FF, HIDDEN, gate_up), (enc.Q8_0, EXPERTS, HIDDEN, FF, down), x[t], idx, w, down_scale=scales)
        bound = 2e-5 * (1 + np.max(np.abs(want)))
        assert np.max(np.abs(got[t] - want)) <= bound, (t, np.max(np.abs(got[t] - want)), bound)
    with pytest.raises(NuclisError):  # the shape rules of matmul: rows % 8, columns % 64
        backend.begin()
        try:
            backend.matmul_experts(gub, ExpertMatrix(enc.Q4_K, EXPERTS, 2 * FF, HIDDEN, gate_up.size), lists, tokens, K, xb, HIDDEN - 4, K, gu_out, 2 * FF)
        finally:
            backend.discard()
    backend.unwrap(gate_up); backend.unwrap(down)
    for buf in (xb, lb, sb, ib, wb, lists, gu_out, hid, y, out):
        backend.release(buf)


@pytest.mark.parametrize("tokens", [256, 301])
def test_grouped_prefill_on_the_tensor_cores_matches_cpu_ffn(backend, tensors, tokens):
    """The prefill of the expert layer at a chunk of 256 token rows (2,048 slot rows, 16 per expert on average; 301: ragged
    groups): `matmulExperts` takes the tensor-core tiles (bf16 operands, F32 accumulate). Each of the two grouped GEMMs is
    checked alone, slot row by slot row for a sample of slots and every output row, against the oracle's matvec on the
    bf16-rounded input: relative L2 <= 2e-2 and per element 4e-3 * sum|w*x| + 1e-6, the bounds of the dense prefill; then
    the whole chain against cpu.experts.ffn at the bf16 tolerance, and the same call on the F32 kernel agrees with both."""
    from test_gpu_prefill import from_bf16_bits, to_bf16_bits
    gate_up, down = tensors
    rng = np.random.default_rng(tokens)
    x = rng.standard_normal((tokens, HIDDEN)).astype(np.float32)
    logits = rng.standard_normal((tokens, EXPERTS)).astype(np.float32)
    gu_t = ExpertMatrix(enc.Q4_K, EXPERTS, 2 * FF, HIDDEN, gate_up.size)
    dn_t = ExpertMatrix(enc.Q8_0, EXPERTS, HIDDEN, FF, down.size)
    slots = tokens * K
    gub, dnb = backend.wrap(gate_up), backend.wrap(down)
    xb = backend.create(x.nbytes); lb = backend.create(logits.nbytes)
    ib = backend.create(slots * 4); wb = backend.create(slots * 4)
    lists = backend.create(Backend.expert_lists_words(slots, EXPERTS) * 4)
    gu_out = backend.create(slots * 2 * FF * 4); hid = backend.create(slots * FF * 4)
    y = backend.create(slots * HIDDEN * 4); out = backend.create(tokens * HIDDEN * 4)
    xb.write(x); lb.write(logits)
    gu_out.write(np.full(slots * 2 * FF, np.nan, dtype=np.float32)); y.write(np.full(slots * HIDDEN, np.nan, dtype=np.float32))
    launches = backend.launch_count
    backend.begin()
    backend.route(lb, EXPERTS, K, tokens, EXPERTS, ib, wb)
    backend.expert_lists(ib, tokens, K, EXPERTS, lists)
    backend.matmul_experts(gub, gu_t, lists, tokens, K, xb, HIDDEN, K, gu_out, 2 * FF)
    backend.gelu_mul_rows(gu_out, gu_out.slice(FF * 4, gu_out.len - FF * 4), hid, FF, slots, 2 * FF, 2 * FF, FF)
    backend.matmul_experts(dnb, dn_t, lists, tokens, K, hid, FF, 1, y, HIDDEN)
    backend.combine_experts(y, wb, ib, None, out, CombineShape(columns=HIDDEN, slots=K, experts=EXPERTS, in_stride=HIDDEN, out_stride=HIDDEN, rows=tokens))
    backend.commit()
    assert backend.launch_count - launches == 8   # the two grouped GEMMs are a gather pass and the tile kernel each
    picked = ib.read(np.uint32, slots)
    gu, hidden_rows, yy = gu_out.floats().reshape(slots, 2 * FF), hid.floats().reshape(slots, FF), y.floats().reshape(slots, HIDDEN)
    assert np.all(np.isfinite(gu)) and np.all(np.isfinite(yy))
    gu_per, dn_per = gate_up.size // EXPERTS, down.size // EXPERTS
    for s in list(range(0, slots, max(1, slots // 24))) + [slots - 1]:
        e = int(picked[s])
        xr = from_bf16_bits(to_bf16_bits(x[s // K]))
        w_e = gate_up[e * gu_per:(e + 1) * gu_per]
        want = oracle.matvec(enc.Q4_K, 2 * FF, HIDDEN, w_e, xr)
        mag = oracle.matvec_abs(enc.Q4_K, 2 * FF, HIDDEN, w_e, xr)
        assert np.max(np.abs(gu[s] - want) / (4e-3 * mag + 1e-6)) <= 1.0 and np.linalg.norm(gu[s] - want) <= 2e-2 * np.linalg.norm(want), ("gate_up", s)
        hr = from_bf16_bits(to_bf16_bits(hidden_rows[s]))
        d_e = down[e * dn_per:(e + 1) * dn_per]
        want = oracle.matvec(enc.Q8_0, HIDDEN, FF, d_e, hr)
        mag = oracle.matvec_abs(enc.Q8_0, HIDDEN, FF, d_e, hr)
        assert np.max(np.abs(yy[s] - want) / (4e-3 * mag + 1e-6)) <= 1.0 and np.linalg.norm(yy[s] - want) <= 2e-2 * np.linalg.norm(want), ("down", s)
    got = out.floats().reshape(tokens, HIDDEN)
    for t in (0, tokens // 2, tokens - 1):
        idx, w = oracle.route(logits[t], K)
        want = oracle.ffn((enc.Q4_K, EXPERTS, 2 * FF, HIDDEN, gate_up), (enc.Q8_0, EXPERTS, HIDDEN, FF, down), x[t], idx, w)
        assert np.linalg.norm(got[t] - want) <= 2e-2 * np.linalg.norm(want), t
    # the F32 kernel on the same lists: the two forms agree at the bf16 tolerance
    backend.generic_only = True
    backend.begin()
    backend.matmul_experts(gub, gu_t, lists, tokens, K, xb, HIDDEN, K, gu_out, 2 * FF)
    backend.commit()
    backend.generic_only = False
    exact = gu_out.floats().reshape(slots, 2 * FF)
    assert np.linalg.norm(gu - exact) <= 2e-2 * np.linalg.norm(exact)
    backend.unwrap(gate_up); backend.unwrap(down)
    for buf in (xb, lb, ib, wb, lists, gu_out, hid, y, out):
        backend.release(buf)


@pytest.mark.parametrize("encoding", [enc.Q5_0, enc.Q5_1, enc.Q4_0, enc.IQ4_NL, enc.Q5_K])
def test_grouped_prefill_reads_the_other_expert_encodings(backend, encoding):
    """`matmulExperts` on an expert tensor stored in the forms real files use for their down experts (GGUF rows, never
    re-laid): each sampled slot row against the oracle's matvec of its expert on the bf16-rounded input, at the bounds
    of the dense prefill."""
    from test_gpu_prefill import from_bf16_bits, to_bf16_bits
    experts, rows, cols, tokens, k = 8, 136, 768, 160, 2
    data = synth.matrix(encoding, experts * rows, cols, seed=950 + encoding)
    per = data.size // experts
    t = ExpertMatrix(encoding, experts, rows, cols, data.size)
    rng = np.random.default_rng(encoding)
    slots = tokens * k
    x = rng.standard_normal((slots, cols)).astype(np.float32)
    idx = rng.integers(0, experts, size=slots).astype(np.uint32)
    wb = backend.wrap(data)
    xb = backend.create(x.nbytes); xb.write(x)
    ib = backend.create(slots * 4); ib.write(idx)
    lists = backend.create(Backend.expert_lists_words(slots, experts) * 4)
    y = backend.create(slots * rows * 4)
    y.write(np.full(slots * rows, np.nan, dtype=np.float32))
    backend.begin()
    backend.expert_lists(ib, tokens, k, experts, lists)
    backend.matmul_experts(wb, t, lists, tokens, k, xb, cols, 1, y, rows)
    backend.commit()
    got = y.floats().reshape(slots, rows)
    assert np.all(np.isfinite(got))
    for s in list(range(0, slots, 13)) + [slots - 1]:
        e = int(idx[s])
        xr = from_bf16_bits(to_bf16_bits(x[s]))
        w_e = data[e * per:(e + 1) * per]
        want = oracle.matvec(encoding, rows, cols, w_e, xr)
        mag = oracle.matvec_abs(encoding, rows, cols, w_e, xr)
        assert np.max(np.abs(got[s] - want) / (4e-3 * mag + 1e-6)) <= 1.0 and np.linalg.norm(got[s] - want) <= 2e-2 * np.linalg.norm(want), s
    backend.unwrap(data)
    for buf in (xb, ib, lists, y):
        backend.release(buf)


@pytest.mark.parametrize("encoding,ff,cols", [(enc.Q4_K, 704, 2816), (enc.Q4_K, 40, 512), (enc.Q8_0, 48, 128)])
@pytest.mark.parametrize("in_group", [1, 2])
@pytest.mark.parametrize("act", [1, 2])
def test_gate_up_with_the_activation_folded_in(backend, encoding, ff, cols, in_group, act):
    """`matvec_experts_gated`: the gate_up GEMV and the activation pass behind it (ops/experts.zig:36-77, 106-117) as one
    launch on the Q4_K kernel (a block takes 16 gate rows and their 16 up rows; 40 rows: a ragged last block), two on the
    others. The same bits as the two operators give, and act(gate) * up against the oracle."""
    experts, slots = 6, 8
    data = synth.matrix(encoding, experts * 2 * ff, cols, seed=60 + ff)
    per = data.size // experts
    t = ExpertMatrix(encoding, experts, 2 * ff, cols, data.size)
    rng = np.random.default_rng(ff + cols)
    groups = slots // in_group
    x = rng.standard_normal((groups, cols)).astype(np.float32)
    idx = rng.integers(0, experts, size=slots).astype(np.uint32)
    wb = backend.wrap(data)
    xb = backend.create(x.nbytes); xb.write(x)
    ib = backend.create(slots * 4); ib.write(idx)
    gu = backend.create(slots * 2 * ff * 4)
    hid, hid2 = backend.create(slots * ff * 4), backend.create(slots * ff * 4)
    before = backend.launch_count
    backend.begin()
    backend.matvec_experts_gated(wb, t, ib, slots, xb, cols, in_group, hid, ff, act=act)
    backend.commit()
    assert backend.launch_count - before == (1 if encoding == enc.Q4_K else 2)
    backend.begin()
    backend.matvec_experts_grouped(wb, t, ib, slots, xb, cols, in_group, gu, 2 * ff)
    if act == 2:
        backend.gelu_mul_rows(gu, gu.slice(ff * 4, gu.len - ff * 4), hid2, ff, slots, 2 * ff, 2 * ff, ff)
    backend.commit()
    got = hid.floats().reshape(slots, ff)
    if act == 2:
        assert np.array_equal(got.view(np.uint32), hid2.floats().reshape(slots, ff).view(np.uint32))
    for s in range(slots):
        e = int(idx[s])
        both = oracle.matvec(encoding, 2 * ff, cols, data[e * per:(e + 1) * per], x[s // in_group])
        g, u = both[:ff], both[ff:]
        want = (oracle.gelu(g) if act == 2 else oracle.silu(g)).astype(np.float64) * u
        assert rel_l2(got[s], want) <= 1e-5, s
    backend.unwrap(data)
    for buf in (xb, ib, gu, hid, hid2):
        backend.release(buf)


def test_gathered_matvec_reads_only_selected_experts(backend):
    # unselected experts hold NaN-decoding bytes (scale 0x7e00): a stray read poisons the output
    experts, rows, cols = 6, 32, 256
    good = synth.matrix(enc.Q8_0, experts * rows, cols, seed=3).reshape(experts, -1).copy()
    per = good.shape[1]
    selected = [4, 1]
    for e in range(experts):
        if e not in selected:
            good[e].reshape(-1, 34)[:, 0:2] = [0x00, 0x7E]
    data = good.reshape(-1)
    t = ExpertMatrix(enc.Q8_0, experts, rows, cols, data.size)
    x = np.random.default_rng(1).standard_normal(cols).astype(np.float32)
    wb = backend.wrap(data)
    xb = backend.create(cols * 4); xb.write(x)
    ib = backend.create(8); ib.write(np.array(selected, dtype=np.uint32))
    yb = backend.create(2 * rows * 4)
    backend.begin()
    backend.matvec_experts(wb, t, ib, 2, xb, 0, yb, rows)
    backend.commit()
    got = yb.floats().reshape(2, rows)
    for s, e in enumerate(selected):
        want = oracle.matvec(enc.Q8_0, rows, cols, data[e * per:(e + 1) * per], x)
        assert np.all(np.isfinite(got[s]))
        assert np.allclose(got[s], want, rtol=1e-5, atol=1e-5)
    # an index past the tensor is clamped, never read out of bounds
    ib.write(np.array([99, 1], dtype=np.uint32))
    backend.begin()
    backend.matvec_experts(wb, t, ib, 2, xb, 0, yb, rows)
    backend.commit()
    backend.unwrap(data)
    for buf in (xb, ib, yb):
        backend.release(buf)


@pytest.mark.parametrize("encoding,rows,cols", [(enc.Q4_K, 50, 768), (enc.Q4_K, 32, 256), (enc.Q4_K, 70, 2048), (enc.Q8_0, 37, 96), (enc.Q8_0, 37, 192), (enc.Q8_0, 8, 704), (enc.Q8_0, 150, 64),
                                                (enc.Q6_K, 24, 512), (enc.Q5_0, 37, 192), (enc.Q5_0, 70, 704), (enc.Q5_1, 37, 96), (enc.Q5_1, 40, 704), (enc.Q4_0, 33, 128),
                                                (enc.Q4_0, 64, 704), (enc.IQ4_NL, 37, 192), (enc.IQ4_NL, 8, 704), (enc.Q5_0, 20, 96), (enc.IQ4_XS, 24, 512)])
@pytest.mark.parametrize("in_group", [1, 3])
def test_expert_gemv_ragged_shapes(backend, encoding, rows, cols, in_group):
    """Row counts that do not fill a block, one to a few blocks per row, slots sharing an input row in groups
    (ops/experts.zig:36-77: slot s reads input row s / in_group) — Q4_K, and Q8_0, Q5_0, Q5_1, Q4_0, IQ4_NL with rows of
    whole 32-bit words, on the specialized kernels, the rest (here also Q5_0 with three blocks a row) on the generic one,
    each against the oracle's matvec of the selected expert."""
    experts, slots = 5, 7
    data = synth.matrix(encoding, experts * rows, cols, seed=40 + rows)
    per = data.size // experts
    t = ExpertMatrix(encoding, experts, rows, cols, data.size)
    rng = np.random.default_rng(rows + cols + in_group)
    groups = (slots + in_group - 1) // in_group
    in_stride = cols + 8
    x = rng.standard_normal((groups, in_stride)).astype(np.float32)
    idx = rng.integers(0, experts, size=slots).astype(np.uint32)
    out_stride = rows + 3
    wb = backend.wrap(data)
    xb = backend.create(x.nbytes); xb.write(x)
    ib = backend.create(slots * 4); ib.write(idx)
    yb = backend.create(slots * out_stride * 4)
    backend.begin()
    backend.matvec_experts_grouped(wb, t, ib, slots, xb, in_stride, in_group, yb, out_stride)
    backend.commit()
    got = yb.floats().reshape(slots, out_stride)[:, :rows]
    for s in range(slots):
        e = int(idx[s])
        xs = x[s // in_group, :cols]
        want = oracle.matvec(encoding, rows, cols, data[e * per:(e + 1) * per], xs)
        scale = oracle.matvec_abs(encoding, rows, cols, data[e * per:(e + 1) * per], xs)
        assert np.max(np.abs(got[s] - want) / np.maximum(scale, 1e-30)) <= 2e-6, (s, e)
    backend.unwrap(data)
    for buf in (xb, ib, yb):
        backend.release(buf)


@pytest.mark.parametrize("encoding,cols", [(enc.Q4_K, 512), (enc.Q8_0, 128), (enc.Q5_0, 128), (enc.Q5_1, 128), (enc.Q4_0, 128), (enc.IQ4_NL, 128)])
def test_expert_gemv_extreme_inputs(backend, encoding, cols):
    """The specialized expert kernels turn the input row into fixed point per chunk of columns: rows scaled by
    1e+-20, a chunk of zeros and a chunk 2^40 times larger than its neighbours stay within the acceptance
    bound; an infinity in the input gives a non-finite output as the F32 arithmetic would."""
    experts, rows, slots = 3, 40, 3
    data = synth.matrix(encoding, experts * rows, cols, seed=77)
    per = data.size // experts
    t = ExpertMatrix(encoding, experts, rows, cols, data.size)
    rng = np.random.default_rng(cols)
    x = rng.standard_normal((slots, cols)).astype(np.float32)
    x[0] *= np.float32(1e20)
    x[1] *= np.float32(1e-20)
    x[2, :32] = 0.0
    x[2, 32:64] *= np.float32(2.0 ** 40)
    idx = np.array([2, 0, 1], dtype=np.uint32)
    wb = backend.wrap(data)
    xb = backend.create(x.nbytes); xb.write(x)
    ib = backend.create(slots * 4); ib.write(idx)
    yb = backend.create(slots * rows * 4)
    backend.begin()
    backend.matvec_experts(wb, t, ib, slots, xb, cols, yb, rows)
    backend.commit()
    got = yb.floats().reshape(slots, rows)
    for s in range(slots):
        e = int(idx[s])
        want = oracle.matvec(encoding, rows, cols, data[e * per:(e + 1) * per], x[s])
        scale = oracle.matvec_abs(encoding, rows, cols, data[e * per:(e + 1) * per], x[s])
        assert np.max(np.abs(got[s] - want) / np.maximum(scale, 1e-30)) <= 2e-6, s
    x[1, 5] = np.inf
    xb.write(x)
    backend.begin()
    backend.matvec_experts(wb, t, ib, slots, xb, cols, yb, rows)
    backend.commit()
    got = yb.floats().reshape(slots, rows)
    assert not np.isfinite(got[1]).any()
    assert np.isfinite(got[0]).all() and np.isfinite(got[2]).all()
    backend.unwrap(data)
    for buf in (xb, ib, yb):
        backend.release(buf)
