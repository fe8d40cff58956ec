"""GPU parity of the persistent chain (`Backend.chaining = True`; off by default): one-token matvecs recorded
back to back run as one kernel that walks them in order (csrc/gemv_chain.cu). The chain must give, bit for bit, what the same operators give
as kernels of their own (`chaining = False`), and both must match the CPU oracle applied operator by
operator. The cases mix Q4_K and planar Q6_K links, a SiLU gate/up pair, a link that reads a slice of the
output before it, matrices too small to occupy every block (blocks that sit an operator out), a matrix
whose K is cut into slices, runs longer than one launch takes, and a run broken by another operator."""
import numpy as np
import pytest

import oracle
from nuclis_b200 import Backend, Matrix, Segment, SegmentMode, encoding as enc, synth
from parity import rel_l2

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


def weights(b, encoding, rows, columns, seed):
    w = synth.matrix(encoding, rows, columns, seed)
    m = Matrix(encoding, rows, columns, w.size)
    wb = upload(b, w)
    if encoding == enc.Q6_K:
        pb, m = b.prepare(wb, m)
        b.release(wb)
        wb = pb
    return wb, m, w


class Layer:
    """QKV -> O (reads the first `hidden` floats of QKV) -> SiLU gate/up pair -> down, like the decode stack."""

    def __init__(self, b, hidden, kv, ffn, seed, down_encoding=enc.Q6_K):
        self.b, self.hidden, self.kv, self.ffn = b, hidden, kv, ffn
        self.qkv = weights(b, enc.Q4_K, hidden + 2 * kv, hidden, seed)
        self.o = weights(b, enc.Q4_K, hidden, hidden, seed + 1)
        self.gate = weights(b, enc.Q4_K, ffn, hidden, seed + 2)
        self.up = weights(b, enc.Q4_K, ffn, hidden, seed + 3)
        self.down = weights(b, down_encoding, hidden, ffn, seed + 4)
        self.down_encoding = down_encoding
        self.t_qkv = b.create((hidden + 2 * kv) * 4)
        self.t_o = b.create(hidden * 4)
        self.t_g = b.create(ffn * 4)
        self.out = b.create(hidden * 4)

    def record(self, xb):
        b = self.b
        b.matvec(self.qkv[0], self.qkv[1], xb, self.t_qkv)
        b.matvec(self.o[0], self.o[1], self.t_qkv.slice(0, self.hidden * 4), self.t_o)
        b.matvec_segments([Segment(self.gate[0], self.gate[1], self.t_g), Segment(self.up[0], self.up[1], self.t_g)], self.t_o, SegmentMode.silu_mul_pair)
        b.matvec(self.down[0], self.down[1], self.t_g, self.out)
        return self.out

    def reference(self, x):
        h, kv, f = self.hidden, self.kv, self.ffn
        qkv = oracle.matvec(enc.Q4_K, h + 2 * kv, h, self.qkv[2], x)
        o = oracle.matvec(enc.Q4_K, h, h, self.o[2], qkv[:h].copy())
        g = oracle.matvec(enc.Q4_K, f, h, self.gate[2], o)
        u = oracle.matvec(enc.Q4_K, f, h, self.up[2], o)
        a = (oracle.silu(g) * u).astype(np.float32)
        return oracle.matvec(self.down_encoding, h, f, self.down[2], a)

    def release(self):
        for wb, _, _ in (self.qkv, self.o, self.gate, self.up, self.down):
            self.b.release(wb)
        for t in (self.t_qkv, self.t_o, self.t_g, self.out):
            self.b.release(t)


def run(b, layers, x, chaining):
    """Records the layers one after another in one recording, each reading the output of the one before; returns the last
    output and the number of kernels the recording launched."""
    b.chaining = chaining
    xb = upload(b, x)
    launches0 = b.launch_count
    b.begin()
    cur = xb
    for layer in layers:
        cur = layer.record(cur)
    b.commit()
    out = cur.floats().copy()
    b.release(xb)
    b.chaining = False
    return out, b.launch_count - launches0


@pytest.mark.parametrize("hidden,kv,ffn,down", [(512, 128, 1024, enc.Q6_K), (256, 256, 768, enc.Q4_K), (1024, 256, 2560, enc.Q6_K)])
def test_chained_layers_match_unchained_and_oracle(backend, hidden, kv, ffn, down):
    b = backend
    layers = [Layer(b, hidden, kv, ffn, 100 + 10 * i, down) for i in range(2)]
    x = synth.activations(1, hidden, 3)[0] * np.float32(1e-2)
    got, n_chain = run(b, layers, x, True)
    alone, n_alone = run(b, layers, x, False)
    assert n_alone == 8 and n_chain == 1, (n_alone, n_chain)
    assert np.array_equal(got.view(np.uint32), alone.view(np.uint32)), "the chain differs from the same operators as kernels of their own"
    want = x
    for layer in layers:
        want = layer.reference(want)
    assert np.all(np.isfinite(want))
    # eight operators deep: the per-operator bound of 1e-5 compounds
    assert rel_l2(got, want) < 1e-4, rel_l2(got, want)
    for layer in layers:
        layer.release()


def test_small_and_sliced_links(backend):
    """A 32-row matrix keeps two blocks busy, the rest sit the operator out; 64 rows x 8192 columns are cut along K."""
    b = backend
    shapes = [(enc.Q4_K, 64, 8192), (enc.Q4_K, 32, 256 * 1), (enc.Q6_K, 8192, 256), (enc.Q4_K, 48, 8192), (enc.Q6_K, 256, 256), (enc.Q4_K, 8192, 256)]
    mats = []
    cols0 = shapes[0][2]
    x = synth.activations(1, cols0, 5)[0]
    # each link's rows feed the next link's columns through a buffer wide enough for it (zero beyond what was written)
    bufs = [upload(b, x)]
    for i, (e, rows, cols) in enumerate(shapes):
        wb, m, w = weights(b, e, rows, cols, 300 + i)
        mats.append((wb, m, w, e, rows, cols))
        nxt = shapes[i + 1][2] if i + 1 < len(shapes) else rows
        bufs.append(upload(b, np.zeros(max(rows, nxt), np.float32)))
    for chaining in (True, False):
        b.chaining = chaining
        l0 = b.launch_count
        b.begin()
        for i, (wb, m, w, e, rows, cols) in enumerate(mats):
            b.matvec(wb, m, bufs[i], bufs[i + 1])
        b.commit()
        n = b.launch_count - l0
        outs = [bufs[i + 1].floats().copy() for i in range(len(mats))]
        if chaining:
            chained, n_chain = outs, n
        else:
            assert n == len(mats) and n_chain == 1
            for a, c in zip(outs, chained):
                assert np.array_equal(a.view(np.uint32), c.view(np.uint32))
    b.chaining = False
    cur = x
    for i, (wb, m, w, e, rows, cols) in enumerate(mats):
        inp = np.zeros(cols, np.float32)
        k = min(cols, cur.size)
        inp[:k] = cur[:k]
        cur = oracle.matvec(e, rows, cols, w, inp)
        assert rel_l2(chained[i][:rows], cur) < 5e-5, (i, rel_l2(chained[i][:rows], cur))
    for wb, *_ in mats:
        b.release(wb)
    for buf in bufs:
        b.release(buf)


def test_long_runs_and_breaks(backend):
    """Forty links are more than one launch takes; an operator of another kind in the middle ends a run."""
    b = backend
    n, hidden = 40, 256
    mats = [weights(b, enc.Q4_K if i % 3 else enc.Q6_K, hidden, hidden, 500 + i) for i in range(n)]
    x = synth.activations(1, hidden, 9)[0] * np.float32(1e-15)  # each link multiplies the size by about nine
    ping = [upload(b, x), upload(b, np.zeros(hidden, np.float32))]
    results = {}
    for chaining in (True, False):
        ping[0].write(x)
        b.chaining = chaining
        l0 = b.launch_count
        b.begin()
        for i, (wb, m, _) in enumerate(mats):
            b.matvec(wb, m, ping[i % 2], ping[(i + 1) % 2])
            if i == 20:
                b.add(ping[(i + 1) % 2], ping[(i + 1) % 2], hidden)  # x += x: not a link
        b.commit()
        results[chaining] = (ping[n % 2].floats().copy(), b.launch_count - l0)
    b.chaining = False
    (got, n_chain), (alone, n_alone) = results[True], results[False]
    assert n_alone == n + 1
    assert n_chain == 2 + 1 + 2, n_chain  # 21 links = 16 + 5, the add, 19 links = 16 + 3
    assert np.array_equal(got.view(np.uint32), alone.view(np.uint32))
    cur = x
    for i, (_, _, w) in enumerate(mats):
        cur = oracle.matvec(enc.Q4_K if i % 3 else enc.Q6_K, hidden, hidden, w, cur)
        if i == 20:
            cur = cur + cur
    assert np.all(np.isfinite(cur)) and rel_l2(got, cur) < 5e-4, rel_l2(got, cur)
    for wb, _, _ in mats:
        b.release(wb)
    for p in ping:
        b.release(p)
