"""The synthetic dense decode layer stack: 64 layers of QKV -> O -> SwiGLU gate/up -> down.

Only the matmul chain of a decoder layer is here (attention, norms and
residuals are other operators' business): per layer

    qkv = Wqkv . h                      Q4_K  [hidden + 2 kv][hidden]
    o   = Wo . qkv[:hidden]             Q4_K  [hidden][hidden]         (+ allreduce)
    a   = silu(Wgate . o) * (Wup . o)   Q4_K  [ffn][hidden] each
    d   = Wdown . a                     Q6_K  [hidden][ffn]            (+ allreduce)

written against the backend's operator interface exactly as a model plan of
the reference would write it (``matvec``, ``matvecSegments`` with the SiLU pair
mode, ``matmul`` for a verify batch; inference/src/models/qwen35_metal.zig:589-640).
Every layer reads the same input hidden state: 64 un-normalised layers of
random weights overflow F32 within a dozen products, and the norms that keep a
real model bounded are not part of this path. Stream order keeps the layers
serial all the same, and every weight byte of every layer is read each step.

With ``ranks`` > 1 the layer is row-split (see ``shard``): each rank holds its
rows of QKV/gate/up and its K slice of O/down, and the partial O and down
outputs are summed over the ranks.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import encoding as enc
from .backend import Backend, Buffer, Matrix, Segment, SegmentMode
from .errors import NuclisError
from .shard import LayerShapes, RankShapes, rank_shapes


@dataclass
class LayerWeights:
    qkv: Buffer
    o: Buffer
    gate: Buffer
    up: Buffer
    down: Buffer


@dataclass
class Stack:
    backend: Backend
    shapes: LayerShapes
    local: RankShapes
    tokens: int
    layers: list[LayerWeights] = field(default_factory=list)

    def __post_init__(self):
        b, s, l, m = self.backend, self.shapes, self.local, self.tokens
        pad = Backend.matmul_padded(m) if m > 1 else 1
        self.m_qkv = Matrix(s.qkv_encoding, l.qkv_rows, s.hidden, enc.matrix_bytes(s.qkv_encoding, l.qkv_rows, s.hidden))
        self.m_o = Matrix(s.o_encoding, s.hidden, l.q_rows, enc.matrix_bytes(s.o_encoding, s.hidden, l.q_rows))
        self.m_gate = Matrix(s.gate_up_encoding, l.ffn_rows, s.hidden, enc.matrix_bytes(s.gate_up_encoding, l.ffn_rows, s.hidden))
        self.m_down = Matrix(s.down_encoding, s.hidden, l.ffn_rows, enc.matrix_bytes(s.down_encoding, s.hidden, l.ffn_rows))
        self.h = b.create(pad * s.hidden * 4)
        self.qkv = b.create(pad * l.qkv_rows * 4)
        self.o = b.create(pad * s.hidden * 4)
        self.g = b.create(pad * l.ffn_rows * 4)
        self.u = b.create(pad * l.ffn_rows * 4)
        self.d = b.create(pad * s.hidden * 4)

    # ---- weights ----
    def weight_bytes_per_layer(self) -> int:
        return self.m_qkv.bytes + self.m_o.bytes + 2 * self.m_gate.bytes + self.m_down.bytes

    def add_layer_buffers(self) -> LayerWeights:
        b = self.backend
        w = LayerWeights(b.create(self.m_qkv.bytes), b.create(self.m_o.bytes), b.create(self.m_gate.bytes),
                         b.create(self.m_gate.bytes), b.create(self.m_down.bytes))
        self.layers.append(w)
        return w

    def fill_layer_torch(self, w: LayerWeights, seed: int) -> None:
        """Random blocks drawn on the device (see ``synth``): local shard shapes, seeded per layer and rank."""
        from . import synth
        s, l = self.shapes, self.local
        for i, (buf, e, rows, cols) in enumerate([(w.qkv, s.qkv_encoding, l.qkv_rows, s.hidden), (w.o, s.o_encoding, s.hidden, l.q_rows),
                                                  (w.gate, s.gate_up_encoding, l.ffn_rows, s.hidden), (w.up, s.gate_up_encoding, l.ffn_rows, s.hidden),
                                                  (w.down, s.down_encoding, s.hidden, l.ffn_rows)]):
            synth.fill_matrix_torch(device_tensor(buf), e, rows, cols, seed * 8 + i)

    def prepare_layer(self, w: LayerWeights) -> None:
        """Load-time re-layout of the matrices whose GGUF rows the specialized kernels cannot address
        (the Q6_K down projection): same bytes, same values. The GGUF copy is released."""
        b = self.backend
        raw = Matrix(self.m_down.encoding, self.m_down.rows, self.m_down.columns, self.m_down.bytes)
        prepared, m = b.prepare(w.down, raw)
        b.release(w.down)
        w.down = prepared
        self.m_down = m

    # ---- the recording of one step ----
    def enable_norms(self, seed: int = 0) -> None:
        """Adds what a pre-norm decoder layer has around its projections (inference/src/models/qwen35_metal.zig:635-640):
        a residual row and the two RMS-norm weight rows (shared by the layers here: their values do not matter to the
        timing). ``record`` then uses the folded operators: four launches a layer, as without the norms."""
        import numpy as np
        b, s = self.backend, self.shapes
        rng = np.random.default_rng(seed + 17)
        self.residual = b.create(s.hidden * 4)
        self.residual0 = (rng.standard_normal(s.hidden) * 0.5).astype(np.float32)
        self.norm_attn, self.norm_ffn = b.create(s.hidden * 4), b.create(s.hidden * 4)
        self.norm_attn_host = (1.0 + 0.1 * rng.standard_normal(s.hidden)).astype(np.float32)
        self.norm_ffn_host = (1.0 + 0.1 * rng.standard_normal(s.hidden)).astype(np.float32)
        self.norm_attn.write(self.norm_attn_host)
        self.norm_ffn.write(self.norm_ffn_host)
        self.residual.write(self.residual0)

    def record_with_norms(self, reduce: bool = False) -> int:
        """One token: x += O(Q(norm(x))); x += down(silu(gate(norm(x))) * up(norm(x))) per layer, the norms folded into the
        staging passes of QKV and of the gate/up pair, the adds into the writes of O and down; with the layer split over
        ranks (``reduce``) the adds are folded into the gathers of the two sums instead."""
        b, hidden = self.backend, self.shapes.hidden
        a_in = self.qkv.slice(0, self.qkv.len)
        for w in self.layers:
            b.matvec_segments_normed([Segment(w.qkv, self.m_qkv, self.qkv)], self.residual, self.norm_attn)
            if reduce:
                b.matvec(w.o, self.m_o, a_in, self.o)
                b.allreduce_sum_add_f32(self.o, self.residual, hidden)
            else:
                b.matvec_add(w.o, self.m_o, a_in, self.residual, self.residual)
            b.matvec_segments_normed([Segment(w.gate, self.m_gate, self.g), Segment(w.up, self.m_gate, self.g)], self.residual, self.norm_ffn,
                                     mode=SegmentMode.silu_mul_pair)
            if reduce:
                b.matvec(w.down, self.m_down, self.g, self.d)
                b.allreduce_sum_add_f32(self.d, self.residual, hidden)
            else:
                b.matvec_add(w.down, self.m_down, self.g, self.residual, self.residual)
        return (6 if reduce else 4) * len(self.layers)

    def record(self, allreduce: bool | None = None) -> int:
        """Records every layer's chain into the open recording; returns how many operators it recorded."""
        b, s, l, m = self.backend, self.shapes, self.local, self.tokens
        reduce = l.ranks > 1 if allreduce is None else allreduce
        ops = 0
        a_in = self.qkv.slice(0, self.qkv.len)  # the Q slice: the first q_rows floats of each token row
        if getattr(self, "residual", None) is not None and m == 1:
            return self.record_with_norms(reduce)
        for w in self.layers:
            if m == 1:
                b.matvec(w.qkv, self.m_qkv, self.h, self.qkv)
                b.matvec(w.o, self.m_o, a_in, self.o)
                ops += 2
                if reduce:
                    b.allreduce_sum_f32(self.o, s.hidden)
                    ops += 1
                try:
                    b.matvec_segments([Segment(w.gate, self.m_gate, self.g), Segment(w.up, self.m_gate, self.g)], self.o, SegmentMode.silu_mul_pair)
                    ops += 1
                except NuclisError as e:
                    if e.name != "MergeDeclined":
                        raise
                    # the caller's fallback of the reference: two projections and the activation (qwen35_metal.zig:597-600)
                    b.matvec(w.gate, self.m_gate, self.o, self.g)
                    b.matvec(w.up, self.m_gate, self.o, self.u)
                    b.silu_mul(self.g, self.u, l.ffn_rows)
                    ops += 3
                b.matvec(w.down, self.m_down, self.g, self.d)
                ops += 1
                if reduce:
                    b.allreduce_sum_f32(self.d, s.hidden)
                    ops += 1
            else:
                b.matmul(w.qkv, self.m_qkv, self.h, s.hidden, self.qkv, l.qkv_rows, m)
                b.matmul(w.o, self.m_o, a_in, l.qkv_rows, self.o, s.hidden, m)
                ops += 2
                if reduce:
                    b.allreduce_sum_f32(self.o, m * s.hidden)
                    ops += 1
                b.matmul(w.gate, self.m_gate, self.o, s.hidden, self.g, l.ffn_rows, m)
                b.matmul(w.up, self.m_gate, self.o, s.hidden, self.u, l.ffn_rows, m)
                b.silu_mul(self.g, self.u, m * l.ffn_rows)
                b.matmul(w.down, self.m_down, self.g, l.ffn_rows, self.d, s.hidden, m)
                ops += 4
                if reduce:
                    b.allreduce_sum_f32(self.d, m * s.hidden)
                    ops += 1
        return ops

    def algorithmic_bytes_per_step(self) -> int:
        """Weight bytes read plus activation bytes read and written by the matmuls, all layers."""
        s, l, m = self.shapes, self.local, self.tokens
        acts = m * 4 * (s.hidden + l.qkv_rows + l.q_rows + s.hidden + 2 * (s.hidden + l.ffn_rows) + l.ffn_rows + s.hidden)
        return len(self.layers) * (self.weight_bytes_per_layer() + acts)


def device_tensor(buf: Buffer):
    """A torch uint8 view of a backend buffer (no copy), for filling it on the device."""
    import torch

    class _Raw:
        pass

    raw = _Raw()
    raw.__cuda_array_interface__ = {"shape": (buf.len,), "typestr": "|u1", "data": (buf.device_ptr, False), "version": 2}
    return torch.as_tensor(raw, device=f"cuda:{buf.backend.device}")


def make_stack(backend: Backend, tokens: int, layers: int, ranks: int = 1, rank: int = 0, seed: int = 0,
               shapes: LayerShapes | None = None, prepare: bool = True) -> Stack:
    shapes = shapes or LayerShapes()
    st = Stack(backend, shapes, rank_shapes(shapes, ranks, rank), tokens)
    for i in range(layers):
        w = st.add_layer_buffers()
        st.fill_layer_torch(w, seed * 100003 + i * 64 + rank)
        if prepare:
            import torch
            torch.cuda.synchronize()
            st.prepare_layer(w)
    return st
