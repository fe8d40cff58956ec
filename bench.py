"""Benchmark of the quantized-weight matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens M] [--impl reference]
    python bench.py --workload gemv|prefill|experts ...        one operator alone (what the profiles capture)

Default workload (the benchmark's config 2): the synthetic dense 27B-shape decode layer stack, 64 layers
of QKV (Q4_K) -> O (Q4_K) -> SiLU gate/up pair (Q4_K) -> down (Q6_K), hidden 5120, intermediate 17408,
random-init weights drawn on the device, hidden state N(0,1). A step is one decode pass of all 64 layers
for M tokens (M = 1: decode; M = 8: the speculative-verify batch). With N GPUs the layers are row-split
over the ranks (strong scaling) with a sum over the ranks after every O and down projection (over NVLink
peer memory, fused with the GEMV that produces the vector; ``--nccl-only`` uses NCCL instead).

One JSON line is printed by rank 0:
  value     tokens per second, whole job, device-timed (CUDA events on the backend's stream, max over
            ranks), inputs resident in HBM;
  e2e       the same through the C ABI with host buffers: each step uploads the hidden state from pinned
            host memory, replays the recorded step and downloads the output row(s);
  roofline  the dominant kernel (the fused Q4_K gate/up GEMV): algorithmic bytes per launch over its
            measured launch time, against the measured HBM copy bandwidth of MEASURED_PEAKS.json;
  parity    one layer of the recorded (sharded) step against the CPU oracle, and whether all ranks hold
            the same bits, checked before anything is timed;
  cpu_baseline  the CPU oracle (a C restatement of the reference's F64 CPU path) timed on this box's host
            cores on a bounded sample (layers of the same stack), scaled to the stack;
  configs   (one GPU) the benchmark's other configurations measured in the same run through the C ABI:
            config 0 (4096 x 4096 Q4_K GEMV over 32 distinct matrices), config 1 (three encodings x two
            shapes x 1, 2, 4, 8 tokens), config 2 at 8 tokens, config 3 (prefill GEMM at 512, 4096 and
            16384 tokens), config 4 (expert chain at 1 and 8 tokens), each with its roofline fraction
            and a CPU sample; (N GPUs) config 4 with the experts sharded over the ranks;
  clocks    SM clock and throttle reasons sampled during the timed region.

``--impl reference`` times the CPU path alone on the same metric: every step is one whole 64-layer pass
(two weight sets in turn) on all host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYERS = 64
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL_HBM_GBS = 8000.0


def measured_peaks():
    """The roofline denominators measured on this pool's B200s, else the stated fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK}, "measured"
    except Exception:
        return dict(FALLBACK), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 50 ms while the timed region runs (read-only)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.rows, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(self.device)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def hbm_roofline(algo_bytes: float, us: float, kernel: str, traffic=None) -> dict:
    peaks, kind = measured_peaks()
    achieved = algo_bytes / (us * 1e-6) / 1e9
    return {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
            "frac_of_nominal_8tbs": achieved / NOMINAL_HBM_GBS, "peak_source": f"{kind} HBM copy bandwidth", "bytes_per_launch": algo_bytes,
            "us_per_launch": us, "traffic": traffic}


# ---- CPU arm: the oracle (test infrastructure) timed as the reference's CPU path ---------------------

def cpu_layer(oracle, shapes, w: dict, h: np.ndarray, tasks=None) -> np.ndarray:
    """One layer of the stack on the CPU oracle (full, unsharded matrices as bytes in ``w``); h is [tokens][hidden]."""
    out = []
    for t in range(h.shape[0]):
        qkv = oracle.matvec(shapes.qkv_encoding, shapes.qkv_rows, shapes.hidden, w["qkv"], h[t], tasks)
        o = oracle.matvec(shapes.o_encoding, shapes.hidden, shapes.hidden, w["o"], qkv[: shapes.hidden], tasks)
        g = oracle.matvec(shapes.gate_up_encoding, shapes.ffn, shapes.hidden, w["gate"], o, tasks)
        u = oracle.matvec(shapes.gate_up_encoding, shapes.ffn, shapes.hidden, w["up"], o, tasks)
        a = (oracle.silu(g) * u).astype(np.float32)
        out.append(oracle.matvec(shapes.down_encoding, shapes.hidden, shapes.ffn, w["down"], a, tasks))
    return np.stack(out)


def cpu_layer_weights(seed: int) -> dict:
    from nuclis_b200 import synth
    from nuclis_b200.shard import LayerShapes
    s = LayerShapes()
    return {"qkv": synth.matrix(s.qkv_encoding, s.qkv_rows, s.hidden, seed), "o": synth.matrix(s.o_encoding, s.hidden, s.hidden, seed + 1),
            "gate": synth.matrix(s.gate_up_encoding, s.ffn, s.hidden, seed + 2), "up": synth.matrix(s.gate_up_encoding, s.ffn, s.hidden, seed + 3),
            "down": synth.matrix(s.down_encoding, s.hidden, s.ffn, seed + 4)}


def cpu_layers_per_second(tokens: int, seconds: float, seed: int = 1):
    """Times layer passes of the stack on the CPU oracle with all host cores for about `seconds`;
    returns (layers per second, cores, seconds spent, layer passes)."""
    import oracle
    from oracle import ref as oref
    from nuclis_b200 import synth
    from nuclis_b200.shard import LayerShapes
    shapes = LayerShapes()
    cores = oref.cores()
    w = cpu_layer_weights(seed)
    h = synth.activations(tokens, shapes.hidden, seed + 5)
    cpu_layer(oracle, shapes, w, h[:1], cores)  # warm the pages and the thread pool
    done, t0 = 0, time.perf_counter()
    while True:
        cpu_layer(oracle, shapes, w, h, cores)
        done += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            return done / dt, cores, dt, done


def run_reference(args, rank: int, world: int):
    """The reference's CPU implementation of the path (its C restatement: the Zig original cannot be built here),
    all host cores, whole 64-layer passes: rank 0 alone runs and prints, the other ranks leave."""
    if rank != 0:
        return
    import oracle
    from oracle import ref as oref
    from nuclis_b200 import synth
    from nuclis_b200.shard import LayerShapes
    oracle.build()
    shapes, cores = LayerShapes(), oref.cores()
    sets = [cpu_layer_weights(11), cpu_layer_weights(23)]  # two weight sets in turn: 418 MB, far beyond the host caches
    h = synth.activations(args.tokens, shapes.hidden, 7)
    ms = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        for layer in range(LAYERS):
            cpu_layer(oracle, shapes, sets[layer & 1], h, cores)
        if i >= args.warmup:
            ms.append((time.perf_counter() - t0) * 1e3)
    ms_per_step = float(np.mean(ms))
    value = args.tokens * 1e3 / ms_per_step
    line = {
        "impl": "reference", "metric": "synthetic 27B-shape decode tok/s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 (f64 accumulate)", "data": "synthetic",
        "config": {"workload": f"config 2: 64-layer 27B-shape decode stack, M={args.tokens}", "tokens": args.tokens, "layers": LAYERS},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": "every step is one whole 64-layer pass on the CPU oracle (C restatement of the reference's cpu.matvec path; the Zig original cannot be built here), two weight sets in turn"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- one operator alone, through the C ABI, device-timed over distinct weights ----------------------

ALGO_BPW = {12: 0.5625, 14: 0.8203125, 8: 1.0625}
ENC_NAME = {12: "q4_k", 14: "q6_k", 8: "q8_0", 13: "q5_k", 2: "q4_0", 6: "q5_0", 7: "q5_1", 20: "iq4_nl", 23: "iq4_xs", 10: "q2_k", 11: "q3_k"}


def device_matrices(b, encoding: int, rows: int, columns: int, copies: int, seed: int, prepare: bool):
    """`copies` distinct random matrices drawn on the device; the encodings that have a prepared planar form in it when `prepare`."""
    import torch
    from nuclis_b200 import Matrix, encoding as enc, synth
    from nuclis_b200.stack import device_tensor
    nbytes = enc.matrix_bytes(encoding, rows, columns)
    m = Matrix(encoding, rows, columns, nbytes)
    bufs = []
    for i in range(copies):
        wb = b.create(nbytes)
        synth.fill_matrix_torch(device_tensor(wb), encoding, rows, columns, seed * 1000 + i)
        torch.cuda.synchronize()
        mm = m
        if prepare and encoding in (enc.Q6_K, enc.Q8_0, enc.Q4_0, enc.Q5_0, enc.Q5_1, enc.IQ4_NL, enc.IQ4_XS, enc.Q2_K, enc.Q3_K):
            pb, mm = b.prepare(wb, m)
            b.release(wb)
            wb = pb
        bufs.append(wb)
    return bufs, mm


def time_gemv(b, encoding: int, rows: int, columns: int, tokens: int, reps: int = 10, seed: int = 3, min_bytes: float = 3.2e8):
    """Microseconds per launch of one GEMV (1 token) or 2..8-row GEMM, cycling distinct matrices (more bytes than L2
    holds) inside one recorded graph; inputs resident."""
    from nuclis_b200 import encoding as enc
    nbytes = enc.matrix_bytes(encoding, rows, columns)
    copies = max(3, int(np.ceil(min_bytes / nbytes)))
    bufs, m = device_matrices(b, encoding, rows, columns, copies, seed, prepare=True)
    x = np.random.default_rng(seed).standard_normal((tokens, columns), dtype=np.float32)
    xb = b.create(x.nbytes); xb.write(x)
    yb = b.create(tokens * rows * 4)
    b.begin()
    for wb in bufs:
        if tokens == 1:
            b.matvec(wb, m, xb, yb)
        else:
            b.matvec_rows(wb, m, xb, columns, yb, rows, tokens)
    g = b.commit_retain()
    b.graph_launch(g, 3)
    us = b.graph_launch(g, reps) / (reps * copies) * 1e3
    b.graph_release(g)
    for wb in bufs:
        b.release(wb)
    b.release(xb); b.release(yb)
    algo = nbytes + tokens * columns * 4 + tokens * rows * 4
    return us, algo, copies


def time_prefill(b, encoding: int, rows: int, columns: int, tokens: int, seed: int = 5):
    """Microseconds per prefill GEMM (bf16 activations, F32 out) on one matrix."""
    import torch
    from nuclis_b200 import Backend, encoding as enc
    from nuclis_b200.stack import device_tensor
    bufs, m = device_matrices(b, encoding, rows, columns, 1, seed, prepare=True)
    padded = Backend.matmul_padded(tokens)
    xb = b.create(padded * columns * 2)
    device_tensor(xb).view(torch.bfloat16).normal_()
    torch.cuda.synchronize()
    yb = b.create(padded * rows * 4)
    b.begin()
    b.matmul(bufs[0], m, xb, columns, yb, rows, tokens, in_dtype=enc.BF16)
    g = b.commit_retain()
    b.graph_launch(g, 3)
    reps = 8 if tokens <= 4096 else 4
    us = b.graph_launch(g, reps) / reps * 1e3
    b.graph_release(g)
    for buf in (bufs[0], xb, yb):
        b.release(buf)
    return us, 2.0 * tokens * rows * columns


def cpu_gemv_sample(encoding: int, rows: int, columns: int, seed: int = 9):
    """One F64-accumulating matvec of the CPU oracle on all host cores: (microseconds, cores)."""
    import oracle
    from oracle import ref as oref
    from nuclis_b200 import synth
    w = synth.matrix(encoding, rows, columns, seed)
    x = synth.activations(1, columns, seed + 1)[0]
    cores = oref.cores()
    oracle.matvec(encoding, rows, columns, w, x, cores)
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or time.perf_counter() - t0 < 0.3:
        oracle.matvec(encoding, rows, columns, w, x, cores)
        reps += 1
    return (time.perf_counter() - t0) / reps * 1e6, cores


class ExpertCase:
    """Config 4: 128 experts, top-8, hidden 2816, expert width 704; gate_up Q4_K [E][1408][2816], down Q8_0
    [E][2816][704] (a 704-column row is no whole number of Q6_K superblocks: the reference refuses it).
    With `ranks` > 1 this rank holds its range of the experts and one sum over the ranks ends a chain."""
    experts, k, hidden, ff = 128, 8, 2816, 704

    def __init__(self, b, tokens: int, seed: int, ranks: int = 1, rank: int = 0, chains: int | None = None):
        import oracle
        from nuclis_b200 import ExpertMatrix, encoding as enc, shard, synth
        self.b, self.tokens, self.ranks, self.rank = b, tokens, ranks, rank
        E, k, hidden, ff = self.experts, self.k, self.hidden, self.ff
        self.first, last = shard.expert_range(E, ranks, rank)
        self.local = last - self.first
        self.gate_up = synth.matrix(enc.Q4_K, E * 2 * ff, hidden, seed + 901)   # every rank draws the whole tensor and keeps its slice
        self.down = synth.matrix(enc.Q8_0, E * hidden, ff, seed + 902)
        gu_per, dn_per = self.gate_up.size // E, self.down.size // E
        self.per_expert = gu_per + dn_per
        gu_l = self.gate_up[self.first * gu_per: last * gu_per]
        dn_l = self.down[self.first * dn_per: last * dn_per]
        self.gu_t = ExpertMatrix(enc.Q4_K, self.local, 2 * ff, hidden, gu_l.size)
        self.dn_t = ExpertMatrix(enc.Q8_0, self.local, hidden, ff, dn_l.size)
        self.gub, self.dnb = b.create(gu_l.size), b.create(dn_l.size)
        self.gub.write(gu_l); self.dnb.write(dn_l)
        self.chains = chains or (16 if tokens == 1 else 6)
        rng = np.random.default_rng(seed)
        slots = self.slots = tokens * k
        self.x = rng.standard_normal((tokens, hidden)).astype(np.float32)
        self.xb = b.create(self.x.nbytes); self.xb.write(self.x)
        self.ib, self.wb = b.create(slots * 4), b.create(slots * 4)
        self.lib, self.lwb = b.create(slots * 4), b.create(slots * 4)
        self.gu_out, self.hid = b.create(slots * 2 * ff * 4), b.create(slots * ff * 4)
        self.y, self.out = b.create(slots * hidden * 4), b.create(tokens * hidden * 4)
        self.logits, self.lbs, self.distinct = [], [], 0
        for _ in range(self.chains):
            lg = rng.standard_normal((tokens, E)).astype(np.float32)
            lb = b.create(lg.nbytes); lb.write(lg)
            self.logits.append(lg); self.lbs.append(lb)
            chosen = {int(e) for t in range(tokens) for e in oracle.route(lg[t], k)[0]}
            self.distinct += len([e for e in chosen if self.first <= e < last])

    def record(self, lb) -> int:
        """One chain: router -> (this rank's view of the routing) -> gate_up with the GELU gate -> down -> combine (-> sum)."""
        from nuclis_b200 import CombineShape
        b, E, k, hidden, ff, tokens, slots = self.b, self.experts, self.k, self.hidden, self.ff, self.tokens, self.slots
        b.route(lb, E, k, tokens, E, self.ib, self.wb)
        ib, wb, ops = self.ib, self.wb, 5
        if self.ranks > 1:
            b.route_local(self.ib, self.wb, slots, self.first, self.local, self.lib, self.lwb)
            ib, wb, ops = self.lib, self.lwb, 7
        # gate_up and the GELU gate in one launch (matvec_experts_gated: matvecExpertsGrouped + geluMulRows)
        b.matvec_experts_gated(self.gub, self.gu_t, ib, slots, self.xb, hidden if tokens > 1 else 0, k if tokens > 1 else 1, self.hid, ff, act=2)
        ops -= 1
        b.matvec_experts(self.dnb, self.dn_t, ib, slots, self.hid, ff, self.y, hidden)
        b.combine_experts(self.y, wb, ib, None, self.out, CombineShape(columns=hidden, slots=k, experts=self.local, in_stride=hidden, out_stride=hidden, rows=tokens))
        if self.ranks > 1:
            b.allreduce_sum_f32(self.out, tokens * hidden)
        return ops

    def parity(self) -> float:
        """Worst |error| / (2e-5 * (1 + max|y|)) of the last recorded chain's output against cpu.experts.ffn (bound 1.0)."""
        import oracle
        from nuclis_b200 import encoding as enc
        E, k, hidden, ff = self.experts, self.k, self.hidden, self.ff
        got = self.out.floats().reshape(self.tokens, hidden)
        worst = 0.0
        for t in range(self.tokens):
            idx, w = oracle.route(self.logits[-1][t], k)
            want = oracle.ffn((enc.Q4_K, E, 2 * ff, hidden, self.gate_up), (enc.Q8_0, E, hidden, ff, self.down), self.x[t], idx, w)
            worst = max(worst, float(np.max(np.abs(got[t] - want)) / (2e-5 * (1.0 + np.max(np.abs(want))))))
        return worst

    def measure(self, steps: int, warmup: int) -> dict:
        b = self.b
        b.begin()
        for lb in self.lbs:
            ops = self.record(lb)
        graph = b.commit_retain()
        worst = self.parity()
        b.graph_launch(graph, max(warmup, 3))
        us = b.graph_launch(graph, steps) / (steps * self.chains) * 1e3
        b.graph_release(graph)
        algo = self.distinct / self.chains * self.per_expert
        roof = hbm_roofline(algo, us, "expert chain (router, gate_up GEMV with the GELU gate, down GEMV, combine)")
        return {"us_per_chain": us, "tokens": self.tokens, "operators_per_chain": ops, "chains_per_replay": self.chains,
                "distinct_expert_mb_per_replay": self.distinct * self.per_expert / 1e6, "parity_worst_over_bound": worst, "roofline": roof}


def expert_prefill(b, tokens: int, seed: int, steps: int = 10) -> dict:
    """The prefill form of config 4's layer: `tokens` token rows routed, their slot rows grouped by expert, both expert
    GEMMs on the tensor-core tiles (router -> lists -> gate_up -> GELU gate -> down -> combine), microseconds per chain."""
    from nuclis_b200 import Backend, CombineShape
    case = ExpertCase(b, 1, seed, chains=1)
    E, k, hidden, ff = case.experts, case.k, case.hidden, case.ff
    slots = tokens * k
    rng = np.random.default_rng(seed + tokens)
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    logits = rng.standard_normal((tokens, E)).astype(np.float32)
    xb, lb = b.create(x.nbytes), b.create(logits.nbytes)
    xb.write(x); lb.write(logits)
    ib, wb = b.create(slots * 4), b.create(slots * 4)
    lists = b.create(Backend.expert_lists_words(slots, E) * 4)
    gu_out, hid = b.create(slots * 2 * ff * 4), b.create(slots * ff * 4)
    y, out = b.create(slots * hidden * 4), b.create(tokens * hidden * 4)
    b.begin()
    b.route(lb, E, k, tokens, E, ib, wb)
    b.expert_lists(ib, tokens, k, E, lists)
    b.matmul_experts(case.gub, case.gu_t, lists, tokens, k, xb, hidden, k, gu_out, 2 * ff)
    b.gelu_mul_rows(gu_out, gu_out.slice(ff * 4, gu_out.len - ff * 4), hid, ff, slots, 2 * ff, 2 * ff, ff)
    b.matmul_experts(case.dnb, case.dn_t, lists, tokens, k, hid, ff, 1, y, hidden)
    b.combine_experts(y, wb, ib, None, out, CombineShape(columns=hidden, slots=k, experts=E, in_stride=hidden, out_stride=hidden, rows=tokens))
    graph = b.commit_retain()
    b.graph_launch(graph, 3)
    us = b.graph_launch(graph, steps) / steps * 1e3
    b.graph_release(graph)
    flops = 2.0 * slots * (2 * ff * hidden + hidden * ff)
    peaks, kind = measured_peaks()
    for buf in (xb, lb, ib, wb, lists, gu_out, hid, y, out):
        b.release(buf)
    return {"us_per_chain": us, "tokens": tokens, "slot_rows": slots, "tflops": flops / us / 1e6,
            "roofline": {"bound": "tensor", "achieved": flops / us / 1e6, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": flops / us / 1e6 / peaks["bf16_tflops"],
                         "peak_source": f"{kind} cuBLAS bf16 (burst)"}}


# ---- parity of one (sharded) layer of the recorded step, before anything is timed -------------------

def layer_parity(b, tokens: int, rank: int, world: int, seed: int) -> dict:
    """One layer with this rank's shards drawn on the device, recorded exactly as the timed step records it, against
    the CPU oracle on the same shards (the partial O and down outputs of the ranks are gathered over gloo and added
    in rank order on the host). Returns the relative L2 error and whether all ranks hold the same bits."""
    import torch
    import torch.distributed as dist
    import oracle
    from nuclis_b200.stack import make_stack
    st = make_stack(b, tokens, 1, ranks=world, rank=rank, seed=seed + 77, prepare=False)
    w, s, l = st.layers[0], st.shapes, st.local
    torch.cuda.synchronize()
    host = {k: getattr(w, k).read() for k in ("qkv", "o", "gate", "up", "down")}  # the GGUF bytes, before the planar re-layout
    st.prepare_layer(w)
    h = np.random.default_rng(seed + 5).standard_normal((tokens, s.hidden), dtype=np.float32)
    (st.h if tokens == 1 else st.h.slice(0, h.nbytes)).write(h)
    b.begin()
    st.record()
    b.commit()
    got = st.d.floats()[: tokens * s.hidden].reshape(tokens, s.hidden).copy()

    def summed(partial: np.ndarray) -> np.ndarray:
        if world == 1:
            return partial
        parts = [torch.zeros_like(torch.from_numpy(partial)) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(partial))
        total = parts[0].numpy().copy()
        for q in parts[1:]:
            total += q.numpy()
        return total

    want = np.empty_like(got)
    for t in range(tokens):
        qkv = oracle.matvec(s.qkv_encoding, l.qkv_rows, s.hidden, host["qkv"], h[t])
        o = summed(oracle.matvec(s.o_encoding, s.hidden, l.q_rows, host["o"], qkv[: l.q_rows]))
        a = (oracle.silu(oracle.matvec(s.gate_up_encoding, l.ffn_rows, s.hidden, host["gate"], o)) *
             oracle.matvec(s.gate_up_encoding, l.ffn_rows, s.hidden, host["up"], o)).astype(np.float32)
        want[t] = summed(oracle.matvec(s.down_encoding, s.hidden, l.ffn_rows, host["down"], a))
    rel = float(np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64)))
    same = True
    if world > 1:
        bits = torch.from_numpy(got.view(np.int32).astype(np.int64).ravel())
        lo, hi = bits.clone(), bits.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = bool(torch.equal(lo, hi))
        t_rel = torch.tensor([rel], dtype=torch.float64)
        dist.all_reduce(t_rel, op=dist.ReduceOp.MAX)
        rel = float(t_rel[0])
    for buf in (w.qkv, w.o, w.gate, w.up, w.down, st.h, st.qkv, st.o, st.g, st.u, st.d):
        b.release(buf)
    return {"rel_l2": rel, "bound": 1e-5, "ok": bool(rel <= 1e-5 and same), "ranks_bit_identical": same,
            "what": f"one layer of the recorded step (tokens={tokens}, tp{world}) against the CPU oracle on the same shards"}


# ---- the other configurations, measured in the same run (one GPU) -----------------------------------

def other_configs(b, args, stack8_value=None, stack_norms=None) -> dict:
    from nuclis_b200 import encoding as enc
    peaks, kind = measured_peaks()
    out = {}
    # config 0: one Q4_K GEMV, 4096 x 4096, 32 distinct matrices (302 MB) cycled inside one graph
    us, algo, copies = time_gemv(b, enc.Q4_K, 4096, 4096, 1, reps=20)
    cpu_us, cores = cpu_gemv_sample(enc.Q4_K, 4096, 4096)
    out["config0"] = {"workload": "Q4_K GEMV 4096x4096, M=1", "us": us, "distinct_matrices": copies, "roofline": hbm_roofline(algo, us, "i8_kernel<Q4K> one token"),
                      "cpu_baseline": {"us": cpu_us, "cores": cores, "kind": "port", "sample": "the whole matvec on the CPU oracle"}}
    # config 1: three encodings x two shapes x 1, 2, 4, 8 tokens
    sweep = {}
    for e in (enc.Q4_K, enc.Q6_K, enc.Q8_0):
        for rows, columns in ((17408, 5120), (5120, 17408)):
            row = {}
            for m in (1, 2, 4, 8):
                us, algo, copies = time_gemv(b, e, rows, columns, m)
                row[f"m{m}"] = {"us": us, "gbs": algo / us / 1e3, "frac": algo / us / 1e3 / peaks["hbm_gbs"]}
            row["m8_over_m1"] = row["m8"]["us"] / row["m1"]["us"]
            cpu_us, cores = cpu_gemv_sample(e, rows, columns)
            row["cpu_baseline"] = {"us_m1": cpu_us, "cores": cores, "kind": "port"}
            sweep[f"{ENC_NAME[e]}_{rows}x{columns}"] = row
    # the other encodings of the integer path: one shape, one and eight tokens
    for e in (enc.Q5_K, enc.Q4_0, enc.Q5_0, enc.Q5_1, enc.IQ4_NL, enc.IQ4_XS, enc.Q2_K, enc.Q3_K):
        row = {}
        for m in (1, 8):
            us, algo, copies = time_gemv(b, e, 17408, 5120, m)
            row[f"m{m}"] = {"us": us, "gbs": algo / us / 1e3, "frac": algo / us / 1e3 / peaks["hbm_gbs"]}
        row["m8_over_m1"] = row["m8"]["us"] / row["m1"]["us"]
        sweep[f"{ENC_NAME[e]}_17408x5120"] = row
    out["config1"] = {"workload": "dequant-fused GEMV / small-M GEMM sweep (all but Q4_K and Q5_K in the prepared planar form)", "peak_gbs": peaks["hbm_gbs"],
                      "peak_source": kind, "cases": sweep}
    if stack8_value is not None:
        out["config2_m8"] = stack8_value
    if stack_norms is not None:
        out["config2_with_norms"] = stack_norms
    # config 3: prefill GEMM, bf16 activations
    pre = {}
    for e, rows, columns in ((enc.Q4_K, 17408, 5120), (enc.Q6_K, 5120, 17408)):
        cpu_us, cores = cpu_gemv_sample(e, rows, columns)
        for tokens in (512, 4096, 16384):
            us, flops = time_prefill(b, e, rows, columns, tokens)
            tf = flops / us / 1e6
            pre[f"{ENC_NAME[e]}_{rows}x{columns}_t{tokens}"] = {
                "us": us, "tflops": tf, "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"],
                                                     "frac_of_sustained": tf / peaks["bf16_tflops_sustained"], "peak_source": f"{kind} cuBLAS bf16 (burst)"},
                "cpu_baseline": {"tflops": flops / (cpu_us * tokens) / 1e6, "cores": cores, "kind": "port", "sample": "one token row on the CPU oracle, scaled to the token count"}}
    # the other encodings: one shape, 4,096 token rows
    for e in (enc.Q8_0, enc.Q5_K, enc.Q4_0, enc.Q5_0, enc.Q5_1, enc.IQ4_NL, enc.IQ4_XS, enc.Q2_K, enc.Q3_K):
        us, flops = time_prefill(b, e, 17408, 5120, 4096)
        tf = flops / us / 1e6
        pre[f"{ENC_NAME[e]}_17408x5120_t4096"] = {"us": us, "tflops": tf, "frac": tf / peaks["bf16_tflops"], "frac_of_sustained": tf / peaks["bf16_tflops_sustained"]}
    out["config3"] = {"workload": "prefill GEMM on tcgen05 (weights decoded to bf16 tiles, F32 accumulate)", "cases": pre}
    # config 4: the expert chain at 1 and 8 tokens
    ex = {}
    for tokens in (1, 8):
        case = ExpertCase(b, tokens, args.seed)
        ex[f"m{tokens}"] = case.measure(max(args.steps, 10), args.warmup)
    ex["prefill_t512"] = expert_prefill(b, 512, args.seed)
    out["config4"] = {"workload": "expert decode chain: 128 experts, top-8, hidden 2816, width 704 (gate_up Q4_K, down Q8_0)", "cases": ex}
    return out


# ---- GPU arm: the layer stack ------------------------------------------------------------------------

def time_stack(b, stack, args, barrier, rank: int):
    """Records one step of `stack`, replays it: (ms per step device-timed, seconds of the end-to-end loop, launches per step,
    operators per step, bytes up, bytes down)."""
    import torch
    tokens = stack.tokens
    h_host = torch.randn(tokens, stack.shapes.hidden, generator=torch.Generator().manual_seed(args.seed)).pin_memory()
    out_host = torch.empty(tokens, stack.shapes.hidden).pin_memory()
    h_np, out_np = h_host.numpy(), out_host.numpy()
    hbuf = stack.h if tokens == 1 else stack.h.slice(0, h_np.nbytes)
    hbuf.write(h_np)
    before = b.launch_count
    b.begin()
    ops = stack.record()
    graph = b.commit_retain()
    launches = b.launch_count - before  # commit_retain runs the recorded step once
    barrier()
    b.graph_launch(graph, max(args.warmup, 3))
    # ---- device-timed region: K steps back to back, inputs resident ----
    barrier()
    ms = b.graph_launch(graph, args.steps)
    barrier()
    # ---- end to end through the C ABI with host buffers ----
    t0 = time.perf_counter()
    for _ in range(args.steps):
        hbuf.write(h_np)
        b.graph_launch(graph, 1)
        b._check(b._lib.nu_cuda_buffer_download(b._h, stack.d.id, stack.d.offset, out_np.ctypes.data, out_np.nbytes))
    e2e_s = time.perf_counter() - t0
    barrier()
    b.graph_release(graph)
    return ms / args.steps, e2e_s, launches, ops, int(h_np.nbytes), int(out_np.nbytes)


def dominant_kernel(b, stack, tokens: int) -> dict:
    """The fused Q4_K gate/up pair of every layer in turn (distinct weights, 6.4 GB > L2), timed alone."""
    from nuclis_b200 import Segment, SegmentMode
    l = stack.local
    b.begin()
    for w in stack.layers:
        if tokens == 1:
            b.matvec_segments([Segment(w.gate, stack.m_gate, stack.g), Segment(w.up, stack.m_gate, stack.g)], stack.o, SegmentMode.silu_mul_pair)
        else:
            b.matmul(w.gate, stack.m_gate, stack.o, stack.shapes.hidden, stack.g, l.ffn_rows, tokens)
    graph = b.commit_retain()
    b.graph_launch(graph, 3)
    us = b.graph_launch(graph, 5) / (5 * len(stack.layers)) * 1e3
    b.graph_release(graph)
    mats = 2 if tokens == 1 else 1
    algo = mats * stack.m_gate.bytes + tokens * stack.shapes.hidden * 4 + tokens * l.ffn_rows * 4
    # ncu dram__bytes_read + write of one launch of this kernel on a 50.1 MB matrix (profiles/), scaled by the bytes of this launch
    traffic = algo * (50.221056 + 0.001024) / 50.13504 if tokens == 1 else None
    return hbm_roofline(algo, us, "i8_kernel<Q4K> (SiLU gate/up pair, one token)" if tokens == 1 else "i8_kernel<Q4K> (gate, token rows)", traffic)


def run_gpu(args, rank: int, world: int, local: int):
    import torch
    import torch.distributed as dist
    from nuclis_b200 import Backend
    from nuclis_b200.stack import Stack, make_stack

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    b = Backend(local)
    b.chaining = args.chain
    if world > 1:
        from nuclis_b200.group import join, torch_all_gather
        join(b, rank, world, torch_all_gather(), peer_memory=not args.nccl_only)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    tokens = args.tokens
    parity = layer_parity(b, tokens, rank, world, args.seed)
    stack = make_stack(b, tokens, args.layers, ranks=world, rank=rank, seed=args.seed)
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_per_step, e2e_s, launches, ops, up, down = time_stack(b, stack, args, barrier, rank)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms_per_step, e2e_s], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step, e2e_s = float(t[0]), float(t[1])
    value = tokens * 1e3 / ms_per_step
    e2e_value = tokens * args.steps / e2e_s

    configs = None
    if world > 1 and not args.no_configs:
        # config 4 with the experts sharded over the ranks: every rank runs the chain on its experts, one sum ends it
        ex = {}
        for m in (1, 8):
            case = ExpertCase(b, m, args.seed, ranks=world, rank=rank)
            barrier()
            r = case.measure(max(args.steps, 10), args.warmup)
            tt = torch.tensor([r["us_per_chain"], r["parity_worst_over_bound"]], dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ex[f"m{m}"] = {"us_per_chain": float(tt[0]), "parity_worst_over_bound": float(tt[1]), "experts_per_rank": case.local, "operators_per_chain": r["operators_per_chain"]}
        configs = {"config4_expert_parallel": {"workload": f"expert chain, 128 experts over {world} ranks, one allreduce of the combined outputs per chain", "cases": ex}}
        if tokens == 1:
            # the sharded stack as a pre-norm decoder runs it: the norms in the staging passes of QKV and gate/up, the residual
            # adds in the gathers of the two sums (the same six launches a layer)
            st3 = Stack(b, stack.shapes, stack.local, 1)
            st3.layers, st3.m_down = stack.layers, stack.m_down
            st3.enable_norms(args.seed)
            ms3, e2e3, launches3, ops3, _, _ = time_stack(b, st3, args, barrier, rank)
            t3 = torch.tensor([ms3, e2e3], dtype=torch.float64)
            dist.all_reduce(t3, op=dist.ReduceOp.MAX)
            configs["config2_with_norms"] = {"workload": f"config 2 with the RMS norms and residual adds of a pre-norm layer folded in, M=1, tp{world}", "tok_s": 1e3 / float(t3[0]),
                                             "ms_per_step": float(t3[0]), "e2e_tok_s": args.steps / float(t3[1]), "operators_per_step": ops3, "launches_per_step": int(launches3)}

    roofline = cpu = None
    if rank == 0:
        roofline = dominant_kernel(b, stack, tokens)
        roofline["chain_achieved"] = stack.algorithmic_bytes_per_step() / (ms_per_step * 1e-3) / 1e9
        if world == 1 and not args.no_configs:
            # config 2 at the other token count, on the same weights
            other = 8 if tokens == 1 else 1
            st2 = Stack(b, stack.shapes, stack.local, other)
            st2.layers, st2.m_down = stack.layers, stack.m_down
            ms2, e2e2, _, ops2, _, _ = time_stack(b, st2, args, barrier, rank)
            stack_other = {"workload": f"config 2: 64-layer stack, M={other}", "tok_s": other * 1e3 / ms2, "ms_per_step": ms2, "e2e_tok_s": other * args.steps / e2e2,
                           "chain_gbs": st2.algorithmic_bytes_per_step() / (ms2 * 1e-3) / 1e9, "operators_per_step": ops2}
            for buf in (st2.h, st2.qkv, st2.o, st2.g, st2.u, st2.d):
                b.release(buf)
            # the same layers as a pre-norm decoder runs them: RMS norm ahead of QKV and of gate/up, residual add behind O
            # and down, folded into those four launches (matvec_segments_normed, matvec_add)
            st3 = Stack(b, stack.shapes, stack.local, 1)
            st3.layers, st3.m_down = stack.layers, stack.m_down
            st3.enable_norms(args.seed)
            ms3, e2e3, launches3, ops3, _, _ = time_stack(b, st3, args, barrier, rank)
            stack_norms = {"workload": "config 2 with the RMS norms and residual adds of a pre-norm layer folded into its four launches, M=1", "tok_s": 1e3 / ms3,
                           "ms_per_step": ms3, "e2e_tok_s": args.steps / e2e3, "operators_per_step": ops3, "launches_per_step": int(launches3)}
            for buf in (st3.h, st3.qkv, st3.o, st3.g, st3.u, st3.d, st3.residual, st3.norm_attn, st3.norm_ffn):
                b.release(buf)
            # the stack's weights make room for the other configurations' tensors
            for w in stack.layers:
                for buf in (w.qkv, w.o, w.gate, w.up, w.down):
                    b.release(buf)
            stack.layers = []
            configs = other_configs(b, args, stack_other, stack_norms)
        if world == 1 and not args.no_cpu:
            import oracle
            oracle.build()
            lps, cores, dt, passes = cpu_layers_per_second(tokens, args.cpu_seconds)
            cpu = {"value": tokens * lps / LAYERS, "unit": "tok/s", "cores": cores, "kind": "port",
                   "sample": f"{passes} layer passes of the same stack on the CPU oracle ({dt:.1f} s), scaled to the {LAYERS} layers of a token"}
        line = {
            "metric": "synthetic 27B-shape decode tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 out; int8 tensor-core products of 4- and 6-bit codes x 24-bit fixed-point activations, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"config 2: {args.layers}-layer 27B-shape decode stack, M={tokens}" + ("" if args.layers == LAYERS else " (NOT the configuration: a profiler-sized stack)"),
                       "tokens": tokens, "layers": args.layers, "parallelism": f"tp{world}", "l2": f"{13.4 * args.layers / LAYERS:.1f} GB of weights per step, far larger than L2",
                       "operators_per_step": ops, "chained": args.chain},
            "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": up, "d2h_bytes_per_step": down},
            "gpu_launches": int(launches) * args.steps,
            "roofline": roofline, "parity": parity, "cpu_baseline": cpu, "clocks": clocks, "configs": configs,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        b.comm_destroy()
        dist.destroy_process_group()
    b.deinit()


# ---- one operator alone (what the ncu captures under profiles/ run) -----------------------------------

def run_one(args):
    from nuclis_b200 import Backend, encoding as enc
    b = Backend(0)
    peaks, kind = measured_peaks()
    if args.workload == "gemv":
        us, algo, copies = time_gemv(b, args.encoding, args.rows, args.columns, args.tokens, reps=args.steps, min_bytes=args.min_bytes)
        line = {"metric": "GEMV / small-M GEMM", "value": us, "unit": "us per launch", "higher_is_better": False,
                "config": {"workload": f"{ENC_NAME.get(args.encoding, args.encoding)} {args.rows}x{args.columns}, M={args.tokens}", "distinct_matrices": copies},
                "roofline": hbm_roofline(algo, us, "GEMV")}
    elif args.workload == "prefill":
        us, flops = time_prefill(b, args.encoding, args.rows, args.columns, args.tokens)
        tf = flops / us / 1e6
        line = {"metric": "prefill GEMM", "value": tf, "unit": "TFLOP/s", "higher_is_better": True,
                "config": {"workload": f"{ENC_NAME.get(args.encoding, args.encoding)} {args.rows}x{args.columns}, T={args.tokens}"}, "us": us,
                "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"], "peak_source": f"{kind} cuBLAS bf16 (burst)"}}
    else:
        case = ExpertCase(b, args.tokens, args.seed)
        r = case.measure(args.steps, args.warmup)
        line = {"metric": "config 4 expert decode chain", "value": r["us_per_chain"], "unit": "us per chain", "higher_is_better": False, **r}
    line.update({"n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "data": "synthetic"})
    print(json.dumps(line), flush=True)
    b.deinit()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-seconds", type=float, default=10.0, help="seconds of layer passes timed on the CPU oracle for cpu_baseline")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="the stack alone: skip the other configurations")
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers of the stack (the configuration has 64; fewer only for a profiler capture, and the line says so)")
    ap.add_argument("--chain", action="store_true", help="runs of matvecs as one persistent kernel each instead of kernels of their own (measured slower; off by default)")
    ap.add_argument("--nccl-only", action="store_true", help="sum the short vectors with NCCL instead of the peer-memory allreduce")
    ap.add_argument("--workload", default="stack", choices=["stack", "gemv", "prefill", "experts"])
    ap.add_argument("--encoding", type=int, default=12, help="GGUF type id of the matrix of --workload gemv / prefill (12 Q4_K, 13 Q5_K, 14 Q6_K, 8 Q8_0, 2 Q4_0, 6 Q5_0, 7 Q5_1, 10 Q2_K, 11 Q3_K, 20 IQ4_NL, 23 IQ4_XS)")
    ap.add_argument("--rows", type=int, default=17408)
    ap.add_argument("--columns", type=int, default=5120)
    ap.add_argument("--min-bytes", type=float, default=3.2e8, help="distinct weight bytes cycled by --workload gemv")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload != "stack":
        if world > 1:
            raise SystemExit("single-operator workloads run on one GPU")
        run_one(args)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torchrun for --gpus > 1 (one rank per GPU)")
    run_gpu(args, rank, world, local)


if __name__ == "__main__":
    main()
