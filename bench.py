"""Benchmark of the quantized-weight matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens M] [--impl reference]

Workload (the benchmark's config 2): the synthetic dense 27B-shape decode layer
stack, 64 layers of QKV (Q4_K) -> O (Q4_K) -> SiLU gate/up pair (Q4_K) -> down
(Q6_K), hidden 5120, intermediate 17408, random-init weights drawn on the
device, hidden state N(0,1). A step is one decode pass of all 64 layers for M
tokens (M = 1: decode; M = 8: the speculative-verify batch). With N GPUs the
layers are row-split over the ranks (strong scaling) with a sum over the ranks
after every O and down projection (over NVLink peer memory, fused with the
GEMV that produces the vector; ``--nccl-only`` uses NCCL instead).

One JSON line is printed by rank 0:
  value     tokens per second, whole job, device-timed (CUDA events on the
            backend's stream, max over ranks), inputs resident in HBM;
  e2e       the same through the C ABI with host buffers: each step uploads the
            hidden state from pinned host memory, replays the recorded step and
            downloads the output row(s);
  roofline  the dominant kernel (the fused Q4_K gate/up decode GEMV): algorithmic
            bytes per launch over its measured launch time, against the measured
            HBM copy bandwidth of MEASURED_PEAKS.json;
  cpu_baseline  the CPU oracle (a C restatement of the reference's F64 CPU path)
            timed on this box's host cores on a bounded sample (layers of the same
            stack), extrapolated to the stack;
  clocks    SM clock and throttle reasons sampled during the timed region.

``--impl reference`` times that CPU path alone on the same metric.

``--workload experts`` times the mixture-of-experts decode chain instead (the
benchmark's config 4: 128 experts, top-8, hidden 2816, expert width 704; router,
Q4_K gate_up GEMV of the routed slots, GELU gate, Q8_0 down GEMV, weighted
combine) for M = ``--tokens`` tokens on one GPU and prints one line of its own.
Several chains with different router logits are recorded into the replayed
graph, so that a replay touches more expert bytes than L2 holds.
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
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


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


# ---- CPU arm --------------------------------------------------------------------------------------

def cpu_layers_per_second(tokens: int, sample_layers: int, seed: int = 1):
    """Times `sample_layers` layers of the stack on the CPU oracle with all host cores; returns
    (layers per second, cores, seconds)."""
    import oracle
    from oracle import ref as oref
    from nuclis_b200 import synth
    from nuclis_b200.shard import LayerShapes
    from nuclis_b200.stack import reference_layer
    shapes = LayerShapes()
    cores = oref.cores()
    w = {"qkv": synth.matrix(shapes.qkv_encoding, shapes.qkv_rows, shapes.hidden, seed),
         "o": synth.matrix(shapes.o_encoding, shapes.hidden, shapes.hidden, seed + 1),
         "gate": synth.matrix(shapes.gate_up_encoding, shapes.ffn, shapes.hidden, seed + 2),
         "up": synth.matrix(shapes.gate_up_encoding, shapes.ffn, shapes.hidden, seed + 3),
         "down": synth.matrix(shapes.down_encoding, shapes.hidden, shapes.ffn, seed + 4)}
    h = synth.activations(tokens, shapes.hidden, seed + 5)
    reference_layer(oracle, shapes, w, h[:1], cores)  # warm the pages and the thread pool
    t0 = time.perf_counter()
    for _ in range(sample_layers):
        reference_layer(oracle, shapes, w, h, cores)
    dt = time.perf_counter() - t0
    return sample_layers / dt, cores, dt


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    import oracle
    oracle.build()
    ms = []
    lps = None
    for i in range(args.warmup + args.steps):
        lps, cores, dt = cpu_layers_per_second(args.tokens, 1, seed=1 + i)
        if i >= args.warmup:
            ms.append(dt * 1e3 * LAYERS)
    ms_per_step = float(np.mean(ms))
    value = args.tokens * 1e3 / ms_per_step
    line = {
        "impl": "reference", "metric": "synthetic 27B-shape decode tok/s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 (f64 accumulate)", "data": "synthetic",
        "config": {"workload": f"config 2: 64-layer 27B-shape decode stack, M={args.tokens}", "tokens": args.tokens, "layers": LAYERS},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": "each step times 1 of 64 layers on the CPU oracle (C restatement of the reference's cpu.matvec path; the Zig original cannot be built here) and multiplies by 64"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- GPU arm --------------------------------------------------------------------------------------

def run_gpu(args, rank: int, world: int, local: int):
    import torch
    import torch.distributed as dist
    from nuclis_b200 import Backend, Matrix, Segment, SegmentMode, encoding as enc
    from nuclis_b200.stack import make_stack

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    b = Backend(local)
    if world > 1:
        from nuclis_b200.group import join, torch_all_gather
        join(b, rank, world, torch_all_gather(), peer_memory=not args.nccl_only)
    tokens = args.tokens
    stack = make_stack(b, tokens, LAYERS, ranks=world, rank=rank, seed=args.seed)
    torch.cuda.synchronize()
    h_host = torch.randn(tokens, stack.shapes.hidden, generator=torch.Generator().manual_seed(args.seed)).pin_memory()
    out_host = torch.empty(tokens, stack.shapes.hidden).pin_memory()
    h_np, out_np = h_host.numpy(), out_host.numpy()
    if tokens == 1:
        stack.h.write(h_np)
    else:
        stack.h.slice(0, h_np.nbytes).write(h_np)

    b.begin()
    ops = stack.record()
    launches_before = b.launch_count
    graph = b.commit_retain()
    launches_per_step = b.launch_count if launches_before == 0 else None
    launches_per_step = b.launch_count  # every recorded operator launched once by commit_retain

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up
    barrier()
    b.graph_launch(graph, max(args.warmup, 3))
    # ---- device-timed region: K steps back to back, inputs resident ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    ms = b.graph_launch(graph, args.steps)
    barrier()
    # ---- end to end through the C ABI with host buffers ----
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        (stack.h if tokens == 1 else stack.h.slice(0, h_np.nbytes)).write(h_np)
        b.graph_launch(graph, 1)
        b._check(b._lib.nu_cuda_buffer_download(b._h, stack.d.id, stack.d.offset, out_np.ctypes.data, out_np.nbytes))
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms, e2e_s], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    ms_per_step = ms / args.steps
    value = tokens * 1e3 / ms_per_step
    e2e_value = tokens * args.steps / e2e_s

    roofline = cpu = None
    if rank == 0:
        # ---- the dominant kernel alone: the fused Q4_K gate/up pair of every layer in turn (distinct weights, 6.4 GB > L2) ----
        peak, peak_kind = measured_peak()
        l = stack.local
        b.begin()
        n_pair = 0
        for w in stack.layers:
            if tokens == 1:
                b.matvec_segments([Segment(w.gate, stack.m_gate, stack.g), Segment(w.up, stack.m_gate, stack.g)], stack.o, SegmentMode.silu_mul_pair)
                n_pair += 1
            else:
                b.matmul(w.gate, stack.m_gate, stack.o, stack.shapes.hidden, stack.g, l.ffn_rows, tokens)
                n_pair += 1
        pair_graph = b.commit_retain()
        b.graph_launch(pair_graph, 3)
        pair_ms = b.graph_launch(pair_graph, 5) / (5 * n_pair)
        mats = 2 if tokens == 1 else 1
        algo = mats * stack.m_gate.bytes + tokens * stack.shapes.hidden * 4 + tokens * l.ffn_rows * 4 * (1 if tokens == 1 else 1)
        achieved = algo / (pair_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "q4k_decode_kernel (SiLU gate/up pair)" if tokens == 1 else "rows_kernel<Q4K> (gate)",
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": f"{peak_kind} HBM copy bandwidth",
                    "bytes_per_launch": algo, "us_per_launch": pair_ms * 1e3,
                    # ncu dram__bytes_read+write of one decode launch (50.21 MB for a 50.14 MB matrix), scaled by the bytes of this launch
                    "traffic": algo * (50.207488 / 50.13504) if tokens == 1 else None,
                    "chain_achieved": stack.algorithmic_bytes_per_step() / (ms_per_step * 1e-3) / 1e9}
        b.graph_release(pair_graph)
        if world == 1 and not args.no_cpu:
            import oracle
            oracle.build()
            lps, cores, dt = cpu_layers_per_second(tokens, args.cpu_layers)
            cpu = {"value": tokens * lps / LAYERS, "unit": "tok/s", "cores": cores, "kind": "port",
                   "sample": f"{args.cpu_layers} layer passes of the same stack on the CPU oracle ({dt:.1f} s), scaled to the {LAYERS} layers of a token"}

    if rank == 0:
        line = {
            "metric": "synthetic 27B-shape decode tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 (fp16 hi+lo tensor-core products, f32 accumulate)", "data": "synthetic",
            "config": {"workload": f"config 2: 64-layer 27B-shape decode stack, M={tokens}", "tokens": tokens, "layers": LAYERS,
                       "parallelism": f"tp{world}", "l2": "13.4 GB of weights per step, far larger than L2", "operators_per_step": ops},
            "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": int(h_np.nbytes), "d2h_bytes_per_step": int(out_np.nbytes)},
            "gpu_launches": int(launches_per_step) * args.steps,
            "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        b.comm_destroy()
        dist.destroy_process_group()
    b.deinit()


def run_experts(args):
    """Config 4 on one GPU: microseconds per expert chain and the bandwidth over the distinct experts' bytes."""
    import oracle
    from nuclis_b200 import Backend, CombineShape, ExpertMatrix, encoding as enc, synth
    experts, k, hidden, ff = 128, 8, 2816, 704
    tokens = args.tokens
    chains = 16 if tokens == 1 else 6
    b = Backend(0)
    gate_up = synth.matrix(enc.Q4_K, experts * 2 * ff, hidden, seed=args.seed + 901)
    down = synth.matrix(enc.Q8_0, experts * hidden, ff, seed=args.seed + 902)
    gu_t = ExpertMatrix(enc.Q4_K, experts, 2 * ff, hidden, gate_up.size)
    dn_t = ExpertMatrix(enc.Q8_0, experts, hidden, ff, down.size)
    gub, dnb = b.wrap(gate_up), b.wrap(down)
    rng = np.random.default_rng(args.seed)
    slots = tokens * k
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    xb = b.create(x.nbytes); xb.write(x)
    ib = b.create(slots * 4); wb = b.create(slots * 4)
    gu_out = b.create(slots * 2 * ff * 4); hid = b.create(slots * ff * 4)
    y = b.create(slots * hidden * 4); out = b.create(tokens * hidden * 4)
    distinct = 0
    lbs = []
    for c in range(chains):
        logits = rng.standard_normal((tokens, experts)).astype(np.float32)
        lb = b.create(logits.nbytes); lb.write(logits)
        lbs.append(lb)
        distinct += len({int(e) for t in range(tokens) for e in oracle.route(logits[t], k)[0]})
    b.begin()
    for lb in lbs:
        b.route(lb, experts, k, tokens, experts, ib, wb)
        b.matvec_experts_grouped(gub, gu_t, ib, slots, xb, hidden if tokens > 1 else 0, k if tokens > 1 else 1, gu_out, 2 * ff)
        b.gelu_mul_rows(gu_out, gu_out.slice(ff * 4, gu_out.len - ff * 4), hid, ff, slots, 2 * ff, 2 * ff, ff)
        b.matvec_experts(dnb, dn_t, ib, slots, hid, ff, y, hidden)
        b.combine_experts(y, wb, ib, None, out, CombineShape(columns=hidden, slots=k, experts=experts, in_stride=hidden, out_stride=hidden, rows=tokens))
    graph = b.commit_retain()
    launches = b.launch_count
    b.graph_launch(graph, max(args.warmup, 3))
    us = b.graph_launch(graph, args.steps) / (args.steps * chains) * 1e3
    # where a chain's time goes: the same operators once more with an event after each (adds the events' own cost)
    names = ["route", "gate_up", "gelu_mul", "down", "combine"]
    b.enable_profiling(len(names) * chains)
    b.begin()
    for lb in lbs:
        b.route(lb, experts, k, tokens, experts, ib, wb)
        b.matvec_experts_grouped(gub, gu_t, ib, slots, xb, hidden if tokens > 1 else 0, k if tokens > 1 else 1, gu_out, 2 * ff)
        b.gelu_mul_rows(gu_out, gu_out.slice(ff * 4, gu_out.len - ff * 4), hid, ff, slots, 2 * ff, 2 * ff, ff)
        b.matvec_experts(dnb, dn_t, ib, slots, hid, ff, y, hidden)
        b.combine_experts(y, wb, ib, None, out, CombineShape(columns=hidden, slots=k, experts=experts, in_stride=hidden, out_stride=hidden, rows=tokens))
    b.commit()
    per_op = b.profile_read().reshape(chains, len(names))[1:].mean(axis=0) * 1e6
    per_expert = gate_up.size // experts + down.size // experts
    algo = distinct / chains * per_expert
    peak, source = measured_peak()
    print(json.dumps({
        "metric": "config 4 expert decode chain", "value": us, "unit": "us per chain", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": False, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config 4: 128 experts, top-8, hidden 2816, width 704", "tokens": tokens, "chains_per_replay": chains,
                   "l2": f"{distinct * per_expert / 1e6:.0f} MB of distinct expert bytes per replay, larger than L2",
                   "kernels": "generic" if os.environ.get("NUCLIS_EXPERTS_GENERIC") == "1" else "specialized"},
        "gpu_launches": launches * args.steps,
        "per_operator_us": {n: round(float(v), 2) for n, v in zip(names, per_op)},
        "roofline": {"bound": "hbm", "achieved": algo / (us * 1e-6) / 1e9, "peak": peak, "unit": "GB/s", "frac": algo / (us * 1e-6) / 1e9 / peak,
                     "peak_source": source + " HBM copy bandwidth", "bytes_per_chain": algo, "traffic": None},
    }), flush=True)
    b.deinit()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-layers", type=int, default=192, help="layer passes timed on the CPU oracle for cpu_baseline (about 10 s)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--nccl-only", action="store_true", help="sum the short vectors with NCCL instead of the peer-memory allreduce")
    ap.add_argument("--workload", default="stack", choices=["stack", "experts"])
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.workload == "experts":
        if world > 1 or args.impl != "ours":
            raise SystemExit("--workload experts runs on one GPU, this library only")
        run_experts(args)
        return
    if args.impl == "reference":
        if args.steps == 20:
            args.steps = 5
        run_reference(args, rank, world)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torchrun for --gpus > 1 (one rank per GPU)")
    run_gpu(args, rank, world, local)


if __name__ == "__main__":
    main()
