"""The row-split layer stack on two GPUs against the CPU oracle: the peer-memory allreduce and the
NCCL allreduce both reproduce the unsharded chain, also with the residual adds folded into the sums and the RMS norm
into the gate/up pair. Needs two GPUs; skipped on a one-GPU box (the
host-side logic of the split is covered on the CPU by tests/test_shard.py)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def gpu_count() -> int:
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


RANK_SCRIPT = r'''
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["NU_ROOT"])
import oracle
from nuclis_b200 import Backend, Matrix, Segment, SegmentMode, encoding as enc, shard, synth
from nuclis_b200.group import join, torch_all_gather
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
peer = os.environ["NU_PEER"] == "1"
torch.cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
b = Backend(rank)
join(b, rank, world, torch_all_gather(), peer_memory=peer)
shapes = shard.LayerShapes(hidden=1024, ffn=2048, kv=256)
local = shard.rank_shapes(shapes, world, rank)
# every rank draws the same full matrices from the seed and keeps its own slice, as a loader would
wo = synth.matrix(enc.Q4_K, shapes.hidden, shapes.hidden, 1)
wg = synth.matrix(enc.Q4_K, shapes.ffn, shapes.hidden, 2)
wu = synth.matrix(enc.Q4_K, shapes.ffn, shapes.hidden, 3)
wd = synth.matrix(enc.Q6_K, shapes.hidden, shapes.ffn, 4)
h = synth.activations(1, shapes.hidden, 5)[0]

def upload(data):
    buf = b.create(data.nbytes); buf.write(data); return buf

q0, q1 = local.q_range
f0, f1 = local.ffn_range
wo_l = upload(shard.slice_columns(wo, enc.Q4_K, shapes.hidden, shapes.hidden, q0, q1))
wg_l = upload(shard.slice_rows(wg, enc.Q4_K, shapes.ffn, shapes.hidden, f0, f1))
wu_l = upload(shard.slice_rows(wu, enc.Q4_K, shapes.ffn, shapes.hidden, f0, f1))
wd_raw = upload(shard.slice_columns(wd, enc.Q6_K, shapes.hidden, shapes.ffn, f0, f1))
m_o = Matrix(enc.Q4_K, shapes.hidden, q1 - q0, wo_l.len)
m_g = Matrix(enc.Q4_K, f1 - f0, shapes.hidden, wg_l.len)
wd_l, m_d = b.prepare(wd_raw, Matrix(enc.Q6_K, shapes.hidden, f1 - f0, wd_raw.len))
a_l = upload(np.ascontiguousarray(h[q0:q1]))
o = b.create(shapes.hidden * 4); g = b.create((f1 - f0) * 4); d = b.create(shapes.hidden * 4)
b.begin()
b.matvec(wo_l, m_o, a_l, o)
b.allreduce_sum_f32(o, shapes.hidden)
b.matvec_segments([Segment(wg_l, m_g, g), Segment(wu_l, m_g, g)], o, SegmentMode.silu_mul_pair)
b.matvec(wd_l, m_d, g, d)
b.allreduce_sum_f32(d, shapes.hidden)
graph = b.commit_retain()
for _ in range(4): b.graph_launch(graph, 1)   # replays reuse the inbox parities
got = d.floats()[: shapes.hidden]
o_ref = oracle.matvec(enc.Q4_K, shapes.hidden, shapes.hidden, wo, h)
act = (oracle.silu(oracle.matvec(enc.Q4_K, shapes.ffn, shapes.hidden, wg, o_ref)) * oracle.matvec(enc.Q4_K, shapes.ffn, shapes.hidden, wu, o_ref)).astype(np.float32)
d_ref = oracle.matvec(enc.Q6_K, shapes.hidden, shapes.ffn, wd, act)
err = np.linalg.norm(got - d_ref) / np.linalg.norm(d_ref)
assert err < 2e-5, err
# every rank holds the same bits
t = torch.from_numpy(got.view(np.int32).astype(np.int64)); lo = t.clone(); hi = t.clone()
dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
assert torch.equal(lo, hi), "ranks disagree"
dist.barrier()
# the same layer as a pre-norm decoder runs it: the residual adds in the gathers of the two sums, the RMS norm in the
# staging pass of the gate/up pair; executed once (the residual accumulates)
rng = np.random.default_rng(11)
r0 = (rng.standard_normal(shapes.hidden) * 0.5).astype(np.float32)
wn = (1.0 + 0.1 * rng.standard_normal(shapes.hidden)).astype(np.float32)
res, wnb = upload(r0), upload(wn)
b.begin()
b.matvec(wo_l, m_o, a_l, o)
b.allreduce_sum_add_f32(o, res, shapes.hidden)
b.matvec_segments_normed([Segment(wg_l, m_g, g), Segment(wu_l, m_g, g)], res, wnb, mode=SegmentMode.silu_mul_pair)
b.matvec(wd_l, m_d, g, d)
b.allreduce_sum_add_f32(d, res, shapes.hidden)
b.commit()
got2 = res.floats()[: shapes.hidden]
x1 = r0 + o_ref
xn = (oracle.rms_norm(x1).astype(np.float64) * wn).astype(np.float32)
act2 = (oracle.silu(oracle.matvec(enc.Q4_K, shapes.ffn, shapes.hidden, wg, xn)) * oracle.matvec(enc.Q4_K, shapes.ffn, shapes.hidden, wu, xn)).astype(np.float32)
x2 = x1 + oracle.matvec(enc.Q6_K, shapes.hidden, shapes.ffn, wd, act2)
err2 = np.linalg.norm(got2 - x2) / np.linalg.norm(x2)
assert err2 < 2e-5, err2
t = torch.from_numpy(got2.view(np.int32).astype(np.int64)); lo = t.clone(); hi = t.clone()
dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
assert torch.equal(lo, hi), "ranks disagree on the residual"
dist.barrier()
if rank == 0: print("TP-GPU-OK", err, err2)
b.comm_destroy(); dist.destroy_process_group(); b.deinit()
'''


@pytest.mark.gpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("peer", ["1", "0"])
def test_two_gpu_stack_matches_the_oracle(tmp_path, peer):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    env = dict(os.environ, NU_ROOT=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29647" if peer == "1" else "29649", WORLD_SIZE="2", NU_PEER=peer)
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "TP-GPU-OK" in outs[0]
