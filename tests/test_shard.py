"""Host-side logic of the tensor-parallel split, on the CPU: shard tables, byte slicing, and that
the partial results of the ranks sum to the unsharded result (checked on the CPU oracle and with
two gloo ranks standing in for two GPUs)."""
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle
from nuclis_b200 import encoding as enc, shard, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_split_tables_cover_everything_at_superblock_granularity():
    s = shard.LayerShapes()
    for n in (1, 2, 4, 8):
        parts = [shard.rank_shapes(s, n, r) for r in range(n)]
        assert sum(p.q_rows for p in parts) == s.hidden and sum(p.ffn_rows for p in parts) == s.ffn
        assert sum(p.kv_rows for p in parts) == s.kv
        assert all(p.q_rows % 256 == 0 and p.ffn_rows % 256 == 0 for p in parts)
        assert parts[0].q_range[0] == 0 and parts[-1].q_range[1] == s.hidden
        for a, b in zip(parts, parts[1:]):
            assert a.q_range[1] == b.q_range[0] and a.ffn_range[1] == b.ffn_range[0]
    assert shard.split_counts(68, 8) == [8, 9, 8, 9, 8, 9, 8, 9]
    assert shard.split_counts(20, 8) == [2, 3, 2, 3, 2, 3, 2, 3]
    assert abs(shard.balance(68, 8) - 8.5 / 9) < 1e-12 and abs(shard.balance(20, 8) - 2.5 / 3) < 1e-12
    with pytest.raises(ValueError):
        shard.rank_shapes(shard.LayerShapes(kv=1001), 8, 0)


def test_expert_ranges_partition_the_experts():
    for ranks in (1, 2, 4, 8):
        spans = [shard.expert_range(128, ranks, r) for r in range(ranks)]
        assert spans[0][0] == 0 and spans[-1][1] == 128
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(e1 - e0 == 128 // ranks for e0, e1 in spans)
    assert [shard.expert_range(10, 4, r) for r in range(4)] == [(0, 2), (2, 5), (5, 7), (7, 10)]
    with pytest.raises(ValueError):
        shard.expert_range(4, 8, 0)
    with pytest.raises(ValueError):
        shard.expert_range(128, 8, 8)


@pytest.mark.parametrize("encoding", [enc.Q4_K, enc.Q6_K, enc.Q8_0])
def test_column_shards_sum_to_the_full_product(encoding):
    rows, columns = 48, 2048
    w = synth.matrix(encoding, rows, columns, seed=9)
    x = synth.activations(1, columns, 10)[0]
    full = oracle.matvec(encoding, rows, columns, w, x).astype(np.float64)
    total = np.zeros(rows)
    for c0, c1 in [(a * 256, b * 256) for a, b in shard.split_ranges(columns // 256, 3)]:
        part = shard.slice_columns(w, encoding, rows, columns, c0, c1)
        assert part.size == enc.matrix_bytes(encoding, rows, c1 - c0)
        total += oracle.matvec(encoding, rows, c1 - c0, part, x[c0:c1]).astype(np.float64)
    assert np.allclose(total, full, rtol=1e-6, atol=1e-6)
    top = shard.slice_rows(w, encoding, rows, columns, 16, 32)
    assert np.array_equal(oracle.matvec(encoding, 16, columns, top, x), oracle.matvec(encoding, rows, columns, w, x)[16:32])
    with pytest.raises(ValueError):
        shard.slice_columns(w, encoding, rows, columns, 8, 256)


RANK_SCRIPT = r'''
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["NU_ROOT"])
import oracle
from nuclis_b200 import encoding as enc, shard, synth
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
shapes = shard.LayerShapes(hidden=512, ffn=1024, kv=64)
local = shard.rank_shapes(shapes, world, rank)
# every rank draws the same full matrices from the seed and keeps its own slice, as a loader would
wo = synth.matrix(enc.Q4_K, shapes.hidden, shapes.hidden, 1)
wg = synth.matrix(enc.Q4_K, shapes.ffn, shapes.hidden, 2)
wd = synth.matrix(enc.Q6_K, shapes.hidden, shapes.ffn, 3)
h = synth.activations(1, shapes.hidden, 4)[0]
a = h[local.q_range[0]:local.q_range[1]]
o = oracle.matvec(enc.Q4_K, shapes.hidden, local.q_rows, shard.slice_columns(wo, enc.Q4_K, shapes.hidden, shapes.hidden, *local.q_range), a)
t = torch.from_numpy(o.astype(np.float64)); dist.all_reduce(t); o_full = t.numpy().astype(np.float32)
g = oracle.matvec(enc.Q4_K, local.ffn_rows, shapes.hidden, shard.slice_rows(wg, enc.Q4_K, shapes.ffn, shapes.hidden, *local.ffn_range), o_full)
d = oracle.matvec(enc.Q6_K, shapes.hidden, local.ffn_rows, shard.slice_columns(wd, enc.Q6_K, shapes.hidden, shapes.ffn, *local.ffn_range), g)
t = torch.from_numpy(d.astype(np.float64)); dist.all_reduce(t); d_full = t.numpy()
if rank == 0:
    o_ref = oracle.matvec(enc.Q4_K, shapes.hidden, shapes.hidden, wo, h)
    g_ref = oracle.matvec(enc.Q4_K, shapes.ffn, shapes.hidden, wg, o_ref)
    d_ref = oracle.matvec(enc.Q6_K, shapes.hidden, shapes.ffn, wd, g_ref)
    err = np.linalg.norm(d_full - d_ref) / np.linalg.norm(d_ref)
    assert np.linalg.norm(o_full - o_ref) / np.linalg.norm(o_ref) < 1e-6, "o"
    assert err < 1e-5, err
    print("TP-OK", err)
dist.destroy_process_group()
'''


def test_two_gloo_ranks_reproduce_the_unsharded_chain(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    env = dict(os.environ, NU_ROOT=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29641", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "TP-OK" in outs[0]


JOIN_SCRIPT = r'''
import os, sys
import torch.distributed as dist
sys.path.insert(0, os.environ["NU_ROOT"])
from nuclis_b200.group import join, torch_all_gather
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)

class FakeBackend:
    """Records what join() asks of a backend; stands in for the CUDA library on a CPU box."""
    calls = []
    @staticmethod
    def comm_unique_id():
        return bytes([7]) * 128
    def comm_init(self, uid, ranks, rank):
        self.calls.append(("init", uid, ranks, rank))
    def comm_peer_handle(self):
        return bytes([rank + 1]) * 64
    def comm_attach_peers(self, handles, rank):
        self.calls.append(("attach", tuple(handles), rank))

b = FakeBackend()
join(b, rank, world, torch_all_gather())
assert b.calls[0] == ("init", bytes([7]) * 128, world, rank), b.calls[0]
assert b.calls[1] == ("attach", tuple(bytes([r + 1]) * 64 for r in range(world)), rank), b.calls[1]
b2 = FakeBackend(); b2.calls = []
join(b2, rank, world, torch_all_gather(), peer_memory=False)
assert [c[0] for c in b2.calls] == ["init"]
try:
    join(b2, world, world, torch_all_gather())
    raise SystemExit("rank outside the group was accepted")
except ValueError:
    pass
print("JOIN-OK")
dist.destroy_process_group()
'''


def test_group_join_exchanges_id_and_inbox_handles_in_rank_order(tmp_path):
    script = tmp_path / "join.py"
    script.write_text(JOIN_SCRIPT)
    env = dict(os.environ, NU_ROOT=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29643", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("JOIN-OK" in o for o in outs)
