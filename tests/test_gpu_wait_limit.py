"""A bounded device-side wait that runs out, without faulting or hanging anything: a two-rank peer-memory
group whose second rank never pushes. The second rank is a child process that only allocates its inbox on the
same GPU and hands over the interprocess handle; it launches nothing. With the wait limit set to 200 ms the
allreduce kernel of rank 0 gives up, returns, and `commit` reports ExecutionFailed; the handle stays usable,
the peer-memory path of the group stays closed (the next sum fails at once), and destroying the group drops the
graphs that hold the peers' addresses."""
import os
import subprocess
import sys
import time

import numpy as np
import pytest

from nuclis_b200 import Backend, NuclisError

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys
sys.path.insert(0, os.environ["NU_ROOT"])
from nuclis_b200 import Backend
b = Backend(0)
print(b.comm_peer_handle().hex(), flush=True)
sys.stdin.readline()          # holds the inbox until the parent is done; never pushes anything
b.deinit()
'''


def test_a_peer_that_never_arrives_ends_the_wait_with_a_status():
    child = subprocess.Popen([sys.executable, "-c", CHILD], env=dict(os.environ, NU_ROOT=ROOT), stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    b = Backend(0)
    try:
        theirs = bytes.fromhex(child.stdout.readline().strip())
        assert len(theirs) == 64
        b.comm_attach_peers([b.comm_peer_handle(), theirs], rank=0)
        b.comm_set_wait_ms(200)
        buf = b.create(5120 * 4)
        buf.write(np.ones(5120, dtype=np.float32))
        b.begin()
        b.allreduce_sum_f32(buf, 5120)
        t0 = time.perf_counter()
        with pytest.raises(NuclisError) as first:
            b.commit()
        waited = time.perf_counter() - t0
        assert first.value.name == "ExecutionFailed" and "never arrived" in str(first.value)
        assert 0.15 <= waited < 5.0, waited            # the limit, not the two-second default nor a hang
        # sticky: the next sum over the group fails at once, without waiting again
        b.begin()
        b.allreduce_sum_f32(buf, 5120)
        t0 = time.perf_counter()
        with pytest.raises(NuclisError) as second:
            b.commit()
        assert second.value.name == "ExecutionFailed" and time.perf_counter() - t0 < 0.15
        # a retained graph that holds the peers' addresses goes away with the group
        b.begin()
        b.allreduce_sum_f32(buf, 5120)
        with pytest.raises(NuclisError):
            b.commit_retain()
        b.comm_destroy()
        with pytest.raises(NuclisError):
            b.graph_launch(1, 1)
        # the handle itself is still usable
        other = b.create(64)
        other.write(np.arange(16, dtype=np.float32))
        assert np.array_equal(other.floats(), np.arange(16, dtype=np.float32))
    finally:
        child.stdin.write("done\n")
        child.stdin.flush()
        child.wait(timeout=60)
        b.deinit()
