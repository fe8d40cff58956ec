"""Shared helpers of the GPU parity tests: acceptance formulas and small fixtures."""
import numpy as np

import oracle
from nuclis_b200 import Matrix, encoding as enc, synth


def rel_l2(got, want) -> float:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    denom = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / denom) if denom > 0 else float(np.linalg.norm(got))


def assert_matvec_close(got, want, magnitude, what="", rel=1e-5, per_element=4e-6):
    """The reference's acceptance for F32 kernels against the F64 CPU result: every element within
    ``4e-6 * sum|w*x| + 1e-6`` (inference/metal-check.zig:3976), and the stated bound on the
    relative L2 error of the whole output (1e-5 for F32 accumulation)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    bound = per_element * np.asarray(magnitude, dtype=np.float64) + 1e-6
    worst = np.max(np.abs(got - want) / bound)
    assert worst <= 1.0, f"{what}: element error {worst:.3f}x the bound"
    r = rel_l2(got, want)
    assert r <= rel, f"{what}: relative L2 {r:.3e} > {rel}"


def make_case(encoding, rows, columns, tokens, seed):
    w = synth.matrix(encoding, rows, columns, seed)
    x = synth.activations(tokens, columns, seed + 1)
    return w, x, Matrix(encoding, rows, columns, w.size)


def expect(encoding, rows, columns, w, x):
    want = oracle.matmul(encoding, rows, columns, w, x)
    mag = np.stack([oracle.matvec_abs(encoding, rows, columns, w, x[t]) for t in range(x.shape[0])])
    return want, mag


def tiled_fixture_matrix(row, rows, columns):
    """A matrix of ``rows`` x ``columns`` whose rows are the golden row's blocks tiled, each row
    starting one block later than the previous (the construction of the reference's wide-row
    checks, inference/metal-check.zig:284-297)."""
    _, elements, size = enc.layout(row["encoding"])
    blocks = row["bytes"].reshape(-1, size)
    per_row = columns // elements
    out = np.empty((rows, per_row, size), dtype=np.uint8)
    for r in range(rows):
        idx = (np.arange(per_row) + r) % blocks.shape[0]
        out[r] = blocks[idx]
    return out.reshape(-1)
