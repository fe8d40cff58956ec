"""Row-split tensor parallelism of one decoder layer's projections: shard tables and byte slicing.

The reference is single-device; this is new design. Column-parallel matrices
(QKV, gate, up) are split along their rows, row-parallel ones (O, down) along K
at 256-column superblock granularity so that each GPU consumes exactly the
slice of the intermediate it produced; the row-parallel outputs are partial sums
that an allreduce completes. A block-quantized row cannot be cut inside a
block, hence the superblock granularity (68 superblocks over 8 GPUs give
8,9,8,9,... not 8.5 each).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import encoding as enc


def split_counts(total: int, parts: int) -> list[int]:
    """``total`` items over ``parts`` ranks, as even as whole items allow: floor((i+1)t/p) - floor(it/p)."""
    return [(i + 1) * total // parts - i * total // parts for i in range(parts)]


def split_ranges(total: int, parts: int) -> list[tuple[int, int]]:
    return [(i * total // parts, (i + 1) * total // parts) for i in range(parts)]


def expert_range(experts: int, ranks: int, rank: int) -> tuple[int, int]:
    """Experts [first, end) a rank holds under expert parallelism: contiguous, as even as the count allows."""
    if not 0 <= rank < ranks or experts < ranks:
        raise ValueError(f"{experts} experts over {ranks} ranks, rank {rank}")
    return split_ranges(experts, ranks)[rank]


@dataclass(frozen=True)
class LayerShapes:
    """Full (unsharded) shapes of the synthetic dense decoder layer."""
    hidden: int = 5120
    ffn: int = 17408
    kv: int = 1024          # rows of K and of V in the fused QKV projection
    qkv_encoding: int = enc.Q4_K
    o_encoding: int = enc.Q4_K
    gate_up_encoding: int = enc.Q4_K
    down_encoding: int = enc.Q6_K

    @property
    def qkv_rows(self) -> int:
        return self.hidden + 2 * self.kv


@dataclass(frozen=True)
class RankShapes:
    """What one rank holds: rows of the column-parallel matrices, K of the row-parallel ones."""
    rank: int
    ranks: int
    q_rows: int        # Q rows of QKV = K of O on this rank
    kv_rows: int       # K rows (and V rows) of QKV on this rank
    ffn_rows: int      # gate and up rows = K of down on this rank
    q_range: tuple[int, int]
    kv_range: tuple[int, int]
    ffn_range: tuple[int, int]

    @property
    def qkv_rows(self) -> int:
        return self.q_rows + 2 * self.kv_rows


def rank_shapes(shapes: LayerShapes, ranks: int, rank: int) -> RankShapes:
    if shapes.hidden % 256 or shapes.ffn % 256:
        raise ValueError("hidden and ffn must be whole superblocks")
    if shapes.kv % ranks:
        raise ValueError("K/V rows must divide over the ranks")
    q0, q1 = split_ranges(shapes.hidden // 256, ranks)[rank]
    f0, f1 = split_ranges(shapes.ffn // 256, ranks)[rank]
    kv = shapes.kv // ranks
    return RankShapes(rank, ranks, (q1 - q0) * 256, kv, (f1 - f0) * 256,
                      (q0 * 256, q1 * 256), (rank * kv, (rank + 1) * kv), (f0 * 256, f1 * 256))


def balance(total: int, ranks: int) -> float:
    """Mean share over largest share of ``total`` superblocks: the efficiency bound of the split."""
    counts = split_counts(total, ranks)
    return (total / ranks) / max(counts)


def slice_rows(data: np.ndarray, encoding: int, rows: int, columns: int, r0: int, r1: int) -> np.ndarray:
    """Rows [r0, r1) of a row-major encoded matrix: a contiguous byte range."""
    stride = enc.row_bytes(encoding, columns)
    assert data.size == rows * stride and 0 <= r0 <= r1 <= rows
    return data[r0 * stride: r1 * stride]


def slice_columns(data: np.ndarray, encoding: int, rows: int, columns: int, c0: int, c1: int) -> np.ndarray:
    """Columns [c0, c1) of every row, gathered into a contiguous [rows][c1-c0] matrix.
    The cut must fall on block boundaries; bytes are copied, values unchanged."""
    _, elements, size = enc.layout(encoding)
    if c0 % elements or c1 % elements:
        raise ValueError("a column split must fall on block boundaries")
    stride = enc.row_bytes(encoding, columns)
    b0, b1 = c0 // elements * size, c1 // elements * size
    return np.ascontiguousarray(data.reshape(rows, stride)[:, b0:b1]).reshape(-1)
