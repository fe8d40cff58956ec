"""GGML storage layouts of the encodings this backend serves.

Mirrors ``layout`` of inference/src/tensor/encoding.zig:29-56 and
``validateRow`` of inference/src/quant/decode.zig:108-120 on the host, so that
descriptors can be sized before any device call.
"""
from __future__ import annotations

F32, F16, Q8_0, Q4_K, Q6_K, BF16 = 0, 1, 8, 12, 14, 30
Q4_0, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, IQ4_NL, IQ4_XS = 2, 6, 7, 10, 11, 13, 20, 23  # bit-exact generic decoders at any alignment; Q5_K, and the prepared forms of the others, also on the integer tensor path

LAYOUTS = {
    F32: ("F32", 1, 4),
    F16: ("F16", 1, 2),
    Q4_0: ("Q4_0", 32, 18),
    Q5_0: ("Q5_0", 32, 22),
    Q5_1: ("Q5_1", 32, 24),
    Q2_K: ("Q2_K", 256, 84),
    Q3_K: ("Q3_K", 256, 110),
    Q5_K: ("Q5_K", 256, 176),
    Q8_0: ("Q8_0", 32, 34),
    Q4_K: ("Q4_K", 256, 144),
    Q6_K: ("Q6_K", 256, 210),
    IQ4_NL: ("IQ4_NL", 32, 18),
    IQ4_XS: ("IQ4_XS", 256, 136),
    BF16: ("BF16", 1, 2),
}


def layout(encoding: int) -> tuple[str, int, int]:
    """(name, elements per block, bytes per block); KeyError for an unknown id."""
    return LAYOUTS[encoding]


def row_bytes(encoding: int, columns: int) -> int:
    """Bytes of one row of ``columns`` values; the row must hold whole blocks."""
    _, elements, size = LAYOUTS[encoding]
    if columns == 0 or columns % elements:
        raise ValueError(f"{columns} columns are not whole {LAYOUTS[encoding][0]} blocks")
    return columns // elements * size


def matrix_bytes(encoding: int, rows: int, columns: int) -> int:
    return rows * row_bytes(encoding, columns)


def bits_per_weight(encoding: int) -> float:
    _, elements, size = LAYOUTS[encoding]
    return 8.0 * size / elements
