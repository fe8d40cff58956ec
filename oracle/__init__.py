"""CPU oracle (test infrastructure): ctypes access to ``libnu_oracle.so``.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import
this package. The product (``nuclis_b200``) never does.
"""
from .ref import (  # noqa: F401
    OK, UNSUPPORTED_ENCODING, INVALID_ROW_LENGTH, INVALID_BYTE_LENGTH, INVALID_SHAPE,
    SCRATCH_TOO_SMALL, INVALID_EXPERT, NON_FINITE,
    OracleError, build, layout, validate_row, row, matvec, matvec_abs, matmul, gelu, silu, rms_norm, route, ffn,
)
