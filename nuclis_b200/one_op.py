"""Runs one matmul operator a few times on synthetic data: the small, self-contained case to put under a profiler.

    python -m nuclis_b200.one_op ENCODING ROWS COLUMNS TOKENS [--prepare] [--bf16]

Three distinct copies of the weights are used in turn, each in its own recording, so that a
profiler can skip the first launch (``-s 1``) and still see a cold matrix.
"""
import sys

import numpy as np

from . import Backend, Matrix, encoding as enc, synth


def main(argv):
    encoding, rows, columns, tokens = (int(a) for a in argv[:4])
    prepare, bf16 = "--prepare" in argv, "--bf16" in argv
    b = Backend(0)
    nbytes = enc.matrix_bytes(encoding, rows, columns)
    w = synth.matrix(encoding, rows, columns, seed=1)
    m = Matrix(encoding, rows, columns, nbytes)
    copies = []
    for _ in range(3):
        wb = b.create(nbytes)
        wb.write(w)
        mm = m
        if prepare:
            pb, mm = b.prepare(wb, m)
            b.release(wb)
            wb = pb
        copies.append((wb, mm))
    padded = Backend.matmul_padded(tokens) if tokens > 8 else tokens
    x = synth.activations(tokens, columns, 2)
    if bf16:
        bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
        xin = np.zeros((padded, columns), dtype=np.uint16)
        xin[:tokens] = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    else:
        xin = np.zeros((padded, columns), dtype=np.float32)
        xin[:tokens] = x
    xb = b.create(xin.nbytes)
    xb.write(xin)
    yb = b.create(padded * rows * 4)
    for wb, mm in copies:
        b.begin()
        if tokens == 1:
            b.matvec(wb, mm, xb, yb)
        elif tokens <= 8:
            b.matvec_rows(wb, mm, xb, columns, yb, rows, tokens)
        else:
            b.matmul(wb, mm, xb, columns, yb, rows, tokens, in_dtype=enc.BF16 if bf16 else enc.F32)
        b.commit()
    print("ok", float(yb.floats()[0]))
    b.deinit()


if __name__ == "__main__":
    main(sys.argv[1:])
