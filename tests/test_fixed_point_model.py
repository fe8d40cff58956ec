"""A numpy model of the arithmetic of the integer-path kernels (csrc/i8_kernel.cuh, i8_q4k.cuh), checked against the CPU
oracle: what the scheme itself costs in accuracy, apart from any kernel.

Per token and superblock of 256 columns the activations are scaled by the power of two that puts their largest magnitude
in [2^21, 2^22), rounded to integers X, and cut into three balanced base-256 digits (signed bytes). The tensor core
multiplies the 4-bit codes with each digit plane exactly (int32); the 6-bit group scales multiply those sums as integers;
the planes are recombined with their weights in F32; the minima meet the group sums of X, which travel as two fp16
pieces (hi + lo) scaled by 2^-12. The only roundings are the one to X (2^-22 of the superblock's largest activation), the
fp16 pieces of the group sums (2^-22 relative) and the F32 sums over the superblocks."""
import numpy as np
import pytest

import oracle
from nuclis_b200 import encoding as enc, synth
from parity import assert_matvec_close


def q4k_fields(data: np.ndarray, rows: int, columns: int):
    """d, dmin [rows][sb]; scales, minima [rows][sb][8]; codes [rows][sb][8][32] of a Q4_K matrix (decode.zig:147-170)."""
    b = data.reshape(rows, columns // 256, 144)
    d = b[:, :, 0:2].copy().view(np.float16)[..., 0].astype(np.float32)
    dmin = b[:, :, 2:4].copy().view(np.float16)[..., 0].astype(np.float32)
    sc = b[:, :, 4:16].astype(np.int32)
    scales = np.empty(b.shape[:2] + (8,), dtype=np.int32)
    minima = np.empty_like(scales)
    for g in range(8):
        if g < 4:
            scales[..., g] = sc[..., g] & 63
            minima[..., g] = sc[..., g + 4] & 63
        else:
            scales[..., g] = (sc[..., g + 4] & 15) | ((sc[..., g - 4] >> 6) << 4)
            minima[..., g] = (sc[..., g + 4] >> 4) | ((sc[..., g] >> 6) << 4)
    qs = b[:, :, 16:144].reshape(rows, -1, 4, 32).astype(np.int32)
    codes = np.empty(b.shape[:2] + (8, 32), dtype=np.int32)
    codes[:, :, 0::2] = qs & 15
    codes[:, :, 1::2] = qs >> 4
    return d, dmin, scales, minima, codes


def stage(x: np.ndarray):
    """The staging pass: per superblock the integers X (as three balanced digit planes), 1 / scale, and the group sums of X as
    the fp16 pieces the kernel keeps."""
    xs = x.reshape(-1, 256).astype(np.float32)
    mx = np.abs(xs).max(axis=1)
    e = (mx.view(np.uint32) >> 23) & 0xff
    ok = (e >= 22) & (e < 255)
    ee = np.where(ok, e, 148).astype(np.int32)        # (a superblock that is not staged: any exponent, its factors are zero)
    scale = np.where(ok, np.ldexp(np.float32(1), 148 - ee), 0).astype(np.float32)   # 2^(275 - e - 127)
    inv = np.where(ok, np.ldexp(np.float32(1), ee - 148), 0).astype(np.float32)
    X = np.rint(xs * scale[:, None]).astype(np.int64)
    assert np.abs(X).max() < 2 ** 22
    y = X + 0x808080                                  # the balanced digits of X are the bytes of X + 0x808080, each less 128
    digits = np.stack([((y >> (8 * i)) & 0xff) - 128 for i in range(3)], axis=0)
    assert np.array_equal((digits * np.array([1, 256, 65536])[:, None, None]).sum(axis=0), X)
    assert digits.min() >= -128 and digits.max() <= 127
    gsum = X.reshape(-1, 8, 32).sum(axis=2).astype(np.float32) * np.float32(2.0 ** -12)
    hi = gsum.astype(np.float16)
    lo = (gsum - hi.astype(np.float32)).astype(np.float16)
    return digits, inv, hi, lo


def model_matvec(data: np.ndarray, rows: int, columns: int, x: np.ndarray) -> np.ndarray:
    d, dmin, scales, minima, codes = q4k_fields(data, rows, columns)
    digits, inv, hi, lo = stage(x)
    planes = digits.reshape(3, -1, 8, 32)             # [plane][sb][group][32]
    # exact integer sums per plane and group, the group scale as an integer factor (int32 in the kernel: below 2^29)
    sums = np.einsum("rsgc,psgc->prsg", codes, planes) * scales[None]
    per_plane = sums.sum(axis=3)
    assert np.abs(per_plane).max() < 2 ** 31
    weights = np.array([1.0, 256.0, 65536.0], dtype=np.float32)
    f = (per_plane.astype(np.float32) * weights[:, None, None]).sum(axis=0, dtype=np.float32)      # F32, as the kernel recombines
    cm = (minima.astype(np.float32) * (hi.astype(np.float32) + lo.astype(np.float32))[None]).sum(axis=2, dtype=np.float32)
    acc = np.zeros(rows, dtype=np.float32)
    for s in range(columns // 256):                   # the kernel adds a superblock's two terms into an F32 accumulator
        acc = acc + f[:, s] * (d[:, s] * inv[s])
        acc = acc + cm[:, s] * (np.float32(-4096.0) * dmin[:, s] * inv[s])
    return acc


@pytest.mark.parametrize("shape", [(64, 1024), (96, 5120)])
@pytest.mark.parametrize("spread", [1.0, 1e6])
def test_the_scheme_holds_the_matvec_bound(shape, spread):
    rows, columns = shape
    data = synth.matrix(enc.Q4_K, rows, columns, seed=columns)
    x = synth.activations(1, columns, seed=rows)[0]
    x[::7] *= np.float32(spread)                       # superblocks with outliers: the scale follows the largest value
    got = model_matvec(data, rows, columns, x)
    want = oracle.matvec(enc.Q4_K, rows, columns, data, x)
    mag = oracle.matvec_abs(enc.Q4_K, rows, columns, data, x)
    assert_matvec_close(got, want, mag, f"model {shape} spread {spread}")
    # outliers a million times the rest cost the small values of their superblock precision: still an order inside 1e-5
    assert np.linalg.norm(got - want) <= (1e-6 if spread == 1.0 else 3e-6) * np.linalg.norm(want)


def test_small_and_special_superblocks():
    # a superblock of zeros (and one below 2^-105) is staged as zeros; the digits of the extremes stay signed bytes
    x = np.zeros(512, dtype=np.float32)
    x[256:] = np.float32(2.0 ** -120)
    digits, inv, hi, lo = stage(x)
    assert not digits.any() and not inv.any() and not hi.any() and not lo.any()
    x = np.full(256, -1.0, dtype=np.float32)
    x[3] = 1.0
    digits, inv, _, _ = stage(x)
    X = (digits * np.array([1, 256, 65536])[:, None, None]).sum(axis=0)[0]
    assert X[3] == 2 ** 21 and X[0] == -2 ** 21 and inv[0] == np.float32(2.0 ** -21)
