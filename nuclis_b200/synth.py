"""Seeded synthetic GGUF blocks with the value distributions of the benchmark configs.

Every field of a block is a legal code drawn at random and only the scales are
calibrated, which is how the reference fills its own generated models
(inference/src/quant/sample.zig:1-8, 51-69).

  Q4_K  d = f16(|N(0,1)| * 1e-3), dmin = f16(|N(0,1)| * 5e-4); 12 uniform bytes of packed
        6-bit scales and minima (the packing is a bijection from 96 bits to sixteen 6-bit
        fields, so uniform bytes give uniform [0,63] fields); 128 uniform quant bytes.
  Q6_K  128 + 64 uniform bytes of low/high code bits; 16 int8 sub-scales uniform in
        [-32,31]; d = f16(|N(0,1)| * 1e-3).
  Q8_0  d = f16(|N(0,1)| * 2e-3); 32 int8 codes uniform in [-127,127].

The numpy generators serve tests and small cases. ``*_torch`` fill device
memory directly for the large benchmark tensors (13 GB would take minutes
through the host); they draw from the same distributions with torch's
generator, so the two give different bytes for the same seed.
"""
from __future__ import annotations

import numpy as np

from . import encoding as enc


def _abs_normal_f16(rng: np.random.Generator, n: int, scale: float) -> np.ndarray:
    return (np.abs(rng.standard_normal(n, dtype=np.float32)) * np.float32(scale)).astype("<f2").view(np.uint8).reshape(n, 2)


def q4_k(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/256 * 144] bytes. Draw order: all d, all dmin, all scale bytes, all quants."""
    blocks = rows * (columns // 256)
    out = np.empty((blocks, 144), dtype=np.uint8)
    out[:, 0:2] = _abs_normal_f16(rng, blocks, 1e-3)
    out[:, 2:4] = _abs_normal_f16(rng, blocks, 5e-4)
    out[:, 4:16] = rng.integers(0, 256, size=(blocks, 12), dtype=np.uint8)
    out[:, 16:144] = rng.integers(0, 256, size=(blocks, 128), dtype=np.uint8)
    return out.reshape(-1)


def q6_k(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/256 * 210] bytes. Draw order: code bits, sub-scales, d."""
    blocks = rows * (columns // 256)
    out = np.empty((blocks, 210), dtype=np.uint8)
    out[:, 0:192] = rng.integers(0, 256, size=(blocks, 192), dtype=np.uint8)
    out[:, 192:208] = rng.integers(-32, 32, size=(blocks, 16), dtype=np.int8).view(np.uint8)
    out[:, 208:210] = _abs_normal_f16(rng, blocks, 1e-3)
    return out.reshape(-1)


def q8_0(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/32 * 34] bytes. Draw order: d, codes."""
    blocks = rows * (columns // 32)
    out = np.empty((blocks, 34), dtype=np.uint8)
    out[:, 0:2] = _abs_normal_f16(rng, blocks, 2e-3)
    out[:, 2:34] = rng.integers(-127, 128, size=(blocks, 32), dtype=np.int8).view(np.uint8)
    return out.reshape(-1)


def q4_0(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/32 * 18] bytes. Draw order: d, nibbles."""
    blocks = rows * (columns // 32)
    out = np.empty((blocks, 18), dtype=np.uint8)
    out[:, 0:2] = _abs_normal_f16(rng, blocks, 2e-2)
    out[:, 2:18] = rng.integers(0, 256, size=(blocks, 16), dtype=np.uint8)
    return out.reshape(-1)


def q5_0(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/32 * 22] bytes. Draw order: d, the plane of fifth bits, nibbles."""
    blocks = rows * (columns // 32)
    out = np.empty((blocks, 22), dtype=np.uint8)
    out[:, 0:2] = _abs_normal_f16(rng, blocks, 1e-2)
    out[:, 2:22] = rng.integers(0, 256, size=(blocks, 20), dtype=np.uint8)
    return out.reshape(-1)


def q5_1(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/32 * 24] bytes. Draw order: d, m, the plane of fifth bits, nibbles."""
    blocks = rows * (columns // 32)
    out = np.empty((blocks, 24), dtype=np.uint8)
    out[:, 0:2] = _abs_normal_f16(rng, blocks, 1e-2)
    out[:, 2:4] = _abs_normal_f16(rng, blocks, 1e-1)
    out[:, 4:24] = rng.integers(0, 256, size=(blocks, 20), dtype=np.uint8)
    return out.reshape(-1)


def q5_k(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/256 * 176] bytes. Draw order: d, dmin, scale bytes, fifth bits and nibbles."""
    blocks = rows * (columns // 256)
    out = np.empty((blocks, 176), dtype=np.uint8)
    out[:, 0:2] = _abs_normal_f16(rng, blocks, 5e-4)
    out[:, 2:4] = _abs_normal_f16(rng, blocks, 5e-4)
    out[:, 4:176] = rng.integers(0, 256, size=(blocks, 172), dtype=np.uint8)
    return out.reshape(-1)


def q2_k(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/256 * 84] bytes. Draw order: scale bytes and codes, d, dmin."""
    blocks = rows * (columns // 256)
    out = np.empty((blocks, 84), dtype=np.uint8)
    out[:, 0:80] = rng.integers(0, 256, size=(blocks, 80), dtype=np.uint8)
    out[:, 80:82] = _abs_normal_f16(rng, blocks, 5e-3)
    out[:, 82:84] = _abs_normal_f16(rng, blocks, 5e-3)
    return out.reshape(-1)


def q3_k(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/256 * 110] bytes. Draw order: high-bit mask, codes and scale bytes, d."""
    blocks = rows * (columns // 256)
    out = np.empty((blocks, 110), dtype=np.uint8)
    out[:, 0:108] = rng.integers(0, 256, size=(blocks, 108), dtype=np.uint8)
    out[:, 108:110] = _abs_normal_f16(rng, blocks, 1e-3)
    return out.reshape(-1)


def iq4_nl(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/32 * 18] bytes. Draw order: d, codes."""
    blocks = rows * (columns // 32)
    out = np.empty((blocks, 18), dtype=np.uint8)
    out[:, 0:2] = _abs_normal_f16(rng, blocks, 2e-4)
    out[:, 2:18] = rng.integers(0, 256, size=(blocks, 16), dtype=np.uint8)
    return out.reshape(-1)


def iq4_xs(rng: np.random.Generator, rows: int, columns: int) -> np.ndarray:
    """[rows * columns/256 * 136] bytes. Draw order: d, scale bits and codes."""
    blocks = rows * (columns // 256)
    out = np.empty((blocks, 136), dtype=np.uint8)
    out[:, 0:2] = _abs_normal_f16(rng, blocks, 1e-5)
    out[:, 2:136] = rng.integers(0, 256, size=(blocks, 134), dtype=np.uint8)
    return out.reshape(-1)


GENERATORS = {enc.IQ4_NL: iq4_nl, enc.IQ4_XS: iq4_xs, enc.Q2_K: q2_k, enc.Q3_K: q3_k, enc.Q4_K: q4_k, enc.Q6_K: q6_k, enc.Q8_0: q8_0, enc.Q4_0: q4_0, enc.Q5_0: q5_0, enc.Q5_1: q5_1, enc.Q5_K: q5_k}


def matrix(encoding: int, rows: int, columns: int, seed: int) -> np.ndarray:
    """Bytes of a ``rows`` x ``columns`` matrix in ``encoding``, everything from ``seed``."""
    return GENERATORS[encoding](np.random.default_rng(seed), rows, columns)


def activations(tokens: int, columns: int, seed: int) -> np.ndarray:
    """F32 [tokens][columns] drawn from N(0,1)."""
    return np.random.default_rng(seed).standard_normal((tokens, columns), dtype=np.float32)


def fill_matrix_torch(dst, encoding: int, rows: int, columns: int, seed: int) -> None:
    """Fills the uint8 CUDA tensor ``dst`` (matrix_bytes long) in place on its device."""
    import torch

    gen = torch.Generator(device=dst.device)
    gen.manual_seed(seed)
    _, elements, size = enc.layout(encoding)
    blocks = rows * (columns // elements)
    view = dst[: blocks * size].view(blocks, size)
    # random_ over the whole tensor gives uniform bytes; the calibrated fields are overwritten below
    view.random_(0, 256, generator=gen)

    def scales(n, s):
        return (torch.randn(n, device=dst.device, generator=gen).abs() * s).to(torch.float16).view(torch.uint8).view(n, 2)

    if encoding == enc.Q4_K:
        view[:, 0:2] = scales(blocks, 1e-3)
        view[:, 2:4] = scales(blocks, 5e-4)
    elif encoding == enc.Q6_K:
        sub = torch.randint(-32, 32, (blocks, 16), device=dst.device, generator=gen, dtype=torch.int8)
        view[:, 192:208] = sub.view(torch.uint8)
        view[:, 208:210] = scales(blocks, 1e-3)
    elif encoding == enc.Q8_0:
        codes = torch.randint(-127, 128, (blocks, 32), device=dst.device, generator=gen, dtype=torch.int8)
        view[:, 2:34] = codes.view(torch.uint8)
        view[:, 0:2] = scales(blocks, 2e-3)
    elif encoding == enc.Q5_K:
        view[:, 0:2] = scales(blocks, 1e-3)
        view[:, 2:4] = scales(blocks, 5e-4)
    elif encoding in (enc.Q4_0, enc.Q5_0, enc.IQ4_NL, enc.IQ4_XS):
        view[:, 0:2] = scales(blocks, 2e-3)   # d leads the block; the other bytes are codes and scale bits, all values legal
    elif encoding == enc.Q5_1:
        view[:, 0:2] = scales(blocks, 2e-3)
        view[:, 2:4] = scales(blocks, 1e-2)
    elif encoding == enc.Q2_K:
        view[:, 80:82] = scales(blocks, 5e-3)
        view[:, 82:84] = scales(blocks, 5e-3)
    elif encoding == enc.Q3_K:
        view[:, 108:110] = scales(blocks, 2e-3)
    else:
        raise ValueError(f"no generator for encoding {encoding}")
