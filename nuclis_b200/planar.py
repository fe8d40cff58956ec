"""Host-side mirror of the load-time re-layout (`Backend.prepare`, csrc/prepare.cu) in numpy.

A loader that would rather re-lay a tensor on the host (to write a pre-laid file, or to check a device) gets the
same bytes here that `nu_cuda_matrix_prepare` writes on the device: every byte of the GGUF form is copied to a new
place, none is changed, and the result is as long as the input. `layout_of` is `prepared_layout` of the library:
the value to put in `Matrix.layout`, or 0 when the encoding (or the shape) keeps its GGUF rows.

The planar forms (rows a multiple of 16, columns a multiple of 256; a superblock is 256 columns):

  1  Q6_K    [rows][superblocks][208] records, then [superblocks][rows] f16 super-scales
  2  Q8_0    [rows][columns] int8 codes, then [columns/32][rows] f16 block scales
  3  Q5_0    [rows][superblocks][160]: 8 x 16 nibble bytes, 8 x 4 bytes of fifth bits; then [superblocks][rows][8] f16 d
  4  Q5_1    the same records; then [superblocks][rows][16] f16: eight d, eight m
  5  Q4_0, IQ4_NL   [rows][superblocks][128] nibble bytes; then [superblocks][rows][8] f16 d
  6  IQ4_XS  [rows][superblocks][128] nibble bytes; then [superblocks][rows][8]: the first eight bytes of each superblock
  7  Q2_K    [rows][superblocks][80]: scale and code bytes; then [superblocks][rows][4]: d, dmin
  8  Q3_K    [rows][superblocks][96]: mask and code bytes; then [superblocks][rows/16][224]: 16 x 12 scale bytes, 16 f16 d
"""
from __future__ import annotations

import numpy as np

from . import encoding as enc

_LAYOUTS = {enc.Q6_K: 1, enc.Q8_0: 2, enc.Q5_0: 3, enc.Q5_1: 4, enc.Q4_0: 5, enc.IQ4_NL: 5, enc.IQ4_XS: 6, enc.Q2_K: 7, enc.Q3_K: 8}


def layout_of(encoding: int, rows: int, columns: int) -> int:
    """The layout `relay` gives this matrix: 0 when it keeps its GGUF rows."""
    if rows % 16 or columns % 256:
        return 0
    return _LAYOUTS.get(encoding, 0)


def _planes(main: np.ndarray, tail: np.ndarray) -> np.ndarray:
    return np.concatenate([np.ascontiguousarray(main).reshape(-1), np.ascontiguousarray(tail).reshape(-1)])


def relay(encoding: int, data: np.ndarray, rows: int, columns: int) -> tuple[np.ndarray, int]:
    """The bytes `Backend.prepare` writes for the GGUF bytes ``data`` of a [rows][columns] matrix, and their layout."""
    data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    layout = layout_of(encoding, rows, columns)
    if layout == 0:
        return data.copy(), 0
    _, elements, size = enc.layout(encoding)
    per_row = columns // elements
    if data.size != rows * per_row * size:
        raise ValueError("data is not rows x columns of this encoding")
    blocks = data.reshape(rows, per_row, size)
    ksb = columns // 256
    if layout == 1:
        # a record: for t = 0..3 (half hh = t >> 1 of the block, column half ch = t & 1) 16 bytes of ql[hh*64 + 16ch ..],
        # 16 of ql[hh*64 + 32 + 16ch ..], 16 of qh[hh*32 + 16ch ..]; then the 16 scale bytes
        rec = np.empty((rows, ksb, 208), dtype=np.uint8)
        for t in range(4):
            hh, ch = t >> 1, t & 1
            rec[:, :, t * 48:t * 48 + 16] = blocks[:, :, hh * 64 + 16 * ch:hh * 64 + 16 * ch + 16]
            rec[:, :, t * 48 + 16:t * 48 + 32] = blocks[:, :, hh * 64 + 32 + 16 * ch:hh * 64 + 48 + 16 * ch]
            rec[:, :, t * 48 + 32:t * 48 + 48] = blocks[:, :, 128 + hh * 32 + 16 * ch:128 + hh * 32 + 16 * ch + 16]
        rec[:, :, 192:208] = blocks[:, :, 192:208]
        return _planes(rec, blocks[:, :, 208:210].transpose(1, 0, 2)), 1
    if layout == 2:
        return _planes(blocks[:, :, 2:34], blocks[:, :, 0:2].transpose(1, 0, 2)), 2
    if layout in (3, 4, 5):
        head = {3: 2, 4: 4, 5: 2}[layout]           # bytes of scales a block starts with
        high = 0 if layout == 5 else 4                # bytes of fifth bits behind them
        b8 = blocks.reshape(rows, ksb, 8, size)
        rec = np.empty((rows, ksb, 128 + 8 * high), dtype=np.uint8)
        rec[:, :, :128] = b8[:, :, :, head + high:].reshape(rows, ksb, 128)
        if high:
            rec[:, :, 128:] = b8[:, :, :, head:head + high].reshape(rows, ksb, 32)
        # scale plane: per (superblock, row) the eight d side by side, then (Q5_1) the eight m
        sc = b8[:, :, :, :head].reshape(rows, ksb, 8, head // 2, 2).transpose(1, 0, 3, 2, 4)
        return _planes(rec, sc), layout
    if layout == 6:
        return _planes(blocks[:, :, 8:136], blocks[:, :, 0:8].transpose(1, 0, 2)), 6
    if layout == 7:
        return _planes(blocks[:, :, 0:80], blocks[:, :, 80:84].transpose(1, 0, 2)), 7
    # layout 8
    tail = np.empty((ksb, rows // 16, 224), dtype=np.uint8)
    scales = blocks[:, :, 96:108].reshape(rows // 16, 16, ksb, 12).transpose(2, 0, 1, 3)   # [sb][tile][row in tile][12]
    d = blocks[:, :, 108:110].reshape(rows // 16, 16, ksb, 2).transpose(2, 0, 1, 3)
    tail[:, :, :192] = scales.reshape(ksb, rows // 16, 192)
    tail[:, :, 192:] = d.reshape(ksb, rows // 16, 32)
    return _planes(blocks[:, :, 0:96], tail), 8


def restore(encoding: int, planar: np.ndarray, rows: int, columns: int, layout: int) -> np.ndarray:
    """The GGUF bytes back from a planar form (the inverse of `relay`)."""
    planar = np.ascontiguousarray(planar, dtype=np.uint8).reshape(-1)
    if layout == 0:
        return planar.copy()
    if layout != layout_of(encoding, rows, columns):
        raise ValueError("not the layout of this encoding and shape")
    # every byte moves, none changes: relay applied to the byte positions tells where each one went
    _, elements, size = enc.layout(encoding)
    n = rows * (columns // elements) * size
    if planar.size != n:
        raise ValueError("planar data is not rows x columns of this encoding")
    # relay works on bytes; positions need more than 8 bits, so move them plane by plane of their base-256 digits
    out = np.empty(n, dtype=np.uint8)
    where = np.zeros(n, dtype=np.int64)
    index = np.arange(n, dtype=np.int64)
    for digit in range(4):
        moved, _ = relay(encoding, ((index >> (8 * digit)) & 0xff).astype(np.uint8), rows, columns)
        where |= moved.astype(np.int64) << (8 * digit)
    out[where] = planar
    return out
