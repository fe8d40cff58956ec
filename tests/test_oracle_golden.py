"""Pins the CPU oracle to the reference's own golden vectors and hand-computed blocks.

Sources of the expectations (paths inside the reference tree):
  * tests/golden/quant_rows.json: rows of inference/src/quant/fixtures/*.json, which
    inference/src/quant/decode.zig:587-592 requires exactly, on deliberately unaligned input;
  * hand-computed blocks of decode.zig:455-473 (Q8_0), :692-704 (Q6_K), :754-764 (Q4_K);
  * error paths of decode.zig:566-585;
  * cpu.matvec known answers of inference/src/backends/cpu/root.zig:167-201, 203-236, 238-298;
  * routing and expert FFN of inference/src/backends/cpu/experts.zig:135-216.
"""
import struct

import numpy as np
import pytest

import oracle


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


def test_layouts():
    assert oracle.layout(12) == (256, 144)
    assert oracle.layout(14) == (256, 210)
    assert oracle.layout(8) == (32, 34)
    assert oracle.layout(0) == (1, 4) and oracle.layout(1) == (1, 2) and oracle.layout(30) == (1, 2)
    assert oracle.layout(2) == (32, 18) and oracle.layout(6) == (32, 22) and oracle.layout(7) == (32, 24) and oracle.layout(13) == (256, 176)
    assert oracle.layout(10) == (256, 84) and oracle.layout(11) == (256, 110)
    assert oracle.layout(20) == (32, 18) and oracle.layout(23) == (256, 136)
    with pytest.raises(oracle.OracleError):
        oracle.layout(999)


def test_golden_rows_exact_on_unaligned_input(golden_rows):
    assert {r["encoding"] for r in golden_rows} == {2, 6, 7, 8, 10, 11, 12, 13, 14, 20, 23}
    for r in golden_rows:
        shifted = np.empty(r["bytes"].size + 1, dtype=np.uint8)
        shifted[1:] = r["bytes"]
        got = oracle.row(r["encoding"], shifted[1:], r["values"].size)
        assert np.array_equal(bits(got), bits(r["values"])), r["name"]


def test_q8_0_signed_extremes_and_block_scales():
    b = np.zeros(68, dtype=np.uint8)
    b[1] = 0x38  # f16 0.5
    b[2], b[3], b[4] = 0x80, 0xFF, 0x7F
    b[35] = 0xC0  # f16 -2
    b[36] = 3
    b[67] = 0xFE
    want = np.zeros(64, dtype=np.float32)
    want[0], want[1], want[2], want[32], want[63] = -64, -0.5, 63.5, -6, 4
    assert np.array_equal(oracle.row(8, b, 64), want)


def test_q4_k_six_bit_coefficients_every_group():
    b = np.full(144, 0xA3, dtype=np.uint8)
    b[0:4] = [0, 0x38, 0, 0x34]  # d=0.5, dmin=0.25
    b[4:16] = [0xC1, 0x82, 0x43, 4, 0x45, 0x86, 0xC7, 8, 0x91, 0xA2, 0xB3, 0xC4]
    expected = np.array([0.25, 8.5, 2.75, 18, 67.25, 159.5, 13.75, 17], dtype=np.float32)
    got = oracle.row(12, b, 256)
    assert np.array_equal(got, np.repeat(expected, 32))


def test_q6_k_signed_scale_extremes_and_quarter_order():
    b = np.full(210, 0xF0, dtype=np.uint8)
    b[128:192] = 0xE4
    scales = np.array([-128, 127, -1, 0, 1, 2, -3, 4, 5, -6, 7, -8, 9, -10, 11, -12], dtype=np.int8)
    b[192:208] = scales.view(np.uint8)
    b[208:210] = [0, 0x38]  # d=0.5
    codes = np.array([-32, -16, 15, 31], dtype=np.float32)
    got = oracle.row(14, b, 256)
    i = np.arange(256)
    want = np.float32(0.5) * scales[i // 16].astype(np.float32) * codes[(i // 32) % 4]
    assert np.array_equal(got, want.astype(np.float32))


def test_f32_f16_bf16_edge_values():
    single = np.array([99, 0, 0, 0xC0, 0x3F, 0, 0, 0x10, 0xC0], dtype=np.uint8)
    assert np.array_equal(oracle.row(0, single[1:], 2), np.array([1.5, -2.25], dtype=np.float32))
    halves = np.array([0, 0x80, 1, 0, 0, 0x3E, 0xFF, 0x7B, 0, 0x7C, 0, 0x7E], dtype=np.uint8)
    got = oracle.row(1, halves, 6)
    assert bits(got)[0] == 0x80000000
    assert got[1] == np.float32(2.0 ** -24) and got[2] == 1.5 and got[3] == 65504
    assert np.isposinf(got[4]) and np.isnan(got[5])
    bf = np.array([0x80, 0x3F, 0x00, 0xC0], dtype=np.uint8)
    assert np.array_equal(oracle.row(30, bf, 2), np.array([1.0, -2.0], dtype=np.float32))


def test_invalid_rows_leave_output_untouched():
    zeros = np.zeros(420, dtype=np.uint8)
    out = np.full(512, 123, dtype=np.float32)
    for enc in (0, 1, 8, 12, 14, 30):
        n, size = oracle.layout(enc)

        def fails(code, data, elements):
            with pytest.raises(oracle.OracleError) as e:
                oracle.row(enc, data, elements, out=out)
            assert e.value.code == code

        fails(oracle.INVALID_ROW_LENGTH, zeros[:0], 0)
        fails(oracle.INVALID_BYTE_LENGTH, zeros[: size - 1], n)
        fails(oracle.INVALID_BYTE_LENGTH, zeros[: size + 1], n)
        fails(oracle.INVALID_BYTE_LENGTH, zeros[:size], n * 2)
        fails(oracle.INVALID_BYTE_LENGTH, zeros[: size * 2], n)
        if n > 1:
            fails(oracle.INVALID_ROW_LENGTH, zeros[:size], n - 1)
    with pytest.raises(oracle.OracleError) as e:
        oracle.row(8, zeros[:34], 31, out=out)
    assert e.value.code == oracle.INVALID_ROW_LENGTH
    for enc in (999, 34):
        with pytest.raises(oracle.OracleError) as e:
            oracle.row(enc, zeros[:0], 512, out=out)
        assert e.value.code == oracle.UNSUPPORTED_ENCODING
    assert np.all(out == 123)
    # Q6_K rows must be whole 256-value superblocks: 704 columns is not a row (2.75 blocks).
    with pytest.raises(oracle.OracleError) as e:
        oracle.validate_row(14, 210 * 3, 704)
    assert e.value.code == oracle.INVALID_ROW_LENGTH


def test_matvec_rectangular_f32_and_f16():
    m = np.array([1, 2, 3, -4, 5, -6], dtype="<f4").view(np.uint8)
    got = oracle.matvec(0, 2, 3, m, np.array([2, -1, 0.5], dtype=np.float32))
    assert np.array_equal(got, np.array([1.5, -16], dtype=np.float32))
    halves = np.array([0, 0x38, 0, 0xC0], dtype=np.uint8)  # 0.5, -2
    assert oracle.matvec(1, 1, 2, halves, np.array([-4, 3], dtype=np.float32))[0] == -8


def test_matvec_f64_accumulation_keeps_small_terms():
    m = np.array([2.0 ** 24, 1, -(2.0 ** 24)], dtype="<f4").view(np.uint8)
    assert oracle.matvec(0, 1, 3, m, np.ones(3, dtype=np.float32))[0] == 1


def test_matvec_q8_multiple_blocks_per_row():
    b = np.ones(136, dtype=np.uint8)
    for i, scale in enumerate([0x3800, 0x4000, 0xBC00, 0x3400]):
        b[i * 34: i * 34 + 2] = np.frombuffer(struct.pack("<H", scale), dtype=np.uint8)
    x = np.ones(64, dtype=np.float32)
    x[32:] = -2
    assert np.array_equal(oracle.matvec(8, 2, 64, b, x), np.array([-112, -48], dtype=np.float32))


def test_matvec_invalid_descriptors_leave_output_untouched():
    out = np.full(2, 123, dtype=np.float32)
    zeros = np.zeros(68, dtype=np.uint8)
    x = np.zeros(256, dtype=np.float32)

    def fails(code, enc, rows, cols, data, xin, o, scratch_len=None):
        with pytest.raises(oracle.OracleError) as e:
            oracle.matvec(enc, rows, cols, data, xin, out=o, scratch_len=scratch_len, tasks=1)
        assert e.value.code == code

    fails(oracle.INVALID_SHAPE, 8, 0, 32, zeros, x[:32], out)
    fails(oracle.INVALID_SHAPE, 8, 2, 0, zeros, x[:0], out)
    fails(oracle.INVALID_SHAPE, 8, 2, 32, zeros, x[:31], out)
    fails(oracle.INVALID_SHAPE, 8, 2, 32, zeros, x[:32], out[:1])
    fails(oracle.SCRATCH_TOO_SMALL, 8, 2, 32, zeros, x[:32], out, scratch_len=31)
    fails(oracle.INVALID_BYTE_LENGTH, 8, 2, 32, zeros[:67], x[:32], out)
    fails(oracle.INVALID_BYTE_LENGTH, 8, 2, 32, zeros[:66], x[:32], out)
    fails(oracle.INVALID_ROW_LENGTH, 8, 2, 16, zeros[:34], x[:16], out)
    fails(oracle.UNSUPPORTED_ENCODING, 999, 2, 32, zeros, x[:32], out)
    assert np.all(out == 123)


def test_basis_vectors_select_golden_columns(golden_rows):
    for r in golden_rows:
        columns, _ = oracle.layout(r["encoding"])
        rows = r["values"].size // columns
        for column in (0, columns // 2 + 1, columns - 1):
            x = np.zeros(columns, dtype=np.float32)
            x[column] = 1
            got = oracle.matvec(r["encoding"], rows, columns, r["bytes"], x)
            # value equality, as the reference's expectEqual: a sum that starts at +0 turns -0 into +0
            assert np.array_equal(got, r["values"].reshape(rows, columns)[:, column])


def test_rows_split_across_tasks_give_the_same_bits():
    rng = np.random.default_rng(19)
    rows, columns = 300, 512
    b = rng.integers(0, 256, size=rows * 16 * 34, dtype=np.uint8)
    scales = (rng.random(rows * 16, dtype=np.float32) - 0.5).astype("<f2").view(np.uint8).reshape(-1, 2)
    b.reshape(-1, 34)[:, :2] = scales
    x = (rng.random(columns, dtype=np.float32) * 2 - 1).astype(np.float32)
    serial = oracle.matvec(8, rows, columns, b, x, tasks=1)
    for tasks in (3, 8):
        split = oracle.matvec(8, rows, columns, b, x, tasks=tasks)
        assert np.array_equal(bits(serial), bits(split))


def test_routing_ties_and_renormalization():
    idx, w = oracle.route(np.array([0.5, 2, -1, 2, 1.5, 2]), 3)
    assert list(idx) == [1, 3, 5]
    assert np.allclose(w, 1 / 3, atol=1e-7)
    idx, w = oracle.route(np.array([0, 1, 2, 3]), 2)
    assert list(idx) == [3, 2]
    assert abs(w[0] - 0.7310585786300049) < 1e-7 and abs(w[1] - 0.2689414213699951) < 1e-7
    idx, w = oracle.route(np.array([1, 1, 1]), 3)
    assert list(idx) == [0, 1, 2] and np.allclose(w, 1 / 3, atol=1e-7)


def test_routing_clamp_and_bad_shapes():
    idx, w = oracle.route(np.array([0, -800, 0]), 1)
    assert idx[0] == 0 and np.isfinite(w[0])
    with pytest.raises(oracle.OracleError):
        oracle.route(np.array([1.0]), 2)
    with pytest.raises(oracle.OracleError):
        oracle.route(np.array([1.0, 2.0]), 0)
    with pytest.raises(oracle.OracleError) as e:
        oracle.route(np.array([1.0, np.nan]), 2)
    assert e.value.code == oracle.NON_FINITE


def test_gathered_ffn_weights_scales_and_sums():
    gate_up = np.array([1, 0, 0, 1, 0, 1, 1, 0], dtype="<f4").view(np.uint8)
    down = np.array([1, 2, 3, 4], dtype="<f4").view(np.uint8)
    gu = (0, 2, 2, 2, gate_up)
    dn = (0, 2, 2, 1, down)
    x = np.array([2, 3], dtype=np.float32)
    got = oracle.ffn(gu, dn, x, np.array([0, 1]), np.array([0.25, 0.75]), down_scale=np.array([1, 0.5]))
    h0 = float(oracle.gelu(np.float32(2))) * 3
    h1 = float(oracle.gelu(np.float32(3))) * 2
    assert np.isclose(got[0], 0.25 * h0 * 1 + 0.75 * 0.5 * h1 * 3, rtol=1e-6)
    assert np.isclose(got[1], 0.25 * h0 * 2 + 0.75 * 0.5 * h1 * 4, rtol=1e-6)
    with pytest.raises(oracle.OracleError) as e:
        oracle.ffn(gu, dn, x, np.array([2]), np.array([1.0]))
    assert e.value.code == oracle.INVALID_EXPERT
    with pytest.raises(oracle.OracleError) as e:
        oracle.ffn(gu, dn, x, np.array([0]), np.array([np.inf]))
    assert e.value.code == oracle.NON_FINITE
    with pytest.raises(oracle.OracleError) as e:
        oracle.ffn(gu, dn, x, np.array([0]), np.array([1.0]), down_scale=np.array([1.0]))
    assert e.value.code == oracle.INVALID_SHAPE


def test_activations_match_their_formulas():
    import math
    for v in (-3.0, -0.5, 0.0, 0.7, 2.0, 11.0):
        f = float(np.float32(v))
        inner = 0.7978845608028654 * f * (1.0 + 0.044715 * f * f)
        assert oracle.gelu(np.float32(v)) == np.float32(0.5 * f * (1.0 + math.tanh(inner)))
        assert oracle.silu(np.float32(v)) == np.float32(f / (1.0 + math.exp(-f)))
    assert np.signbit(oracle.silu(np.float32(-np.inf))) and oracle.silu(np.float32(-np.inf)) == 0
