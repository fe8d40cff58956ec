"""The host-side mirror of the load-time re-layout (`nuclis_b200.planar`): a permutation of the GGUF bytes with an exact
inverse, for every encoding that has a planar form, and untouched bytes for those that have none. The device's
`prepare` is checked against it byte for byte in tests/test_gpu_matvec.py."""
import numpy as np
import pytest

from nuclis_b200 import encoding as enc, planar, synth

PLANAR = {enc.Q6_K: 1, enc.Q8_0: 2, enc.Q5_0: 3, enc.Q5_1: 4, enc.Q4_0: 5, enc.IQ4_NL: 5, enc.IQ4_XS: 6, enc.Q2_K: 7, enc.Q3_K: 8}


@pytest.mark.parametrize("encoding", sorted(PLANAR))
@pytest.mark.parametrize("shape", [(16, 256), (48, 1280)])
def test_relay_is_a_permutation_with_an_exact_inverse(encoding, shape):
    rows, columns = shape
    data = synth.matrix(encoding, rows, columns, seed=7 + encoding)
    out, layout = planar.relay(encoding, data, rows, columns)
    assert layout == PLANAR[encoding] == planar.layout_of(encoding, rows, columns)
    assert out.size == data.size and out.dtype == np.uint8
    assert np.array_equal(np.sort(out), np.sort(data))            # every byte is somewhere, none is changed
    assert not np.array_equal(out, data)
    assert np.array_equal(planar.restore(encoding, out, rows, columns, layout), data)


def test_positions_follow_the_documented_planes():
    # Q8_0: the codes of row r, block k sit at [r][k][32]; the f16 scale of that block at [k][r] behind all codes
    rows, columns = 16, 256
    data = synth.matrix(enc.Q8_0, rows, columns, seed=3)
    out, _ = planar.relay(enc.Q8_0, data, rows, columns)
    blocks = data.reshape(rows, columns // 32, 34)
    r, k = 5, 3
    assert np.array_equal(out[(r * 8 + k) * 32:(r * 8 + k + 1) * 32], blocks[r, k, 2:])
    assert np.array_equal(out[rows * columns + (k * rows + r) * 2:][:2], blocks[r, k, :2])
    # Q3_K: the 12 scale bytes of row r, superblock s sit in the tile of 16 rows r belongs to, the d of the 16 rows behind them
    rows, columns = 32, 512
    data = synth.matrix(enc.Q3_K, rows, columns, seed=4)
    out, _ = planar.relay(enc.Q3_K, data, rows, columns)
    blocks = data.reshape(rows, 2, 110)
    r, s = 21, 1
    tile = rows * 2 * 96 + (s * (rows // 16) + r // 16) * 224
    assert np.array_equal(out[(r * 2 + s) * 96:(r * 2 + s + 1) * 96], blocks[r, s, :96])
    assert np.array_equal(out[tile + (r % 16) * 12:][:12], blocks[r, s, 96:108])
    assert np.array_equal(out[tile + 192 + (r % 16) * 2:][:2], blocks[r, s, 108:110])


@pytest.mark.parametrize("encoding,rows,columns", [(enc.Q4_K, 32, 512), (enc.Q5_K, 32, 512), (enc.Q6_K, 20, 512), (enc.Q8_0, 32, 288)])
def test_matrices_without_a_planar_form_keep_their_bytes(encoding, rows, columns):
    data = synth.matrix(encoding, rows, columns, seed=1)
    out, layout = planar.relay(encoding, data, rows, columns)
    assert layout == 0 and np.array_equal(out, data)
    assert np.array_equal(planar.restore(encoding, out, rows, columns, 0), data)


def test_relay_refuses_bytes_of_another_shape():
    data = synth.matrix(enc.Q6_K, 16, 256, seed=1)
    with pytest.raises(ValueError):
        planar.relay(enc.Q6_K, data[:-2], 16, 256)
    with pytest.raises(ValueError):
        planar.restore(enc.Q6_K, data, 16, 256, 2)
