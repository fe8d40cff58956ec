"""The GGUF tensor directory reader and weights view (nuclis_b200/gguf.py) against the reference's rules
(inference/src/formats/gguf.zig:305-412 and its rejection tests :560-700; inference/src/runtime/weights.zig:8-31).
The CPU part needs no device; the GPU part loads a written file through the view and runs it."""
import struct

import numpy as np
import pytest

import oracle
from nuclis_b200 import encoding as enc, gguf, synth


def small_model(tmp_path, alignment=32):
    rng = np.random.default_rng(3)
    tensors = [
        ("blk.0.attn_q.weight", (512, 64), enc.Q4_K, synth.matrix(enc.Q4_K, 64, 512, 1)),
        ("blk.0.ffn_down.weight", (256, 48), enc.Q6_K, synth.matrix(enc.Q6_K, 48, 256, 2)),
        ("output.weight", (256, 80), enc.Q8_0, synth.matrix(enc.Q8_0, 80, 256, 3)),
        ("blk.0.ffn_gate_up_exps.weight", (256, 32, 4), enc.Q4_K, synth.matrix(enc.Q4_K, 4 * 32, 256, 4)),
        ("output_norm.weight", (256,), enc.F32, rng.standard_normal(256).astype(np.float32).view(np.uint8)),
    ]
    path = str(tmp_path / "small.gguf")
    gguf.write(path, tensors, {"general.architecture": "qwen35", "qwen35.block_count": 1, "general.alignment": alignment})
    return path, tensors


def test_directory_round_trip(tmp_path):
    path, tensors = small_model(tmp_path)
    with gguf.View(path) as view:
        doc = view.document
        assert doc.version == 3 and doc.alignment == 32 and doc.data_offset % 32 == 0
        assert doc.metadata["general.architecture"] == "qwen35" and doc.metadata["qwen35.block_count"] == 1
        assert [t.name for t in doc.tensors] == [t[0] for t in tensors]
        for t, (name, dims, encoding_id, data) in zip(doc.tensors, tensors):
            assert t.dimensions == dims and t.encoding_id == encoding_id and t.bytes == data.size and t.offset % 32 == 0
            assert np.array_equal(view.bytes(t), data)
        m, data = view.matrix(doc.tensor("blk.0.attn_q.weight"))
        assert (m.rows, m.columns, m.encoding, m.bytes) == (64, 512, enc.Q4_K, 64 * 2 * 144)   # dimension 0 is K, dimension 1 is N
        e, _ = view.expert_matrix(doc.tensor("blk.0.ffn_gate_up_exps.weight"))
        assert (e.experts, e.rows, e.columns) == (4, 32, 256)
        with pytest.raises(gguf.GgufError):
            view.matrix(doc.tensor("output_norm.weight"))
        # a row decoded from the mapped bytes is the oracle's decode of the generator's bytes
        stride = m.bytes // m.rows
        assert np.array_equal(oracle.row(enc.Q4_K, data[5 * stride:6 * stride], 512), oracle.row(enc.Q4_K, tensors[0][3][5 * stride:6 * stride], 512))


def test_other_alignments(tmp_path):
    path, _ = small_model(tmp_path, alignment=64)
    with gguf.View(path) as view:
        assert view.document.alignment == 64 and all(t.offset % 64 == 0 for t in view.document.tensors)


def header(tensor_count=0, metadata=b"", metadata_count=0, magic=gguf.MAGIC, version=3):
    return struct.pack("<IIQQ", magic, version, tensor_count, metadata_count) + metadata


def s(text):
    raw = text.encode()
    return struct.pack("<Q", len(raw)) + raw


def tensor_entry(name, dims, encoding_id, offset):
    return s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", encoding_id, offset)


@pytest.mark.parametrize("image,error", [
    (header(magic=0x46554746), "InvalidMagic"),
    (header(version=2), "UnsupportedVersion"),
    (header(metadata=s("general.alignment") + struct.pack("<II", gguf.UINT32, 0), metadata_count=1), "InvalidAlignment"),
    (header(metadata=s("general.alignment") + struct.pack("<II", gguf.UINT32, 3), metadata_count=1), "InvalidAlignment"),
    (header(metadata=s("general.alignment") + struct.pack("<IQ", gguf.UINT64, 32), metadata_count=1), "InvalidAlignment"),
    (header(metadata=(s("a") + struct.pack("<II", gguf.UINT32, 1)) * 2, metadata_count=2), "DuplicateMetadata"),
    (header(metadata=s("a") + struct.pack("<I", 99), metadata_count=1), "InvalidMetadataType"),
    (header(metadata=s("a") + struct.pack("<IB", gguf.BOOL, 2), metadata_count=1), "InvalidBoolean"),
    (header(1) + tensor_entry("t", (), enc.F32, 0), "InvalidShape"),                      # rank 0
    (header(1) + tensor_entry("t", (4, 0), enc.F32, 0), "InvalidShape"),                  # a zero dimension
    (header(1) + tensor_entry("t", (704, 8), enc.Q6_K, 0), "InvalidShape"),               # 704 columns are no whole Q6_K superblocks
    (header(1) + tensor_entry("t", (256, 8), 99, 0), "UnsupportedTensorType"),
    (header(1) + tensor_entry("t", (256, 8), enc.Q4_K, 16), "InvalidAlignment"),          # offset off the 32-byte grid
    (header(1) + tensor_entry("t", (256, 8), enc.Q4_K, 0) + b"\0" * 32, "TensorOutOfBounds"),  # fewer bytes behind the directory than the tensor needs
    (header(2) + tensor_entry("t", (4,), enc.F32, 0) + tensor_entry("t", (4,), enc.F32, 32), "DuplicateTensor"),
    (header(1)[:20], "EndOfStream"),
])
def test_rejections_carry_the_reference_error_names(image, error):
    with pytest.raises(gguf.GgufError) as e:
        gguf.parse(image)
    assert e.value.name == error


def test_overlapping_tensors_are_rejected():
    directory = header(2) + tensor_entry("a", (16,), enc.F32, 0) + tensor_entry("b", (16,), enc.F32, 32)
    directory += b"\0" * ((32 - len(directory) % 32) % 32)
    with pytest.raises(gguf.GgufError) as e:
        gguf.parse(directory + b"\0" * 128)     # a: 64 bytes from 0, b starts at 32
    assert e.value.name == "OverlappingTensors"


@pytest.mark.gpu
def test_a_written_file_drives_the_kernels(tmp_path):
    """Tensors of a GGUF file, through the view, onto the device, through the operators, against the oracle."""
    from nuclis_b200 import Backend
    from parity import assert_matvec_close
    rows, columns = 1024, 2048
    tensors = [("blk.0.ffn_gate.weight", (columns, rows), enc.Q4_K, synth.matrix(enc.Q4_K, rows, columns, 11)),
               ("blk.0.ffn_down.weight", (columns, rows), enc.Q6_K, synth.matrix(enc.Q6_K, rows, columns, 12)),
               ("output.weight", (columns, rows), enc.Q8_0, synth.matrix(enc.Q8_0, rows, columns, 13))]
    path = str(tmp_path / "model.gguf")
    gguf.write(path, tensors)
    x = synth.activations(1, columns, 14)[0]
    with gguf.View(path) as view, Backend(0) as b:
        xb = b.create(columns * 4)
        xb.write(x)
        for t in view.document.tensors:
            wb, m = view.upload(b, t)
            assert m.layout == (0 if t.encoding_id == enc.Q4_K else 1 if t.encoding_id == enc.Q6_K else 2)
            yb = b.create(rows * 4)
            b.begin()
            b.matvec(wb, m, xb, yb)
            b.commit()
            _, data = view.matrix(t)
            want = oracle.matvec(t.encoding_id, rows, columns, data, x)
            mag = oracle.matvec_abs(t.encoding_id, rows, columns, data, x)
            assert_matvec_close(yb.floats(), want, mag, t.name)
            # re-laid on the host instead: the same bytes on the device, the same result
            hb, hm = view.upload(b, t, prepare="host")
            assert hm.layout == m.layout and np.array_equal(hb.read(), wb.read())
            y2 = b.create(rows * 4)
            b.begin()
            b.matvec(hb, hm, xb, y2)
            b.commit()
            assert np.array_equal(y2.floats().view(np.uint32), yb.floats().view(np.uint32))


@pytest.mark.gpu
def test_output_head_and_greedy_selection():
    """The output head at the vocabulary size of the 27B-shape model (248,320 rows; a shorter K keeps the test small)
    followed by `argmax` on the device: the selected token is the oracle's arg-max of the oracle's logits
    whenever the two best logits are further apart than the kernel's error bound; ties go to the lowest index;
    a logit that is not finite gives 0xffffffff (ops/sampling.zig:73-86)."""
    from nuclis_b200 import Backend, Matrix
    rows, columns = 248320, 512
    w = synth.matrix(enc.Q6_K, rows, columns, 21)
    x = synth.activations(1, columns, 22)[0]
    with Backend(0) as b:
        wb = b.wrap(w)
        pb, m = b.prepare(wb, Matrix(enc.Q6_K, rows, columns, w.size))
        xb, yb, rb = b.create(columns * 4), b.create(rows * 4), b.create(4)
        xb.write(x)
        b.begin()
        b.matvec(pb, m, xb, yb)
        b.argmax(yb, rows, rb)
        b.commit()
        logits = yb.floats()
        picked = int(rb.read(np.uint32, 1)[0])
        want = oracle.matvec(enc.Q6_K, rows, columns, w, x)
        assert np.linalg.norm(logits - want) / np.linalg.norm(want) <= 1e-5
        assert picked == int(np.argmax(logits)) and logits[picked] == logits.max()
        order = np.argsort(want)
        if want[order[-1]] - want[order[-2]] > 1e-5 * abs(want[order[-1]]) + 1e-6:
            assert picked == int(order[-1])
        # ties: the lowest index wins; lengths that are no multiple of anything
        for count, values in ((1, [3.0]), (7, [1, 5, 5, 2, 5, 0, -1]), (1000, None), (100003, None)):
            v = np.asarray(values, dtype=np.float32) if values is not None else np.random.default_rng(count).integers(-50, 50, count).astype(np.float32)
            lb = b.create(v.nbytes)
            lb.write(v)
            b.begin(); b.argmax(lb, count, rb); b.commit()
            assert int(rb.read(np.uint32, 1)[0]) == int(np.argmax(v)), count   # numpy's argmax also takes the first of equals
            v[count // 2] = np.nan
            lb.write(v)
            b.begin(); b.argmax(lb, count, rb); b.commit()
            assert int(rb.read(np.uint32, 1)[0]) == 0xFFFFFFFF
            b.release(lb)
