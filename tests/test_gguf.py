"""The GGUF reader (dwim_b200/gguf.py) against the reference's own round-trip
test (inference/gguf.rs:331-375) and against gguf-py's writer, the published
implementation of the container; then a k-quant matrix from file to device."""
import numpy as np
import pytest

from conftest import max_rel_err


def test_reads_back_what_it_wrote(tmp_path):
    """reads_back_what_it_wrote, inference/gguf.rs:331-375: the same file, the same checks."""
    from dwim_b200 import gguf
    path = tmp_path / "test.gguf"
    meta = {"general.architecture": (8, "qwen35"), "qwen35.block_count": (4, 2), "list": (9, (5, [-1, 1])), "scale": (6, 0.5)}
    f32s = np.array([1.0, 2.0, 3.0], "<f4").tobytes()
    bf16 = (np.arange(8, dtype="<u2") << 8).tobytes()
    gguf.write(path, meta, [("norm", [3], gguf.F32, f32s), ("w", [4, 2], gguf.BF16, bf16)])
    g = gguf.Gguf(path)
    assert g.meta["general.architecture"] == "qwen35" and g.meta["qwen35.block_count"] == 2
    assert g.meta["scale"] == 0.5 and g.meta["list"][0] == -1
    assert "missing" not in g.meta
    assert g.f32s("norm").tolist() == [1.0, 2.0, 3.0]
    w = g.matrix("w")
    assert w.shape == (2, 4) and w.data.view(np.uint16)[3] == 3 << 8
    with pytest.raises(ValueError):
        g.matrix("norm")                       # not a matrix
    with pytest.raises(KeyError):
        g.info("nothing")
    assert g.info("w").shape() == (2, 4) and g.info("w").size() == 16


def test_reads_what_gguf_py_writes(tmp_path, oracle):
    """A file written by the published implementation: k-quant tensors come out as
    the bytes that went in, with the shape the engine's convention gives them."""
    gg = pytest.importorskip("gguf")
    from dwim_b200 import gguf
    rng = np.random.default_rng(5)
    rows, cols = 24, 512
    w = (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)
    blocks = {"q4_k": oracle.quantize("q4_k", w), "q6_k": oracle.quantize("q6_k", w), "q8_0": oracle.quantize("q8_0", w)}
    types = {"q4_k": gg.GGMLQuantizationType.Q4_K, "q6_k": gg.GGMLQuantizationType.Q6_K, "q8_0": gg.GGMLQuantizationType.Q8_0}
    path = tmp_path / "k.gguf"
    writer = gg.GGUFWriter(str(path), "qwen35")
    writer.add_uint32("qwen35.block_count", 2)
    for name, b in blocks.items():
        writer.add_tensor(f"blk.0.{name}.weight", b.reshape(rows, -1), raw_dtype=types[name])
    writer.add_tensor("norm", np.arange(cols, dtype=np.float32))
    writer.write_header_to_file()
    writer.write_kv_data_to_file()
    writer.write_tensors_to_file()
    writer.close()
    g = gguf.Gguf(path)
    assert g.meta["general.architecture"] == "qwen35" and g.meta["qwen35.block_count"] == 2
    for name, b in blocks.items():
        t = g.matrix(f"blk.0.{name}.weight")
        assert t.shape == (rows, cols) and np.array_equal(t.data, b)
        assert g.info(f"blk.0.{name}.weight").dtype == {"q4_k": 12, "q6_k": 14, "q8_0": 8}[name]
    assert np.array_equal(g.f32s("norm"), np.arange(cols, dtype=np.float32))


def test_f32_matrices_are_rounded_to_bf16(tmp_path, oracle):
    from dwim_b200 import gguf
    x = np.array([[1.0, 1.00390625, 3.14159, -2.5e-3], [65504.0, 1e-20, -0.0, 7.0]], "<f4")
    path = tmp_path / "f.gguf"
    gguf.write(path, {}, [("m", [4, 2], gguf.F32, x.tobytes())])
    t = gguf.Gguf(path).matrix("m")
    assert t.fmt == gguf.BF16 and np.array_equal(t.data.view(np.uint16), oracle.to_bf16(x))


@pytest.mark.gpu
def test_k_quant_matrix_from_file_to_device(tmp_path, dev, oracle):
    """File -> Gguf.matrix -> upload -> matmul for Q4_K, and the 128-wide column
    groups of a linear-attention output projection (inference/qwen35/mod.rs:845-847),
    which are not whole Q4_K blocks: regrouped through the device as Q8_0."""
    from dwim_b200 import gguf
    rng = np.random.default_rng(6)
    rows, cols = 320, 1024
    w = (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)
    blocks = oracle.quantize("q4_k", w)
    path = tmp_path / "m.gguf"
    gguf.write(path, {"general.alignment": (4, 64)}, [("blk.3.ssm_out.weight", [cols, rows], 12, blocks.tobytes())])
    t = gguf.Gguf(path).matrix("blk.3.ssm_out.weight")
    x = rng.standard_normal((3, cols)).astype(np.float32)
    out = dev.alloc(3 * rows)
    dev.matmul(out, dev.upload(t), dev.buffer(x))
    assert max_rel_err(dev.read(out), oracle.matmul("q4_k", blocks, rows, cols, x)) <= 1e-4
    order = [5, 0, 7, 2, 1, 6, 3, 4]                       # 128-wide groups, shuffled
    regrouped = gguf.column_groups(dev, t, 128, order)
    assert regrouped.fmt == 8 and regrouped.shape == (rows, cols)
    decoded = oracle.dequantize("q4_k", blocks, rows, cols).reshape(rows, 8, 128)[:, order, :].reshape(rows, cols)
    assert np.array_equal(regrouped.data, oracle.quantize("q8_0", decoded))
    whole = gguf.column_groups(dev, t, 256, [3, 1, 0, 2])  # whole blocks: byte moves
    assert whole.fmt == 12 and np.array_equal(whole.data, t.select_column_groups(256, [3, 1, 0, 2]).data)
