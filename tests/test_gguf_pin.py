"""Pins the oracle's block decoders to a published implementation of the GGUF
formats: ``gguf.quants.dequantize`` of the gguf-py package (the Python package
llama.cpp ships; 0.19.0 in this image).

The reference engine has no Q4_K code at all (inference/gguf.rs:28-33 knows
type ids 0, 2, 3, 8, 14, 30 only), so for Q4_K the layout and evaluation order
of ``oracle.dequantize`` would otherwise rest on this repository's own
definition.  Here every decoder must agree bit for bit with gguf-py, on blocks
the oracle's quantizers emit and on random bit patterns with finite scales.
Q6_K and Q8_0 are pinned a second time this way (their first pin is the
reference's own known-answer tests).  Skipped where gguf-py is not installed.
"""
import numpy as np
import pytest

gguf = pytest.importorskip("gguf")
from gguf import GGMLQuantizationType as T   # noqa: E402
from gguf.quants import dequantize as gguf_dequantize   # noqa: E402

TYPES = {"q4_k": (T.Q4_K, 144, 256, (1, 3)), "q6_k": (T.Q6_K, 210, 256, (209,)), "q8_0": (T.Q8_0, 34, 32, (1,))}


def published(fmt, blocks, rows, cols):
    qtype, size, per, _ = TYPES[fmt]
    return gguf_dequantize(np.ascontiguousarray(blocks).reshape(rows, cols // per * size), qtype).astype(np.float32)


def same_bits(a, b):
    a, b = np.ascontiguousarray(a, np.float32), np.ascontiguousarray(b, np.float32)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("fmt", sorted(TYPES))
def test_decoder_equals_gguf_py_on_quantizer_output(oracle, fmt):
    rng = np.random.default_rng(101)
    rows, cols = 48, 2048
    w = (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)
    w[0, :256] = 0.0
    w[1, 7] = 5.0
    w[2] *= 1e-4
    blocks = oracle.quantize(fmt, w)
    assert same_bits(oracle.dequantize(fmt, blocks, rows, cols), published(fmt, blocks, rows, cols))


@pytest.mark.parametrize("fmt", sorted(TYPES))
def test_decoder_equals_gguf_py_on_random_bit_patterns(oracle, fmt):
    """Every field at arbitrary values: all 6-bit scale/minimum packings, every
    nibble and 2-bit plane, negative sub-scales, either sign of d and dmin."""
    rng = np.random.default_rng(102)
    _, size, per, scale_bytes = TYPES[fmt]
    rows, cols = 64, 1024
    blocks = rng.integers(0, 256, rows * (cols // per) * size, dtype=np.uint8)
    b = blocks.reshape(-1, size)
    for off in scale_bytes:
        b[:, off] &= 0xBB              # the f16 scales stay finite (exponent below 0x1f), either sign
    assert same_bits(oracle.dequantize(fmt, blocks, rows, cols), published(fmt, blocks, rows, cols))


def test_q4_k_scale_packing_equals_gguf_py(oracle):
    """The 12 bytes of 6-bit scales and minimums, one block per packing case."""
    rng = np.random.default_rng(103)
    for _ in range(200):
        sc, m = rng.integers(0, 64, 8).astype(np.uint8), rng.integers(0, 64, 8).astype(np.uint8)
        block = np.zeros(144, np.uint8)
        block[0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
        block[2:4] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
        block[4:16] = oracle.q4k_pack_scales(sc, m)
        block[16:] = 0x11                      # every quant is 1: weight = sc_j - m_j
        out = published("q4_k", block, 1, 256)[0]
        assert np.array_equal(out.reshape(8, 32)[:, 0], sc.astype(np.float32) - m.astype(np.float32))
