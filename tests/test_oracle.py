"""The CPU oracle against the reference's own known-answer tests and
properties (transcribed in tests/golden/reference_kats.json), and against its
committed outputs (tests/golden/oracle_cases.npz)."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
KATS = json.load(open(os.path.join(HERE, "golden", "reference_kats.json")))


def test_f16_round_trips_what_it_can_represent(oracle):
    # gpu/cpu.rs:510-533
    for x in KATS["f16_round_trip_values"]["values"]:
        bits = oracle.to_f16([x])
        assert oracle.to_f16(oracle.from_f16(bits))[0] == bits[0], x
    bits = np.arange(65536, dtype=np.uint16)
    finite = (bits & 0x7C00) != 0x7C00
    assert np.array_equal(oracle.to_f16(oracle.from_f16(bits[finite])), bits[finite])
    # and the decoder agrees with IEEE half precision everywhere
    assert np.array_equal(oracle.from_f16(bits[finite]), bits[finite].view(np.float16).astype(np.float32))


def test_f16_rounds_to_nearest_and_clamps(oracle):
    # gpu/cpu.rs:560-575
    for case in KATS["f16_rounding"]["cases"]:
        back = oracle.from_f16(oracle.to_f16([case["x"]]))[0]
        assert back == np.float32(case["back"]), case
    x = np.random.default_rng(0).standard_normal(200_000).astype(np.float32) * 3
    assert np.array_equal(oracle.to_f16(x), x.astype(np.float16).view(np.uint16))


def test_bf16_is_the_top_half_rounded_to_even(oracle):
    # gpu/float.rs:5-8, 30-36
    x = np.random.default_rng(1).standard_normal(100_000).astype(np.float32)
    bits = oracle.to_bf16(x)
    back = oracle.bf16(bits)
    assert np.array_equal(back.view(np.uint32) & 0xFFFF, np.zeros_like(bits, dtype=np.uint32))
    assert np.all(np.abs(back - x) <= np.abs(x) * 2.0 ** -8)
    assert oracle.to_bf16([1.0 + 2.0 ** -8])[0] == 0x3F80          # a tie rounds to even
    assert oracle.to_bf16([1.0 + 3 * 2.0 ** -8])[0] == 0x3F82


def test_quantize_rounds_to_the_nearest_multiple_of_the_scale(oracle):
    # gpu/cpu.rs:535-558
    k = KATS["quantize_block"]
    block = np.zeros(32, np.float32)
    block[:8] = k["head"]
    bits, q = oracle.quantize_block(block)
    assert oracle.from_f16([bits])[0] == k["scale"]
    assert list(q[:8]) == k["quants_head"]
    ramp = np.array([(i - 13.3) * 0.37 for i in range(32)], np.float32)
    bits, q = oracle.quantize_block(ramp)
    d = oracle.from_f16([bits])[0]
    assert np.all(np.abs(ramp - q.astype(np.float32) * d) <= d / 2)
    assert np.abs(q.astype(int)).max() == 127
    bits, q = oracle.quantize_block(np.zeros(32, np.float32))
    assert bits == 0 and not q.any()
    bits, q = oracle.quantize_block(np.full(32, -1e8, np.float32))
    assert oracle.from_f16([bits])[0] == 65504.0 and np.all(q == -127)


def test_q4_0_puts_the_largest_weight_at_minus_eight(oracle):
    # gpu/quant.rs:213-230
    x = np.zeros(32, np.float32)
    x[5], x[20], x[31] = -0.5, 0.25, 0.125
    scales, quants = oracle.quantize_q4_0_row_split(x)
    assert oracle.from_f16(scales)[0] == 0.0625
    assert quants[5] & 0xF == 0 and quants[4] >> 4 == 12 and quants[15] >> 4 == 10 and quants[0] == 0x88
    assert np.array_equal(oracle.dequantize_q4_0_row_split(scales, quants), x)


def test_q4_1_adds_the_minimum(oracle):
    # inference/quants.rs:220-233
    block = bytearray()
    block += oracle.to_f16([0.5]).tobytes() + oracle.to_f16([-2.0]).tobytes()
    block += bytes(j | (15 - j) << 4 for j in range(16))
    out = oracle.dequantize_q4_1(np.frombuffer(bytes(block), np.uint8), 32)
    for j in range(16):
        assert out[j] == j * 0.5 - 2.0 and out[j + 16] == (15 - j) * 0.5 - 2.0


def test_q6_k_places_bits_and_scales_as_llama_cpp_does(oracle):
    # inference/quants.rs:236-275
    for key in ("first", "second"):
        k = KATS["q6_k_blocks"][key]
        block = np.zeros(210, np.uint8)
        for i, v in k["set_bytes"].items():
            block[int(i)] = v
        block[208:210] = np.frombuffer(oracle.to_f16([k["d"]]).tobytes(), np.uint8)
        out = oracle.dequantize("q6_k", block, 1, 256)[0]
        exp = k["expect"]
        single = next(int(i) for i in exp if i.isdigit())
        lo, hi = next(map(int, key_.split("_")[1:3]) for key_ in exp if key_.startswith("range"))
        lo, hi = int(lo), int(hi)
        in_range = next(v for key_, v in exp.items() if key_.startswith("range"))
        for i, v in enumerate(out):
            want = exp[str(single)] if i == single else in_range if lo <= i < hi else exp["elsewhere"]
            assert v == np.float32(want), (key, i, v, want)


def test_q8_0_round_trips_within_a_step(oracle):
    # gpu/quant.rs:198-211
    x = oracle.Lcg(1).floats(256)
    scales, quants = oracle.quantize_q8_0_row_split(x)
    back = oracle.dequantize_q8_0_row_split(scales, quants)
    for b in range(8):
        blk, bk = x[32 * b:32 * b + 32], back[32 * b:32 * b + 32]
        step = np.abs(blk).max() / 127.0
        assert np.all(np.abs(blk - bk) <= step * 0.51)


def test_dots_match_dequantized(oracle):
    # gpu/quant.rs:232-257
    for cols in KATS["dots_match_dequantized"]["cols"]:
        w, x = oracle.Lcg(2).floats(cols), oracle.Lcg(3).floats(cols)
        scales, quants = oracle.quantize_q8_0_row_split(w)
        back = oracle.dequantize_q8_0_row_split(scales, quants)
        want = np.float32(0)
        for a, b in zip(back, x):   # the test's own sequential f32 sum
            want = np.float32(want + a * b)
        assert abs(oracle.dot_q8_0_split(scales, quants, x) - want) < 1e-4 * cols
        scales, quants = oracle.quantize_q4_0_row_split(w)
        back = oracle.dequantize_q4_0_row_split(scales, quants)
        want = np.float32(0)
        for a, b in zip(back, x):
            want = np.float32(want + a * b)
        assert abs(oracle.dot_q4_0_split(scales, quants, x) - want) < 1e-4 * cols


def test_packed_blocks_read_back_the_same_in_either_layout(oracle):
    # inference/quants.rs:206-218 (the Q8_0 half; the device takes Q8_0 in file layout)
    x = oracle.Lcg(1).floats(256)
    scales, quants = oracle.quantize_q8_0_row_split(x)
    packed = oracle.q8_0_split_to_file(scales, quants)
    from_file = oracle.dequantize("q8_0", packed, 2, 128).ravel()
    assert np.array_equal(from_file, oracle.dequantize_q8_0_row_split(scales, quants))
    assert np.all(np.abs(x - from_file) < 0.005)
    s2, q2 = oracle.q8_0_file_to_split(packed)
    assert np.array_equal(s2, scales) and np.array_equal(q2, quants)
    # the whole-row quantizer writes the same bytes
    assert np.array_equal(oracle.quantize("q8_0", x.reshape(2, 128)), packed)
    # and the GGUF-layout dot is the split-layout dot
    xx = oracle.Lcg(9).floats(256)
    assert oracle.dot("q8_0", packed, xx) == oracle.dot_q8_0_split(scales, quants, xx)


def test_requantizing_keeps_weights_within_a_step(oracle):
    # inference/quants.rs:277-284
    x = oracle.Lcg(2).floats(128)
    back = oracle.dequantize("q8_0", oracle.quantize("q8_0", x.reshape(2, 64)), 2, 64).ravel()
    assert np.all(np.abs(x - back) < 1.0 / 127.0)


# ---- the formats the reference does not have: self-consistency -----------------
def test_q4_k_scale_packing_round_trips_every_pattern(oracle):
    rng = np.random.default_rng(3)
    for _ in range(2000):
        sc, m = rng.integers(0, 64, 8, dtype=np.uint8), rng.integers(0, 64, 8, dtype=np.uint8)
        s2, m2 = oracle.q4k_unpack_scales(oracle.q4k_pack_scales(sc, m))
        assert np.array_equal(sc, s2) and np.array_equal(m, m2)
    for _ in range(2000):   # and every 12-byte pattern unpacks to 6-bit values that pack back
        b = rng.integers(0, 256, 12, dtype=np.uint8)
        sc, m = oracle.q4k_unpack_scales(b)
        assert sc.max() < 64 and m.max() < 64
        assert np.array_equal(oracle.q4k_pack_scales(sc, m), b)


def test_q4_k_block_layout_by_hand(oracle):
    # d = 0.5, dmin = 0.25; sub-block 5 has scale 33 (needs the high bits),
    # minimum 47; weight 5*32 + 7 has quant 9: (0.5*33)*9 - 0.25*47
    sc, m = np.zeros(8, np.uint8), np.zeros(8, np.uint8)
    sc[5], m[5] = 33, 47
    block = np.zeros(144, np.uint8)
    block[0:2] = np.frombuffer(oracle.to_f16([0.5]).tobytes(), np.uint8)
    block[2:4] = np.frombuffer(oracle.to_f16([0.25]).tobytes(), np.uint8)
    block[4:16] = oracle.q4k_pack_scales(sc, m)
    block[16 + 2 * 32 + 7] = 9 << 4          # group 2, byte 7, high nibble = sub-block 5
    out = oracle.dequantize("q4_k", block, 1, 256)[0]
    for i, v in enumerate(out):
        want = 16.5 * 9 - 11.75 if i == 167 else -11.75 if 160 <= i < 192 else 0.0
        assert v == np.float32(want), (i, v, want)


@pytest.mark.parametrize("fmt,steps", [("q4_k", 15), ("q6_k", 63), ("q8_0", 254)])
def test_quantizers_keep_weights_within_a_step(oracle, fmt, steps):
    rng = np.random.default_rng(7)
    w = (0.02 * rng.standard_normal((8, 1024))).astype(np.float32)
    w[0, :256] = 0.0                       # an all-zero block
    w[1, 5] = 3.0                          # an outlier
    blocks = oracle.quantize(fmt, w)
    back = oracle.dequantize(fmt, blocks, 8, 1024)
    assert np.all(back[0, :256] == 0.0)
    # Error bound per scale unit (256 weights; 32 for Q8_0): half a step of the
    # unit's widest group, plus the coarseness of the 6-/8-bit group scales and
    # minimums, which are multiples of that widest step over 63 (or 127).
    unit = 32 if fmt == "q8_0" else 256
    wu, bu = w.reshape(-1, unit), back.reshape(-1, unit)
    group = {"q4_k": 32, "q6_k": 16, "q8_0": 32}[fmt]
    wg = w.reshape(-1, unit // group, group)
    span = (wg.max(2) - np.minimum(wg.min(2), 0)) if fmt == "q4_k" else 2 * np.abs(wg).max(2)
    span = span.max(1)
    assert np.all(np.abs(wu - bu).max(1) <= span * (0.55 / steps + 0.02) + 1e-7)


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k", "q8_0"])
def test_dot_is_the_dequantized_dot(oracle, fmt):
    rng = np.random.default_rng(11)
    for cols in (256, 1024, 5120):
        w = (0.02 * rng.standard_normal((1, cols))).astype(np.float32)
        x = rng.standard_normal(cols).astype(np.float32)
        blocks = oracle.quantize(fmt, w)
        back = oracle.dequantize(fmt, blocks, 1, cols)[0].astype(np.float64)
        want = float(back @ x.astype(np.float64))
        scale = float(np.sqrt((back * back).sum() * (x.astype(np.float64) ** 2).mean()))
        assert abs(oracle.dot(fmt, blocks, x) - want) < 2e-6 * scale + 1e-6


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k", "q8_0"])
def test_matmul_is_token_major_and_thread_count_does_not_matter(oracle, fmt):
    rng = np.random.default_rng(13)
    rows, cols, n = 37, 512, 3
    blocks = oracle.quantize(fmt, (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    x = rng.standard_normal((n, cols)).astype(np.float32)
    out = oracle.matmul(fmt, blocks, rows, cols, x)
    rb = oracle.row_bytes(fmt, cols)
    for t in range(n):
        for r in (0, 5, rows - 1):
            assert out[t, r] == np.float32(oracle.dot(fmt, blocks[r * rb:(r + 1) * rb], x[t]))
    saved = oracle.threads()
    oracle.set_threads(1)
    assert np.array_equal(out, oracle.matmul(fmt, blocks, rows, cols, x))
    oracle.set_threads(saved)
    # the fused operators are their definitions (gpu/mod.rs:256-285)
    base = rng.standard_normal((n, rows)).astype(np.float32)
    assert np.array_equal(oracle.matmul_add(fmt, blocks, rows, cols, x, base), base + out)
    up = oracle.quantize(fmt, (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    g, u = out, oracle.matmul(fmt, up, rows, cols, x)
    want = g * (np.float32(1) / (np.float32(1) + np.exp(-g))) * u
    assert np.allclose(oracle.swiglu(fmt, blocks, up, rows, cols, x), want, rtol=1e-6, atol=1e-9)


def test_oracle_reproduces_its_committed_outputs(oracle):
    g = np.load(os.path.join(HERE, "golden", "oracle_cases.npz"))
    for fmt in ("q4_k", "q6_k", "q8_0"):
        w, x, blocks = g[f"{fmt}_w"], g[f"{fmt}_x"], g[f"{fmt}_blocks"]
        rows, cols = w.shape
        assert np.array_equal(oracle.quantize(fmt, w), blocks)
        assert np.array_equal(oracle.dequantize(fmt, blocks, rows, cols).view(np.uint32), g[f"{fmt}_dequant"].view(np.uint32))
        assert np.array_equal(oracle.matmul(fmt, blocks, rows, cols, x), g[f"{fmt}_matmul"])
        assert np.array_equal(oracle.swiglu(fmt, blocks, g[f"{fmt}_up_blocks"], rows, cols, x), g[f"{fmt}_swiglu"])


# ---- the operators either side of the product ------------------------------------------
def test_rmsnorm_restates_the_cpu_device(oracle):
    """gpu/cpu.rs:157-166 in numpy, step by step in f32, against the C restatement."""
    rng = oracle.Lcg(5)
    for dim, rows in [(128, 5), (1024, 3), (8, 1)]:      # gpu/tests.rs:611-622
        w, x = rng.floats(dim), rng.floats(dim * rows).reshape(rows, dim)
        want = x.copy()
        for r in range(rows):
            s = np.float32(0.0)
            for v in x[r]:
                s = np.float32(s + np.float32(v * v))
            scale = np.float32(1.0) / np.sqrt(np.float32(s / np.float32(dim)) + np.float32(1e-6), dtype=np.float32)
            want[r] = x[r] * (scale * w)
        assert np.array_equal(oracle.rmsnorm(x, w, 1e-6), want)


def test_bf16_dot_and_argmax(oracle):
    rng = oracle.Lcg(4)
    cols = 27                                            # three chunks of eight and a rest of three (gpu/cpu.rs:370-384)
    wbits = (rng.floats(cols).view(np.uint32) >> 16).astype(np.uint16)
    x = rng.floats(cols)
    w = oracle.bf16(wbits)
    acc = np.zeros(8, np.float32)
    for k in range(0, 24, 8):
        acc += w[k:k + 8] * x[k:k + 8]
    rest = np.float32(0.0)
    for k in range(24, cols):
        rest = np.float32(rest + np.float32(w[k] * x[k]))
    total = np.float32(0.0)
    for a in acc:
        total = np.float32(total + a)
    assert oracle.matmul_bf16(wbits, 1, cols, x)[0, 0] == np.float32(total + rest)
    assert oracle.argmax([1.0, 5.0, 5.0, 2.0]) == 1      # the first of equals (inference/qwen35/mod.rs:702-710)
    assert oracle.argmax([np.nan, 1.0]) == 0             # nothing compares greater than a NaN at index 0
    assert oracle.argmax([-np.inf, -np.inf]) == 0
