"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a B200.

Modelled on the reference's generic device suite (gpu/tests.rs): the same
deterministic generator, the same shape lists, the same two error checks —
plus bit-exact checks of the decoders and quantizers, the committed golden
cases, and the stricter "max relative error 1e-3" bar.
"""
import json
import os

import numpy as np
import pytest

from conftest import close, close_batch, max_rel_err

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
KATS = json.load(open(os.path.join(HERE, "golden", "reference_kats.json")))
FORMATS = ("q4_k", "q6_k", "q8_0")

# max |got - want| / max(|want|, rms(want)); the matmul bar
TOL = 1e-3


def kcols(fmt, cols):
    """The reference's shapes with cols made whole blocks of the format."""
    per = 32 if fmt == "q8_0" else 256
    return (cols + per - 1) // per * per


def lcg_weights(oracle, rng, fmt, rows, cols):
    """Rng::q8_0-style (gpu/tests.rs:87-103): a row of LCG floats at a time, quantized."""
    w = rng.floats(rows * cols).reshape(rows, cols)
    return oracle.quantize(fmt, w)


def upload(dev, fmt, rows, cols, blocks):
    from dwim_b200 import Tensor
    return dev.upload(Tensor(fmt, (rows, cols), blocks))


# ---- device plumbing (gpu/tests.rs:166-186, 962-975) --------------------------------
def test_write_and_read_round_trip(dev, oracle):
    data = oracle.Lcg(1).floats(100_003)
    assert np.array_equal(dev.read(dev.buffer(data)), data)


def test_alloc_is_zeroed_and_resize_keeps_capacity(dev):
    from dwim_b200 import DeviceError
    buf = dev.alloc(1000)
    assert not dev.read(buf).any()
    dev.write(buf, np.arange(1000, dtype=np.float32))
    dev.resize(buf, 10)
    assert np.array_equal(dev.read(buf), np.arange(10, dtype=np.float32))
    dev.resize(buf, 1000)
    assert np.array_equal(dev.read(buf)[:10], np.arange(10, dtype=np.float32))
    with pytest.raises(DeviceError):
        dev.resize(buf, 1001)
    assert len(dev.read(dev.alloc(0))) == 0


def test_device_reports_itself(dev):
    assert "B200" in dev.name()
    assert dev.memory() > 1 << 30
    assert dev.batch() == 2048


# ---- decoders: bit-exact -----------------------------------------------------------------
@pytest.mark.parametrize("fmt", FORMATS)
def test_dequantize_is_bit_exact(dev, oracle, fmt):
    rng = np.random.default_rng(21)
    for rows, cols in [(1, 256), (37, 1024), (300, 5120)]:
        w = (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)
        blocks = oracle.quantize(fmt, w)
        got = dev.dequantize(upload(dev, fmt, rows, cols, blocks))
        want = oracle.dequantize(fmt, blocks, rows, cols)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("fmt", FORMATS)
def test_dequantize_random_bit_patterns_is_bit_exact(dev, oracle, fmt):
    """Every field at arbitrary values, not only what a quantizer emits."""
    from dwim_b200 import row_bytes
    rng = np.random.default_rng(22)
    rows, cols = 64, 1024
    blocks = rng.integers(0, 256, rows * row_bytes(fmt, cols), dtype=np.uint8)
    # keep the f16 scales finite (inf/nan scales are not weights)
    size = {"q4_k": 144, "q6_k": 210, "q8_0": 34}[fmt]
    b = blocks.reshape(-1, size)
    for off in {"q4_k": (1, 3), "q6_k": (209,), "q8_0": (1,)}[fmt]:
        b[:, off] &= 0x3B          # exponent below 0x1f
    got = dev.dequantize(upload(dev, fmt, rows, cols, blocks))
    want = oracle.dequantize(fmt, blocks, rows, cols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q6_k_known_answers_on_the_device(dev, oracle):
    # inference/quants.rs:236-275, decoded by the device
    block = np.zeros(210, np.uint8)
    block[37], block[128 + 5], block[192 + 2] = 0b1010, 0b1100, 3
    block[208:210] = np.frombuffer(oracle.to_f16([0.25]).tobytes(), np.uint8)
    out = dev.dequantize(upload(dev, "q6_k", 1, 256, block))[0]
    assert out[37] == 19.5 and all(out[i] == -24.0 for i in range(32, 48) if i != 37)
    assert not out[:32].any() and not out[48:].any()


@pytest.mark.parametrize("fmt", FORMATS)
def test_quantize_is_byte_exact(dev, oracle, fmt):
    rng = np.random.default_rng(23)
    w = (0.02 * rng.standard_normal((96, 2048))).astype(np.float32)
    w[0, :256] = 0.0
    w[1, 7] = 5.0
    w[2, :64] = np.float32(1e-30)
    w[3, 300] = -65536.0
    assert np.array_equal(dev.quantize(fmt, w).data, oracle.quantize(fmt, w))
    lcg = oracle.Lcg(5).floats(64 * 512).reshape(64, 512)
    assert np.array_equal(dev.quantize(fmt, lcg).data, oracle.quantize(fmt, lcg))


# ---- matmul ---------------------------------------------------------------------------
@pytest.mark.parametrize("fmt", FORMATS)
def test_block_matmul_matches_cpu(dev, oracle, fmt):
    """block_matmul_matches_cpu (gpu/tests.rs:219-262): the reference's shapes, its
    generator (weights Rng(80) shape after shape, x = Rng(rows + n)), its checks."""
    rng = oracle.Lcg(80)
    for rows, cols, n in KATS["matmul_shapes"]["shapes"]:
        cols = kcols(fmt, cols)
        blocks = lcg_weights(oracle, rng, fmt, rows, cols)
        x = oracle.Lcg(rows + n).floats(n * cols)
        want = oracle.matmul(fmt, blocks, rows, cols, x)
        out = dev.alloc(n * rows)
        dev.matmul(out, upload(dev, fmt, rows, cols, blocks), dev.buffer(x))
        got = dev.read(out).reshape(n, rows)
        what = f"{fmt} {rows}x{cols} n={n}"
        if n == 1:
            close(got, want, 1e-4)
        close_batch(got, want, what)
        assert max_rel_err(got, want) <= TOL, what


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 6, 7, 8, 9, 15, 16, 17])
def test_matmul_token_counts_at_model_width(dev, oracle, fmt, n):
    rng = np.random.default_rng(31 + n)
    rows, cols = 333, 5120
    blocks = oracle.quantize(fmt, (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    x = rng.standard_normal((n, cols)).astype(np.float32)
    out = dev.alloc(n * rows)
    dev.matmul(out, upload(dev, fmt, rows, cols, blocks), dev.buffer(x))
    got, want = dev.read(out).reshape(n, rows), oracle.matmul(fmt, blocks, rows, cols, x)
    assert max_rel_err(got, want) <= TOL
    # the small-M kernel keeps products exact: expect fp32-summation noise only
    assert max_rel_err(got, want) <= 2e-5


@pytest.mark.parametrize("fmt", FORMATS)
def test_matmul_bf16_activations(dev, oracle, fmt):
    """Config 2's inputs: rows of N(0,1) scaled to RMS 1, rounded to bf16."""
    rng = np.random.default_rng(41)
    rows, cols = 1000, 5120
    blocks = oracle.quantize(fmt, (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    weight = upload(dev, fmt, rows, cols, blocks)
    for n in (1, 7, 16):
        x = rng.standard_normal((n, cols)).astype(np.float32)
        x /= np.sqrt((x * x).mean(1, keepdims=True))
        bits = oracle.to_bf16(x)
        xb = dev.alloc(n * cols)
        dev.write_bf16(xb, bits)
        assert np.array_equal(dev.read(xb), oracle.bf16(bits))
        out = dev.alloc(n * rows)
        dev.matmul(out, weight, xb)
        want = oracle.matmul(fmt, blocks, rows, cols, oracle.bf16(bits))
        assert max_rel_err(dev.read(out).reshape(n, rows), want) <= 2e-5


@pytest.mark.parametrize("fmt", FORMATS)
def test_matmul_golden_cases(dev, fmt):
    """The committed oracle outputs (tests/golden/oracle_cases.npz)."""
    g = np.load(os.path.join(HERE, "golden", "oracle_cases.npz"))
    w, x, blocks = g[f"{fmt}_w"], g[f"{fmt}_x"], g[f"{fmt}_blocks"]
    rows, cols = w.shape
    n = x.shape[0]
    assert np.array_equal(dev.quantize(fmt, w).data, blocks)
    weight = upload(dev, fmt, rows, cols, blocks)
    assert np.array_equal(dev.dequantize(weight).view(np.uint32), g[f"{fmt}_dequant"].view(np.uint32))
    out, scratch = dev.alloc(n * rows), dev.alloc(n * rows)
    dev.matmul(out, weight, dev.buffer(x))
    assert max_rel_err(dev.read(out), g[f"{fmt}_matmul"]) <= 2e-5
    dev.swiglu(out, weight, upload(dev, fmt, rows, cols, g[f"{fmt}_up_blocks"]), dev.buffer(x), scratch)
    assert max_rel_err(dev.read(out), g[f"{fmt}_swiglu"]) <= 1e-4


@pytest.mark.parametrize("bf16", [False, True])
def test_q4_k_gemm_scale_extremes(dev, oracle, bf16):
    """The tensor-core kernel folds a block's minimums into the same accumulator
    as its quants, scaled by dmin/d: rows whose blocks have d = 0, dmin = 0, either
    sign, or dmin up to 2^40 times d must still match the CPU result."""
    rng = np.random.default_rng(47)
    rows, cols, n = 256, 1024, 40
    blocks = oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)).copy()
    regimes = [(1e-3, 2e-3), (0.0, 0.05), (0.05, 0.0), (0.0, 0.0), (1e-3, 0.1), (1e-4, 6.0), (2.4e-7, 30.0),
               (6e-8, 60000.0), (-1e-3, 2e-3), (1e-3, -2e-3), (3e-5, 1.0), (1.0, 6e-8)]
    v = blocks.reshape(rows, cols // 256, 144)
    for r in range(rows):
        d, dmin = regimes[r % len(regimes)]
        v[r, :, 0:2] = np.frombuffer(np.float16(d).tobytes(), np.uint8)
        v[r, :, 2:4] = np.frombuffer(np.float16(dmin).tobytes(), np.uint8)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    xb = dev.alloc(n * cols)
    if bf16:
        bits = oracle.to_bf16(x)
        dev.write_bf16(xb, bits)
        x = oracle.bf16(bits).reshape(n, cols)
    else:
        dev.write(xb, x)
    out = dev.alloc(n * rows)
    dev.matmul(out, upload(dev, "q4_k", rows, cols, blocks), xb)
    got, want = dev.read(out).reshape(n, rows), oracle.matmul("q4_k", blocks, rows, cols, x).reshape(n, rows)
    for k, (d, dmin) in enumerate(regimes):
        g, w = got[:, k::len(regimes)], want[:, k::len(regimes)]
        if d == 0.0 and dmin == 0.0:
            assert not g.any() and not w.any()
        else:
            assert max_rel_err(g, w) <= 2e-5, f"d={d} dmin={dmin}: {max_rel_err(g, w):.2e}"


def test_shadow_is_rebuilt_after_a_write(dev, oracle):
    """One input buffer reused: across formats (different operand layouts) and
    after being overwritten."""
    rng = np.random.default_rng(43)
    rows, cols = 64, 512
    w = (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)
    xb, out = dev.alloc(2 * cols), dev.alloc(2 * rows)
    for trial in range(2):
        x = rng.standard_normal((2, cols)).astype(np.float32)
        dev.write(xb, x)
        for fmt in FORMATS:
            blocks = oracle.quantize(fmt, w)
            dev.matmul(out, upload(dev, fmt, rows, cols, blocks), xb)
            assert max_rel_err(dev.read(out), oracle.matmul(fmt, blocks, rows, cols, x)) <= 2e-5


# ---- fused operators (gpu/tests.rs:816-871) ---------------------------------------------
@pytest.mark.parametrize("fmt", FORMATS)
def test_swiglu_matches_cpu(dev, oracle, fmt):
    rng = oracle.Lcg(22)
    for rows, cols, n in KATS["fused_shapes"]["shapes"]:
        cols = kcols(fmt, cols)
        gate, up = lcg_weights(oracle, rng, fmt, rows, cols), lcg_weights(oracle, rng, fmt, rows, cols)
        x = rng.floats(n * cols)
        want = oracle.swiglu(fmt, gate, up, rows, cols, x)
        out, scratch = dev.alloc(n * rows), dev.alloc(n * rows)
        dev.swiglu(out, upload(dev, fmt, rows, cols, gate), upload(dev, fmt, rows, cols, up), dev.buffer(x), scratch)
        got = dev.read(out)
        close_batch(got, want, f"{fmt} {rows}x{cols} n={n}")
        assert max_rel_err(got, want) <= TOL


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("n", [1, 2, 3, 5, 8, 9])
def test_swiglu_one_launch_at_model_width(dev, oracle, fmt, n):
    """Up to eight tokens take gate and up in a single launch; nine go the
    two-launch way.  Rows that are not a whole tile, both ways against the CPU."""
    rng = np.random.default_rng(53 + n)
    rows, cols = 1000, 5120
    gate = oracle.quantize(fmt, (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    up = oracle.quantize(fmt, (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    x = rng.standard_normal((n, cols)).astype(np.float32)
    out, scratch = dev.alloc(n * rows), dev.alloc(n * rows)
    dev.swiglu(out, upload(dev, fmt, rows, cols, gate), upload(dev, fmt, rows, cols, up), dev.buffer(x), scratch)
    want = oracle.swiglu(fmt, gate, up, rows, cols, x)
    assert max_rel_err(dev.read(out), want) <= 2e-5


@pytest.mark.parametrize("fmt", FORMATS)
def test_matmul_add_matches_cpu(dev, oracle, fmt):
    rng = oracle.Lcg(23)
    for rows, cols, n in KATS["fused_shapes"]["shapes"]:
        cols = kcols(fmt, cols)
        blocks = lcg_weights(oracle, rng, fmt, rows, cols)
        inp, x = rng.floats(n * cols), rng.floats(n * rows)
        want = oracle.matmul_add(fmt, blocks, rows, cols, inp, x).ravel()
        out, scratch = dev.buffer(x), dev.alloc(n * rows)
        dev.matmul_add(out, upload(dev, fmt, rows, cols, blocks), dev.buffer(inp), scratch)
        got = dev.read(out)
        # what was added, which is what a batch's error is a part of
        close_batch(got - x, want - x, f"{fmt} {rows}x{cols} n={n}")
        assert max_rel_err(got - x, want - x) <= TOL


# ---- misuse is an error code, never a fault (the trait's panics) ------------------------------
def test_misuse_is_reported(dev, oracle):
    from dwim_b200 import DeviceError, Tensor
    rng = np.random.default_rng(47)
    blocks = oracle.quantize("q4_k", (0.02 * rng.standard_normal((32, 512))).astype(np.float32))
    w = upload(dev, "q4_k", 32, 512, blocks)
    with pytest.raises(DeviceError):               # x is not rows of cols
        dev.matmul(dev.alloc(32), w, dev.alloc(500))
    with pytest.raises(DeviceError):               # out has the wrong length
        dev.matmul(dev.alloc(33), w, dev.alloc(512))
    with pytest.raises(DeviceError):               # write of the wrong length
        dev.write(dev.alloc(8), np.zeros(9, np.float32))
    with pytest.raises(DeviceError):               # gate and up differ
        w2 = upload(dev, "q4_k", 16, 512, blocks[: 16 * 288])
        dev.swiglu(dev.alloc(32), w, w2, dev.alloc(512), dev.alloc(32))
    L = dev._L
    import ctypes as C
    h = C.c_void_p()
    assert L.dwim_b200_upload(dev._ctx, 12, 32, 512, blocks.ctypes.data, blocks.size - 1, C.byref(h)) == -1   # truncated
    assert L.dwim_b200_upload(dev._ctx, 2, 32, 512, blocks.ctypes.data, blocks.size, C.byref(h)) == -2        # Q4_0: unknown here
    assert L.dwim_b200_upload(dev._ctx, 12, 32, 500, blocks.ctypes.data, blocks.size, C.byref(h)) == -2       # not whole blocks
    assert b"blocks" in L.dwim_b200_last_error(dev._ctx)
    # the device still works afterwards
    out = dev.alloc(32)
    x = rng.standard_normal(512).astype(np.float32)
    dev.matmul(out, w, dev.buffer(x))
    assert max_rel_err(dev.read(out), oracle.matmul("q4_k", blocks, 32, 512, x)) <= 2e-5
    dev.sync()


def test_empty_inputs(dev, oracle):
    blocks = oracle.quantize("q8_0", np.ones((4, 64), np.float32))
    w = upload(dev, "q8_0", 4, 64, blocks)
    dev.matmul(dev.alloc(0), w, dev.alloc(0))       # no tokens
    w0 = upload(dev, "q8_0", 0, 64, np.zeros(0, np.uint8))
    dev.matmul(dev.alloc(0), w0, dev.alloc(64))     # no rows
    dev.sync()


# ---- BASELINE's full sizes: oracle on a row sample + size-independent properties ------------------
def full_size_case(dev, oracle, fmt, rows, cols, n, seed, bf16=False):
    rng = np.random.default_rng(seed)
    w = (0.02 * rng.standard_normal((rows, cols), dtype=np.float32)).astype(np.float32)
    t = dev.quantize(fmt, w)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    weight = dev.upload(t)
    xb = dev.alloc(n * cols)
    if bf16:
        bits = oracle.to_bf16(x)
        x = oracle.bf16(bits).reshape(n, cols)
        dev.write_bf16(xb, bits)
    else:
        dev.write(xb, x)
    out = dev.alloc(n * rows)
    dev.matmul(out, weight, xb)
    got = dev.read(out).reshape(n, rows)
    # (1) the oracle on every row
    want = oracle.matmul(fmt, t.data, rows, cols, x)
    assert max_rel_err(got, want) <= TOL
    # (2) the device quantizer wrote the oracle's bytes (a row sample) and decodes them bit-exactly
    sample = rng.choice(rows, 64, replace=False)
    assert np.array_equal(t.select_rows(sample).data, oracle.quantize(fmt, w[sample]))
    # (3) linearity: W.(2x) = 2 W.x (a power of two scales every term; only
    # f16-subnormal remainders of tiny activations can round differently)
    dev.write(xb, 2.0 * x)
    out2 = dev.alloc(n * rows)
    dev.matmul(out2, weight, xb)
    assert max_rel_err(dev.read(out2).reshape(n, rows), 2.0 * got) <= 1e-6
    # (4) a second run gives the same bits (fixed summation order)
    dev.write(xb, x)
    dev.matmul(out2, weight, xb)
    assert np.array_equal(dev.read(out2).reshape(n, rows), got)
    return got, want


def test_config1_q4_k_gemv_full_size(dev, oracle):
    """BASELINE config 1: Q4_K [17408, 5120] . x[1, 5120], W seed 0, x seed 1."""
    w = (0.02 * np.random.default_rng(0).standard_normal((17408, 5120), dtype=np.float32))
    x = np.random.default_rng(1).standard_normal((1, 5120)).astype(np.float32)
    t = dev.quantize("q4_k", w)
    assert t.data.size == 50_135_040
    weight = dev.upload(t)
    assert np.array_equal(dev.dequantize(weight).view(np.uint32),
                          oracle.dequantize("q4_k", t.data, 17408, 5120).view(np.uint32))
    out = dev.alloc(17408)
    dev.matmul(out, weight, dev.buffer(x))
    got, want = dev.read(out), oracle.matmul("q4_k", t.data, 17408, 5120, x).ravel()
    close(got, want, 1e-4)
    assert max_rel_err(got, want) <= 2e-5
    # against the unquantized product: within quantization noise (a sanity check on the format itself)
    exact = (w.astype(np.float64) @ x[0].astype(np.float64))
    assert np.sqrt(np.mean((got - exact) ** 2)) < 0.12 * np.sqrt(np.mean(exact ** 2))


@pytest.mark.parametrize("fmt,rows,cols,n", [
    ("q4_k", 12288, 5120, 8), ("q8_0", 5120, 5120, 8), ("q4_k", 5120, 17408, 4), ("q6_k", 151936, 5120, 1)])
def test_config3_shapes_full_size(dev, oracle, fmt, rows, cols, n):
    full_size_case(dev, oracle, fmt, rows, cols, n, seed=3)


def test_config2_q4_k_m16_bf16_full_size(dev, oracle):
    full_size_case(dev, oracle, "q4_k", 17408, 5120, 16, seed=2, bf16=True)


# ---- sharding: the device's re-assembly against the host statement of it ---------------------
def test_gather_rows_matches_the_host_assembly(dev):
    from dwim_b200 import shard
    rng = np.random.default_rng(51)
    for rows, world, align, n in [(17408, 8, 16, 3), (5120, 2, 16, 16), (77, 4, 16, 2), (100, 3, 7, 5)]:
        pr = shard.part_rows(rows, world, align)
        parts = rng.standard_normal((world, n, pr)).astype(np.float32)
        out = dev.alloc(n * rows)
        dev.gather_rows(out, dev.buffer(parts), n, rows, world, align)
        assert np.array_equal(dev.read(out).reshape(n, rows), shard.assemble(parts, n, rows, world, align))


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 40])
def test_feed_forward_block_on_one_gpu(dev, oracle, n):
    """ShardedFFN with a world of one: swiglu, then the down projection of the
    f32 intermediate, against the CPU's two steps."""
    from dwim_b200 import Tensor, shard
    rng = np.random.default_rng(61 + n)
    hidden, inner = 512, 1024
    mk = lambda r, c: Tensor("q4_k", (r, c), oracle.quantize("q4_k", (0.05 * rng.standard_normal((r, c))).astype(np.float32)))
    gate, up, down = mk(inner, hidden), mk(inner, hidden), mk(hidden, inner)
    x = rng.standard_normal((n, hidden)).astype(np.float32)
    block = shard.ShardedFFN(dev, gate, up, down)
    got = dev.read(block.forward(dev.buffer(x))).reshape(n, hidden)
    h = oracle.swiglu("q4_k", gate.data, up.data, inner, hidden, x)
    want = oracle.matmul("q4_k", down.data, hidden, inner, h).reshape(n, hidden)
    assert max_rel_err(got, want) <= 5e-5


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("n", [1, 2, 5, 8])
def test_int8_routine_activation_extremes(dev, oracle, fmt, n):
    """Up to eight tokens go through int8 digit planes with one exponent per 256
    activations: outliers, zeros, a zero unit, tiny and huge magnitudes."""
    rng = np.random.default_rng(71 + n)
    rows, cols = 96, 2048
    blocks = oracle.quantize(fmt, (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    weight = upload(dev, fmt, rows, cols, blocks)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    x[:, 7] = 3.0e4                   # an outlier in the first unit
    x[:, 256:512] = 0.0               # a unit of zeros
    x[:, 512:768] *= 1e-30            # tiny
    x[:, 768:1024] *= 1e20            # huge
    x[:, 1024:1280:2] = 0.0           # every other one zero
    x[:, 1300] = -65504.0
    out = dev.alloc(n * rows)
    dev.matmul(out, weight, dev.buffer(x))
    got, want = dev.read(out).reshape(n, rows), oracle.matmul(fmt, blocks, rows, cols, x)
    assert np.isfinite(got).all()
    # three digit planes (three to eight tokens) round an activation at 2^-23 of its unit's largest
    assert max_rel_err(got, want) <= (2e-5 if n <= 2 else 1e-4)


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("scale", [1e5, 1e20, 1e-30])
def test_gemm_activation_range(dev, oracle, scale, bf16):
    """Forty tokens through the tensor-core kernel with activations far outside
    f16's range: every token's row is scaled by its own power of two on the way in
    and back on the way out, so nothing is clamped or flushed."""
    rng = np.random.default_rng(79)
    rows, cols, n = 256, 1024, 40
    blocks = oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    x = rng.standard_normal((n, cols)).astype(np.float32)
    x[::2] *= np.float32(scale)               # every other token: neighbours keep their own range
    x[1, 7] = 3.0e4
    xb = dev.alloc(n * cols)
    if bf16:
        bits = oracle.to_bf16(x)
        dev.write_bf16(xb, bits)
        x = oracle.bf16(bits).reshape(n, cols)
    else:
        dev.write(xb, x)
    out = dev.alloc(n * rows)
    dev.matmul(out, upload(dev, "q4_k", rows, cols, blocks), xb)
    got, want = dev.read(out).reshape(n, rows), oracle.matmul("q4_k", blocks, rows, cols, x)
    assert np.isfinite(got).all()
    for t in range(n):                         # per token: the tokens' magnitudes differ by up to 10^30
        assert max_rel_err(got[t], want[t]) <= 2e-5, (t, max_rel_err(got[t], want[t]))


# ---- the operators either side of the product (the norm before it, the arg-max after it, bf16 matrices) ----
def test_normalize_matches_cpu(dev, oracle):
    """normalize_matches_cpu (gpu/tests.rs:788-812): the reference's shapes and
    generator; then the model's width, where the same launch also writes the next
    product's operand form: the product of the normalized rows must match too."""
    rng = oracle.Lcg(21)
    for dim, rows in KATS["normalize_shapes"]["shapes"]:
        w, x = rng.floats(dim), rng.floats(dim * (rows + 1))
        rng.floats(dim * rows)                 # the reference draws y for its add check here
        out = dev.alloc(dim * rows)
        dev.normalize(out, dev.buffer(x), dev.buffer(w), dim * rows, 1e-6)
        close(dev.read(out), oracle.rmsnorm(x[: dim * rows], w, 1e-6), 1e-5)
    g = np.random.default_rng(83)
    cols, wrows = 5120, 320
    blocks = oracle.quantize("q4_k", (0.02 * g.standard_normal((wrows, cols))).astype(np.float32))
    weight = upload(dev, "q4_k", wrows, cols, blocks)
    for n in (1, 2, 5, 8, 12, 40, 300):
        x = (3.0 * g.standard_normal((n, cols))).astype(np.float32)
        w = (1.0 + 0.1 * g.standard_normal(cols)).astype(np.float32)
        normed, out = dev.alloc(n * cols), dev.alloc(n * wrows)
        dev.normalize(normed, dev.buffer(x), dev.buffer(w), n * cols, 1e-6)
        launches = dev.launches
        dev.matmul(out, weight, normed)
        want_n = oracle.rmsnorm(x, w, 1e-6)
        close(dev.read(normed), want_n, 1e-5)
        # the device's own normalized rows (they differ from the CPU's by summation order) through the oracle
        want = oracle.matmul("q4_k", blocks, wrows, cols, dev.read(normed).reshape(n, cols))
        assert max_rel_err(dev.read(out), want) <= (2e-5 if n <= 2 or n > 8 else 1e-4), n
        assert dev.launches - launches == 1, "the product ran an activation prologue of its own"


def test_bf16_matmul_matches_cpu(dev, oracle):
    """matmul_matches_cpu (gpu/tests.rs:178-196): bf16 weights, the reference's
    shapes, generator and tolerance; and the gate matrices' shape in the model."""
    from dwim_b200 import Tensor
    rng = oracle.Lcg(4)
    shapes = [tuple(s) for s in KATS["bf16_matmul_shapes"]["shapes"]] + [(96, 5120, 1), (96, 5120, 5)]
    for rows, cols, n in shapes:
        wbits = (rng.floats(rows * cols).view(np.uint32) >> 16).astype(np.uint16)   # Rng::bf16, gpu/tests.rs:60-68
        x = rng.floats(n * cols)
        weight = dev.upload(Tensor("bf16", (rows, cols), wbits))
        assert np.array_equal(dev.dequantize(weight), oracle.bf16(wbits).reshape(rows, cols))
        out = dev.alloc(n * rows)
        dev.matmul(out, weight, dev.buffer(x))
        close(dev.read(out), oracle.matmul_bf16(wbits, rows, cols, x), 1e-4)


def test_argmax_on_the_device(dev, oracle):
    rng = np.random.default_rng(91)
    vocab = 151936
    for n in (1, 5):
        logits = rng.standard_normal((n, vocab)).astype(np.float32)
        logits[0, 777] = logits[0, 99999] = 9.0     # a tie: the first index wins (inference/qwen35/mod.rs:702-710)
        if n > 1:
            logits[1, :] = -np.inf
            logits[2, 5] = np.nan
            logits[3, 0] = 50.0
        got = dev.argmax(dev.buffer(logits), vocab)
        want = [oracle.argmax(row) for row in logits]
        assert got.tolist() == want


def test_back_to_back_products_see_their_own_inputs(dev, oracle):
    """Small-M kernels start while the kernel ahead still runs: every product of a
    chain must still use the input written just before it, and accumulate in order."""
    rng = np.random.default_rng(83)
    rows, cols = 640, 1024
    tensors = [oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)) for _ in range(2)]
    weights = [upload(dev, "q4_k", rows, cols, t) for t in tensors]
    xb, acc = dev.alloc(cols), dev.alloc(rows)
    xs = rng.standard_normal((12, cols)).astype(np.float32)
    want = np.zeros(rows, np.float32)
    for i, x in enumerate(xs):
        dev.write(xb, x)
        dev.matmul_add(acc, weights[i % 2], xb)        # acc += w . x, twelve times without a sync
        want = oracle.matmul_add("q4_k", tensors[i % 2], rows, cols, x, want).reshape(rows)
    assert max_rel_err(dev.read(acc), want) <= 2e-5


def test_gemm_above_the_batch_size(dev, oracle):
    """More tokens than Device::batch() in one call, ragged against every tile size."""
    rng = np.random.default_rng(89)
    rows, cols, n = 200, 512, 2049
    blocks = oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    x = rng.standard_normal((n, cols)).astype(np.float32)
    out = dev.alloc(n * rows)
    dev.matmul(out, upload(dev, "q4_k", rows, cols, blocks), dev.buffer(x))
    assert max_rel_err(dev.read(out), oracle.matmul("q4_k", blocks, rows, cols, x)) <= 2e-5


# ---- the benchmarked GEMM configurations at full size -----------------------------------------
def bf16_rows(oracle, rng, n, cols):
    """Config 2's activations: rows of N(0,1) scaled to RMS 1, rounded to bf16."""
    x = rng.standard_normal((n, cols)).astype(np.float32)
    x /= np.sqrt((x * x).mean(1, keepdims=True))
    bits = oracle.to_bf16(x)
    return bits, oracle.bf16(bits).reshape(n, cols)


def sampled_rows(rows, rng, count=384):
    """First, last and a ragged middle stretch of the 128-row tiles, plus random rows."""
    picks = set(range(min(rows, 130))) | set(range(max(0, rows - 130), rows)) | set(range(rows // 2 - 3, min(rows, rows // 2 + 64)))
    picks |= set(int(r) for r in rng.choice(rows, min(rows, count), replace=False))
    return np.array(sorted(picks))


_full_weights = {}


def full_weight(dev, rows, cols, seed):
    """A full-size Q4_K matrix, quantized on the device once per session."""
    key = (rows, cols, seed)
    if key not in _full_weights:
        w = 0.02 * np.random.default_rng(seed).standard_normal((rows, cols), dtype=np.float32)
        t = dev.quantize("q4_k", w)
        _full_weights.clear()                      # one at a time: 50 MB of blocks, 356 MB of f32 behind them
        _full_weights[key] = (t, dev.upload(t))
    return _full_weights[key]


@pytest.mark.parametrize("rows,cols,n", [
    (17408, 5120, 128), (17408, 5120, 512), (17408, 5120, 2048),       # config 2: gate / up
    (5120, 17408, 128), (5120, 17408, 2048),                            # the transposed down projection
    (17401, 5120, 512)])                                                # a ragged last row tile
def test_config2_gemm_full_size(dev, oracle, rows, cols, n):
    """BASELINE config 2 as the benchmark runs it: Q4_K W x bf16 X through the
    256-column tensor-core kernel, against the oracle on a row sample that covers
    the first, last and middle row tiles and every token; plus run-to-run bit
    equality over the whole output."""
    rng = np.random.default_rng(2000 + n)
    t, weight = full_weight(dev, rows, cols, seed=0 if rows != 17401 else 9)
    bits, x = bf16_rows(oracle, rng, n, cols)
    xb, out = dev.alloc(n * cols), dev.alloc(n * rows)
    dev.write_bf16(xb, bits)
    dev.matmul(out, weight, xb)
    got = dev.read(out).reshape(n, rows)
    assert np.isfinite(got).all()
    sample = sampled_rows(rows, rng)
    want = oracle.matmul("q4_k", t.select_rows(sample).data, sample.size, cols, x)
    err = max_rel_err(got[:, sample], want)
    assert err <= TOL, f"max relative error {err:.2e}"
    assert err <= 2e-5, f"exact products: only summation order may differ, got {err:.2e}"
    close_batch(got[:, sample], want, f"q4_k {rows}x{cols} n={n}")
    dev.matmul(out, weight, xb)
    assert np.array_equal(dev.read(out).reshape(n, rows), got)


@pytest.mark.parametrize("n", [17, 33, 130, 300])
def test_gemm_bf16_token_counts(dev, oracle, n):
    """bf16 activations (one f16 column per token) at every tile width of the
    tensor-core kernel: 32, 64, 256 columns, ragged against each."""
    rng = np.random.default_rng(3000 + n)
    rows, cols = 1000, 5120
    blocks = oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    bits, x = bf16_rows(oracle, rng, n, cols)
    xb, out = dev.alloc(n * cols), dev.alloc(n * rows)
    dev.write_bf16(xb, bits)
    dev.matmul(out, upload(dev, "q4_k", rows, cols, blocks), xb)
    assert max_rel_err(dev.read(out).reshape(n, rows), oracle.matmul("q4_k", blocks, rows, cols, x)) <= 2e-5


@pytest.mark.parametrize("bf16", [True, False])
def test_gemm_fused_epilogues_at_256_columns(dev, oracle, bf16):
    """matmul_add and swiglu through the 256-column kernel (300 tokens of bf16
    input, or 150 of f32 travelling as two columns each)."""
    rng = np.random.default_rng(3100 + bf16)
    rows, cols, n = 1030, 5120, 300 if bf16 else 150
    gate = oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    up = oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    xb = dev.alloc(n * cols)
    if bf16:
        bits, x = bf16_rows(oracle, rng, n, cols)
        dev.write_bf16(xb, bits)
    else:
        x = rng.standard_normal((n, cols)).astype(np.float32)
        dev.write(xb, x)
    wg, wu = upload(dev, "q4_k", rows, cols, gate), upload(dev, "q4_k", rows, cols, up)
    out, scratch = dev.alloc(n * rows), dev.alloc(n * rows)
    dev.swiglu(out, wg, wu, xb, scratch)
    assert max_rel_err(dev.read(out), oracle.swiglu("q4_k", gate, up, rows, cols, x)) <= 1e-4
    res = rng.standard_normal((n, rows)).astype(np.float32)
    acc = dev.buffer(res)
    dev.matmul_add(acc, wg, xb)
    got, want = dev.read(acc).reshape(n, rows), oracle.matmul_add("q4_k", gate, rows, cols, x, res)
    assert max_rel_err(got - res, want - res) <= 1e-4


@pytest.mark.parametrize("fmt", ["q6_k", "q8_0"])
@pytest.mark.parametrize("n,bf16", [(12, False), (33, False), (65, True), (130, False), (300, True)])
def test_dense_pair_gemm_for_q6_k_and_q8_0(dev, oracle, fmt, n, bf16):
    """Above the small-M kernel's eight tokens Q6_K and Q8_0 go in groups of eight
    (up to 64 tokens) and then through the dense kernel on dequantized f16 pairs:
    every tile width, ragged rows, both activation forms, fused epilogues.  The
    dense kernel sums the whole of K in the tensor cores' accumulator, whose
    additions are not rounded to nearest: its error grows with K (6e-5 at 5120)."""
    rng = np.random.default_rng(4000 + n)
    rows, cols = 1030, 2304
    gate = oracle.quantize(fmt, (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    up = oracle.quantize(fmt, (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    xb = dev.alloc(n * cols)
    if bf16:
        bits, x = bf16_rows(oracle, rng, n, cols)
        dev.write_bf16(xb, bits)
    else:
        x = rng.standard_normal((n, cols)).astype(np.float32)
        dev.write(xb, x)
    wg, wu = upload(dev, fmt, rows, cols, gate), upload(dev, fmt, rows, cols, up)
    out, scratch = dev.alloc(n * rows), dev.alloc(n * rows)
    dev.matmul(out, wg, xb)
    assert max_rel_err(dev.read(out), oracle.matmul(fmt, gate, rows, cols, x)) <= (2e-5 if n <= 64 else 1e-4)
    dev.swiglu(out, wg, wu, xb, scratch)
    assert max_rel_err(dev.read(out), oracle.swiglu(fmt, gate, up, rows, cols, x)) <= 1e-4
    res = rng.standard_normal((n, rows)).astype(np.float32)
    acc = dev.buffer(res)
    dev.matmul_add(acc, wu, xb)
    got, want = dev.read(acc).reshape(n, rows), oracle.matmul_add(fmt, up, rows, cols, x, res)
    assert max_rel_err(got - res, want - res) <= 1e-4


@pytest.mark.parametrize("fmt,rows,cols,n", [("q6_k", 151936, 5120, 128), ("q8_0", 5120, 5120, 2048), ("q6_k", 20000, 5120, 512)])
def test_dense_pair_gemm_full_size(dev, oracle, fmt, rows, cols, n):
    """Config 3's matrices at GEMM sizes: several row panels (the vocabulary head),
    against the oracle on sampled rows and every token."""
    rng = np.random.default_rng(4100 + n)
    srows = 2048                                      # distinct rows; the matrix repeats them (generation time)
    base = oracle.quantize(fmt, (0.02 * rng.standard_normal((srows, cols))).astype(np.float32))
    from dwim_b200 import Tensor, row_bytes
    reps = -(-rows // srows)
    blocks = np.tile(base.reshape(srows, -1), (reps, 1))[:rows].reshape(-1)
    weight = dev.upload(Tensor(fmt, (rows, cols), blocks))
    bits, x = bf16_rows(oracle, rng, n, cols)
    xb, out = dev.alloc(n * cols), dev.alloc(n * rows)
    dev.write_bf16(xb, bits)
    dev.matmul(out, weight, xb)
    got = dev.read(out).reshape(n, rows)
    sample = sampled_rows(rows, rng)
    rb = row_bytes(fmt, cols)
    want = oracle.matmul(fmt, blocks.reshape(rows, rb)[sample].reshape(-1), sample.size, cols, x)
    assert max_rel_err(got[:, sample], want) <= 2e-4


# ---- the boundary: a caller's stream, a caller's writes -----------------------------------------
def test_adopted_stream_and_touch(oracle):
    """The composition an engine would use: the library opened on the caller's
    stream, a buffer wrapped over the caller's memory, a kernel of the caller's
    (torch, on that stream) rewriting it between two products.  After touch the
    second product sees the new data; the stream orders everything."""
    import torch
    from dwim_b200 import B200, Tensor
    stream = torch.cuda.Stream()
    d = B200(0, stream=stream.cuda_stream)
    try:
        rng = np.random.default_rng(97)
        rows, cols, n = 640, 1024, 3
        blocks = oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
        weight = d.upload(Tensor("q4_k", (rows, cols), blocks))
        x1 = rng.standard_normal((n, cols)).astype(np.float32)
        x2 = rng.standard_normal((n, cols)).astype(np.float32)
        with torch.cuda.stream(stream):
            xt = torch.from_numpy(x1).cuda(non_blocking=False)
            x2t = torch.from_numpy(x2).cuda(non_blocking=False)
            ot = torch.empty(n * rows, dtype=torch.float32, device="cuda")
        stream.synchronize()
        xb, out = d.wrap(xt.data_ptr(), n * cols), d.wrap(ot.data_ptr(), n * rows)
        d.matmul(out, weight, xb)
        with torch.cuda.stream(stream):
            first = ot.clone()
            xt.copy_(x2t)                    # the caller's kernel, ordered by the shared stream
        d.touch(xb)
        d.matmul(out, weight, xb)
        with torch.cuda.stream(stream):
            second = ot.clone()
        stream.synchronize()
        d.sync()
        assert max_rel_err(first.cpu().numpy(), oracle.matmul("q4_k", blocks, rows, cols, x1)) <= 2e-5
        assert max_rel_err(second.cpu().numpy(), oracle.matmul("q4_k", blocks, rows, cols, x2)) <= 2e-5
    finally:
        d.close()


@pytest.mark.parametrize("n", [1, 6, 40])
def test_feed_forward_block_push_exchange_in_a_world_of_one(dev, oracle, n):
    """matmul_scatter, reduce_gather and the barriers with a single rank: the
    whole result is this rank's slice, its one slot the whole sum."""
    from dwim_b200 import Tensor, shard
    rng = np.random.default_rng(161 + n)
    hidden, inner = 512, 1024
    mk = lambda r, c: Tensor("q4_k", (r, c), oracle.quantize("q4_k", (0.05 * rng.standard_normal((r, c))).astype(np.float32)))
    gate, up, down = mk(inner, hidden), mk(inner, hidden), mk(hidden, inner)
    x = rng.standard_normal((n, hidden)).astype(np.float32)
    block = shard.ShardedFFN(dev, gate, up, down, exchange="push")
    got = dev.read(block.forward(dev.buffer(x))).reshape(n, hidden)
    h = oracle.swiglu("q4_k", gate.data, up.data, inner, hidden, x)
    want = oracle.matmul("q4_k", down.data, hidden, inner, h).reshape(n, hidden)
    assert max_rel_err(got, want) <= 5e-5


def test_shared_buffer_in_a_world_of_one(dev, oracle):
    """matmul_gather and the barrier with a single rank: two row shards written
    into one shared result at their offsets, as two ranks would."""
    rng = np.random.default_rng(99)
    rows, cols = 1000, 1024
    from dwim_b200 import Tensor
    t = Tensor("q4_k", (rows, cols), oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)))
    for n in (1, 5, 40):
        x = rng.standard_normal((n, cols)).astype(np.float32)
        out, handle = dev.shared_alloc(n * rows)
        dev.shared_connect(out, 1, 0, [handle])
        xb = dev.buffer(x)
        for b, e in ((0, 496), (496, 1000)):
            dev.matmul_gather(out, dev.upload(t.slice_rows(b, e)), xb, b, rows)
        dev.shared_barrier(out)
        assert max_rel_err(dev.read(out), oracle.matmul("q4_k", t.data, rows, cols, x)) <= 2e-5


def test_shared_result_of_two_ranks_on_one_gpu(dev, oracle):
    """Two ranks of one process (dwim_b200_shared_connect_local): each rank's matmul_gather must put
    its rows into BOTH copies of the shared result -- the small-M kernel's peer stores, the
    tensor-core kernel's TMA stores (slices on 16-byte boundaries) and its register stores (a slice
    that is not).  No barrier kernel: both ranks share the GPU, and the stream orders them."""
    from dwim_b200 import Tensor
    rng = np.random.default_rng(101)
    cols = 1024
    for rows, cut in ((1000, 496), (1002, 499)):          # aligned slices / a slice that starts on an odd row
        t = Tensor("q4_k", (rows, cols), oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)))
        shards = [(0, cut, dev.upload(t.slice_rows(0, cut))), (cut, rows, dev.upload(t.slice_rows(cut, rows)))]
        for n in (3, 40, 300):
            x = rng.standard_normal((n, cols)).astype(np.float32)
            want = oracle.matmul("q4_k", t.data, rows, cols, x)
            copies = [dev.shared_alloc(n * rows)[0] for _ in range(2)]
            for r in range(2):
                dev.shared_connect_local(copies[r], 2, r, copies)
            xb = dev.buffer(x)
            for r, (b, e, w) in enumerate(shards):
                dev.matmul_gather(copies[r], w, xb, b, rows)
            for r in range(2):
                assert max_rel_err(dev.read(copies[r]), want) <= 2e-5, (rows, n, r)


def test_activation_precision_f16(dev, oracle):
    """f32 activations as one f16 column on request (the reference device's own precision, `halves`,
    gpu/cuda/mod.rs:313-384): it passes the reference's gate for that device (rms error below 1e-3 of
    the typical magnitude and the worst below 1e-2, gpu/tests.rs:198-211), not this library's 1e-3
    on the worst element, and is really another path than the exact one."""
    from dwim_b200 import DeviceError
    g = np.random.default_rng(91)
    rows, cols, n = 384, 5120, 40
    blocks = oracle.quantize("q4_k", (0.02 * g.standard_normal((rows, cols))).astype(np.float32))
    weight = upload(dev, "q4_k", rows, cols, blocks)
    x = g.standard_normal((n, cols)).astype(np.float32)
    x[3] *= 1e4                                    # a token of another magnitude keeps its own scale
    want = oracle.matmul("q4_k", blocks, rows, cols, x)
    xb, out = dev.buffer(x), dev.alloc(n * rows)
    dev.matmul(out, weight, xb)
    exact = max_rel_err(dev.read(out), want)
    dev.activation_precision("f16")
    try:
        dev.matmul(out, weight, xb)
        got = dev.read(out).reshape(n, rows)
        half = max_rel_err(got, want)
        typical = np.sqrt((want.reshape(n, rows) ** 2).mean(axis=1, keepdims=True))      # per token: one is 1e4 times the others
        half_rms = float(np.sqrt((((got - want.reshape(n, rows)) / typical) ** 2).mean()))
    finally:
        dev.activation_precision("exact")
    dev.matmul(out, weight, xb)
    again = max_rel_err(dev.read(out), want)
    assert exact <= 1e-5 and again <= 1e-5, (exact, again)
    assert 1e-5 < half <= 1e-2 and half_rms <= 1e-3, (half, half_rms)
    with pytest.raises(DeviceError):
        dev._check(dev._L.dwim_b200_activation_precision(dev._ctx, 7))
