"""The entry point that allocates nothing, ``dwim_b200_matmul_static``.

Some callers cannot allocate device memory when they multiply: their GPU
memory is one arena sized at start-up, or they run where cudaMalloc is not
allowed.  For them the library keeps the activations' operand scratch in a
fixed array of its own.  This checks, through the C ABI, that the entry point
gives what ``dwim_b200_matmul`` gives, on two calls in a row (the second must
not see anything of the first in the shared array), and that it refuses what
does not fit.  Collected last on purpose: a run that stops at the first
failure has then already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k", "q8_0"])
def test_static_scratch_matmul_matches_the_allocating_one(dev, oracle, fmt):
    from dwim_b200 import Tensor
    rng = np.random.default_rng(61)
    rows, cols = 333, 5120
    blocks = oracle.quantize(fmt, (0.02 * rng.standard_normal((rows, cols))).astype(np.float32))
    weight = dev.upload(Tensor(fmt, (rows, cols), blocks))
    for n in (5, 1):                                   # two calls in a row, the larger first
        x = rng.standard_normal((n, cols)).astype(np.float32)
        xb, want_b, got_b = dev.buffer(x), dev.alloc(n * rows), dev.alloc(n * rows)
        dev.matmul(want_b, weight, xb)                 # the existing entry point
        dev.matmul_static(got_b, weight, xb)           # the one that allocates nothing
        want, got = dev.read(want_b), dev.read(got_b)
        # the same kernels in the same order: the same bits
        assert np.array_equal(got, want)
        ref = oracle.matmul(fmt, blocks, rows, cols, x).ravel()
        den = np.maximum(np.abs(ref), np.sqrt(np.mean(ref * ref)))
        assert np.max(np.abs(got - ref) / den) <= 2e-5
        # and it allocates nothing: the device's free memory is the same before and after
        dev.sync()
        free_before = dev.memory()
        dev.matmul_static(got_b, weight, xb)
        dev.sync()
        assert dev.memory() == free_before
        assert np.array_equal(dev.read(got_b), want)


def test_static_scratch_wrapper_checks_lengths(dev, oracle):
    """A short output buffer must be refused on the host, not written past on the device."""
    from dwim_b200 import DeviceError, Tensor
    blocks = oracle.quantize("q8_0", np.ones((16, 256), np.float32))
    weight = dev.upload(Tensor("q8_0", (16, 256), blocks))
    with pytest.raises(DeviceError):
        dev.matmul_static(dev.alloc(2 * 16 - 1), weight, dev.alloc(2 * 256))
    with pytest.raises(DeviceError):
        dev.matmul_static(dev.alloc(2 * 16), weight, dev.alloc(2 * 256 + 3))


def test_static_scratch_refuses_what_does_not_fit(dev, oracle):
    from dwim_b200 import DeviceError, Tensor
    rows, cols = 16, 5120
    blocks = oracle.quantize("q8_0", np.ones((rows, cols), np.float32))
    weight = dev.upload(Tensor("q8_0", (rows, cols), blocks))
    with pytest.raises(DeviceError) as e:              # more tokens than the small-M kernel takes at once
        dev.matmul_static(dev.alloc(9 * rows), weight, dev.alloc(9 * cols))
    assert "at most" in str(e.value)
    wide = 8 * 65536                                   # 8 tokens of 65536 columns: 1.7 MB of operand scratch
    blocks = oracle.quantize("q8_0", np.ones((1, 65536), np.float32))
    weight = dev.upload(Tensor("q8_0", (1, 65536), blocks))
    with pytest.raises(DeviceError) as e:
        dev.matmul_static(dev.alloc(8), weight, dev.alloc(wide))
    assert "fixed array" in str(e.value)
    dev.sync()
