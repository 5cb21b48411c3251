"""The C-ABI library and the host-side logic, without a GPU: the library
loads, exports every symbol the header declares, and refuses to open a device
that is not there.  No kernel runs here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from dwim_b200 import build, _lib
    build.build()
    return _lib.lib()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "dwim_b200.h")).read()
    return sorted(set(re.findall(r"DWIM_B200_API\s+[^;(]*?\b(dwim_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(L):
    from dwim_b200 import _lib
    names = header_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(L, name), f"{name} is declared in the header but not exported"
    # and the Python binding declares exactly the header's functions
    assert sorted(_lib.SIGNATURES) == names


def test_open_without_a_device_fails_loudly(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from dwim_b200 import B200, DeviceError
    with pytest.raises(DeviceError) as e:
        B200(0)
    assert e.value.code == -5     # ENODEV: there is no CPU fallback to fall back to
    assert b"CUDA" in L.dwim_b200_last_error(None) or b"device" in L.dwim_b200_last_error(None)


def test_null_handles_are_rejected(L):
    assert L.dwim_b200_sync(None) == -1
    assert L.dwim_b200_matmul(None, None, None, None) == -1
    assert L.dwim_b200_alloc(None, 16, None) == -1
    assert L.dwim_b200_buffer_len(None) == 0
    assert L.dwim_b200_batch(None) == 0


def test_row_bytes_matches_the_block_sizes(L):
    from dwim_b200 import Q4_K, Q6_K, Q8_0, row_bytes
    assert L.dwim_b200_row_bytes(Q4_K, 5120) == 20 * 144 == row_bytes("q4_k", 5120)
    assert L.dwim_b200_row_bytes(Q6_K, 5120) == 20 * 210 == row_bytes("q6_k", 5120)
    assert L.dwim_b200_row_bytes(Q8_0, 5120) == 160 * 34 == row_bytes("q8_0", 5120)
    assert L.dwim_b200_row_bytes(Q4_K, 5000) == 0      # not whole blocks
    assert L.dwim_b200_row_bytes(Q8_0, 48) == 0
    assert L.dwim_b200_row_bytes(7, 256) == 0          # unknown format
    with pytest.raises(ValueError):
        row_bytes("q4_k", 5000)
    # the sizes BASELINE quotes
    assert 17408 * row_bytes("q4_k", 5120) == 50_135_040
    assert 151936 * row_bytes("q6_k", 5120) == 638_131_200
    assert 5120 * row_bytes("q8_0", 5120) == 27_852_800


def test_shard_rows_covers_every_row_once(L):
    from dwim_b200 import shard_rows
    for rows, world, align in [(17408, 8, 16), (17408, 2, 16), (5120, 4, 16), (151936, 8, 16), (77, 4, 16), (1, 8, 16),
                               (0, 2, 16), (68, 8, 1), (100, 3, 7)]:
        cuts = [shard_rows(rows, r, world, align) for r in range(world)]
        assert cuts[0][0] == 0 and cuts[-1][1] == rows
        for (b0, e0), (b1, e1) in zip(cuts, cuts[1:]):
            assert e0 == b1 and b0 <= e0
        sizes = [e - b for b, e in cuts]
        assert sizes[0] == max(sizes)                     # rank 0 holds the most
        assert all(b % align == 0 for b, _ in cuts if b < rows)
        assert max(sizes) - min(sizes) < 2 * align
    # 68 superblocks over 8 ranks: four ranks of 9 and four of 8
    assert [e - b for b, e in (shard_rows(68, r, 8, 1) for r in range(8))] == [9, 9, 9, 9, 8, 8, 8, 8]
    b, e = C.c_size_t(), C.c_size_t()
    assert L.dwim_b200_shard_rows(10, 2, 2, 1, C.byref(b), C.byref(e)) == -1
    assert L.dwim_b200_shard_rows(10, 0, 0, 1, C.byref(b), C.byref(e)) == -1


def test_tensor_selects_rows_and_column_groups(oracle):
    # after select_rows / select_column_groups, gpu/mod.rs:72-136 and their
    # tests at gpu/cpu.rs:455-508: selecting on the packed bytes equals
    # selecting on the decoded weights
    from dwim_b200 import Tensor
    rng = np.random.default_rng(5)
    w = (0.02 * rng.standard_normal((12, 1024))).astype(np.float32)
    for fmt, width in (("q4_k", 256), ("q6_k", 512), ("q8_0", 64)):
        t = Tensor(fmt, w.shape, oracle.quantize(fmt, w))
        whole = oracle.dequantize(fmt, t.data, 12, 1024)
        rows = [3, 3, 0, 11]
        s = t.select_rows(rows)
        assert s.shape == (4, 1024)
        assert np.array_equal(oracle.dequantize(fmt, s.data, 4, 1024), whole[rows])
        groups = [1, 0, 1] if fmt != "q8_0" else [5, 0, 15, 5]
        c = t.select_column_groups(width, groups)
        assert c.shape == (12, len(groups) * width)
        want = np.concatenate([whole[:, g * width:(g + 1) * width] for g in groups], axis=1)
        assert np.array_equal(oracle.dequantize(fmt, c.data, 12, c.cols), want)
        assert np.array_equal(t.slice_rows(2, 7).data, t.select_rows(range(2, 7)).data)
    with pytest.raises(ValueError):
        Tensor("q4_k", (2, 256), np.zeros(100, np.uint8))
    with pytest.raises(ValueError):
        Tensor("q4_k", (2, 512), np.zeros(2 * 288, np.uint8)).select_column_groups(128, [0])   # not whole blocks
