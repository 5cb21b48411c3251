"""The reference engine's own CUDA tile kernel (matmul_tile.cu:94-258), compiled
from its sources into oracle/_ref/ and fed by this repository's restatement of
its host side (oracle/ref_gpu.py), against the CPU oracle's Q4_0 dot
(gpu/quant.rs:128-152).  This pins the harness that races that kernel against
this library's kernels in the benchmark: a baseline that computed something
else would be no baseline.  Tolerance: the reference's own for its tensor-core
path (gpu/tests.rs:198-211), which rounds weights and activations to f16."""
import numpy as np
import pytest

from conftest import close_batch


def test_tiling_restates_q4_0_words(oracle):
    """gpu/cuda/mod.rs:642-704 on a matrix with a ragged last group of rows."""
    from oracle import ref_gpu
    rng = np.random.default_rng(3)
    w = (0.02 * rng.standard_normal((130, 96))).astype(np.float32)
    scales, quants = ref_gpu.quantize_q4_0(w)
    tiled, tiled_scales = ref_gpu.tile_q4_0(scales, quants)
    assert tiled.shape == (2, 2, 128, 8) and tiled_scales.shape == (2, 2, 2, 128)
    for row, block in [(0, 0), (5, 1), (129, 2), (77, 2)]:
        g, r, t, v = row // 128, row % 128, block // 2, block % 2
        b = quants[row, block]
        for i in range(4):
            want = int.from_bytes(bytes([b[2 * i], b[2 * i + 8], b[2 * i + 1], b[2 * i + 9]]), "little")
            assert tiled[g, t, r, i * 2 + v] == want
        assert tiled_scales[g, t, v, r] == scales[row, block]
    assert not tiled[1, :, 2:].any() and not tiled_scales[1, :, :, 2:].any()     # rows past the matrix
    assert not tiled[:, 1, :, 1::2].any() and not tiled_scales[:, 1, 1].any()    # the block past the row


@pytest.mark.gpu
def test_reference_tile_kernel_matches_its_cpu_path(dev, oracle):
    import torch
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("oracle/_ref/dwim_tile.cubin has not been built (make -C oracle ref_gpu, where the reference's sources are)")
    rng = oracle.Lcg(80)
    rows, cols, n = 1030, 1152, 130                     # gpu/tests.rs:225-237: ragged rows, wide and narrow token tiles
    w = rng.floats(rows * cols).reshape(rows, cols)
    x = oracle.Lcg(rows + n).floats(n * cols).reshape(n, cols)
    scales, quants = ref_gpu.quantize_q4_0(w)
    tiled, tiled_scales = ref_gpu.tile_q4_0(scales, quants)
    ref = ref_gpu.RefTile()
    d_w = torch.from_numpy(tiled.view(np.int32)).cuda()
    d_s = torch.from_numpy(tiled_scales.view(np.int16)).cuda()
    d_x = torch.from_numpy(oracle.to_f16(x).view(np.int16)).cuda()      # the reference's to_f16: nearest, clamped
    out = torch.zeros(n * rows, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    ref.matmul(out.data_ptr(), d_w.data_ptr(), d_s.data_ptr(), d_x.data_ptr(), rows, cols, n, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(n, rows)
    want = np.empty((n, rows), np.float32)
    for r in range(rows):
        for t in range(n):
            want[t, r] = oracle.dot_q4_0_split(scales[r], quants[r].reshape(-1), x[t])
    close_batch(got, want, "reference tile kernel, Q4_0 1030x1152 n=130")
