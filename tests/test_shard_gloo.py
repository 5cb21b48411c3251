"""The multi-GPU path's host logic on CPU: two gloo ranks shard a matrix by
output rows, each multiplies its slice (the oracle stands in for the GPU
kernel), the slices are all-gathered and re-assembled, and every rank must
hold the unsharded product."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank: int, world: int, port: int, cases, queue):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import oracle
    from dwim_b200 import Tensor, shard
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        for fmt, rows, cols, n, align in cases:
            rng = np.random.default_rng(7)          # every rank draws the same matrix
            w = (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)
            x = rng.standard_normal((n, cols)).astype(np.float32)
            whole = Tensor(fmt, (rows, cols), oracle.quantize(fmt, w))
            begin, end = shard.plan(rows, world, align)[rank]
            mine = whole.slice_rows(begin, end)
            pr = shard.part_rows(rows, world, align)
            part = np.zeros((n, pr), np.float32)
            if end > begin:
                part[:, : end - begin] = oracle.matmul(fmt, mine.data, end - begin, cols, x)
            gathered = [torch.empty(n * pr) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(part.reshape(-1)))
            parts = np.stack([g.numpy() for g in gathered])
            got = shard.assemble(parts, n, rows, world, align)
            want = oracle.matmul(fmt, whole.data, rows, cols, x)
            assert np.array_equal(got, want), (fmt, rows, cols, n, rank)
        queue.put((rank, "ok"))
    except Exception as e:   # noqa: BLE001 - reported to the parent
        queue.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_row_sharding_over_two_gloo_ranks():
    import torch.multiprocessing as mp
    cases = [("q4_k", 96, 512, 3, 16), ("q8_0", 77, 64, 2, 16), ("q6_k", 40, 256, 1, 16), ("q4_k", 17, 256, 2, 16)]
    ctx = mp.get_context("spawn")
    queue, port, world = ctx.Queue(), _free_port(), 2
    procs = [ctx.Process(target=_rank, args=(r, world, port, cases, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results


def test_assemble_is_the_inverse_of_the_plan():
    from dwim_b200 import shard
    rng = np.random.default_rng(1)
    for rows, world, align, n in [(17408, 8, 16, 2), (5120, 4, 16, 3), (77, 4, 16, 2), (68, 8, 1, 1), (5, 8, 16, 1)]:
        full = rng.standard_normal((n, rows)).astype(np.float32)
        pr = shard.part_rows(rows, world, align)
        parts = np.zeros((world, n, pr), np.float32)
        for r, (b, e) in enumerate(shard.plan(rows, world, align)):
            parts[r, :, : e - b] = full[:, b:e]
        assert np.array_equal(shard.assemble(parts, n, rows, world, align), full)


def _ffn_rank(rank: int, world: int, port: int, cases, queue):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import oracle
    from dwim_b200 import Tensor, shard
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        for hidden, inner, n in cases:
            rng = np.random.default_rng(11)         # every rank draws the same block
            mk = lambda r, c: Tensor("q4_k", (r, c), oracle.quantize("q4_k", (0.05 * rng.standard_normal((r, c))).astype(np.float32)))
            gate, up, down = mk(inner, hidden), mk(inner, hidden), mk(hidden, inner)
            x = rng.standard_normal((n, hidden)).astype(np.float32)
            g, u, d = shard.ffn_shard(gate, up, down, rank, world)
            b, e = shard.ffn_cuts(inner, world)[rank]
            assert g.shape == u.shape == (e - b, hidden) and d.shape == (hidden, e - b)
            # the rank's K slice of down decodes to the same weights as the whole matrix's columns
            partial = np.zeros((n, hidden), np.float32)
            if e > b:
                assert np.array_equal(oracle.dequantize("q4_k", d.data, hidden, e - b),
                                      oracle.dequantize("q4_k", down.data, hidden, inner)[:, b:e])
                h = oracle.swiglu("q4_k", g.data, u.data, e - b, hidden, x).reshape(n, e - b)
                partial = oracle.matmul("q4_k", d.data, hidden, e - b, h).reshape(n, hidden)
            t = torch.from_numpy(partial.copy())
            dist.all_reduce(t)
            h = oracle.swiglu("q4_k", gate.data, up.data, inner, hidden, x).reshape(n, inner)
            want = oracle.matmul("q4_k", down.data, hidden, inner, h).reshape(n, hidden)
            # the ranks' partial sums are added in another order than one row's blocks: fp32 noise only
            err = np.abs(t.numpy() - want).max() / np.sqrt((want * want).mean())
            assert err < 1e-5, (hidden, inner, n, rank, err)
        queue.put((rank, "ok"))
    except Exception as e:   # noqa: BLE001 - reported to the parent
        queue.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_feed_forward_block_over_two_gloo_ranks():
    """gate/up by rows, down by the same K blocks, one all-reduce: the sum of the
    ranks' partial outputs is the unsharded block's output."""
    import torch.multiprocessing as mp
    cases = [(256, 1024, 2), (512, 768, 1), (256, 256, 3)]   # the last: one rank holds nothing
    ctx = mp.get_context("spawn")
    queue, port, world = ctx.Queue(), _free_port(), 2
    procs = [ctx.Process(target=_ffn_rank, args=(r, world, port, cases, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results


def test_feed_forward_cuts_match_the_model():
    from dwim_b200 import shard
    # 17408 / 256 = 68 blocks: even over 2 and 4 ranks, 9 + 9 + 9 + 9 + 8 + 8 + 8 + 8 over 8
    assert [e - b for b, e in shard.ffn_cuts(17408, 8)] == [2304] * 4 + [2048] * 4
    assert [e - b for b, e in shard.ffn_cuts(17408, 4)] == [4352] * 4
    cuts = shard.ffn_cuts(17408, 8)
    assert cuts[0][0] == 0 and cuts[-1][1] == 17408 and all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
