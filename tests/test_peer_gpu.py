"""The multi-GPU forms on two GPUs of one box: two processes, one per GPU,
exchange their handles over gloo.  The small all-reduce over peer memory on
vectors of several lengths many times over (slots are reused every other
call); the tensor-parallel feed-forward block with that reduction against the
CPU; the row-sharded product whose epilogue stores into every rank's copy of
the result; and a wait that runs out (a peer that never arrives), reported as
a status and an error code with nothing left hanging."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank: int, world: int, port: int, queue):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import oracle
    from dwim_b200 import B200, Tensor, shard
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dev = B200(rank)
        peer = shard.PeerReduce(dev, rank, world, 8192)
        for n in (1, 5, 1024, 1025, 5120, 8192):
            for it in range(6):
                vecs = [np.random.default_rng(1000 * n + 10 * it + r).standard_normal(n).astype(np.float32) for r in range(world)]
                buf = dev.buffer(vecs[rank])
                peer(buf, n)
                want = vecs[0].copy()
                for v in vecs[1:]:
                    want = want + v                      # rank order, as the kernel adds
                got = dev.read(buf)
                assert np.array_equal(got, want), (n, it, rank, np.abs(got - want).max())
        # the feed-forward block, one and two tokens, partial sums through the mailbox
        rng = np.random.default_rng(17)                  # every rank draws the same block
        hidden, inner = 512, 1024
        mk = lambda r, c: Tensor("q4_k", (r, c), oracle.quantize("q4_k", (0.05 * rng.standard_normal((r, c))).astype(np.float32)))
        gate, up, down = mk(inner, hidden), mk(inner, hidden), mk(hidden, inner)
        block = shard.ShardedFFN(dev, gate, up, down, rank, world, peer=peer)
        for n in (1, 2):
            x = rng.standard_normal((n, hidden)).astype(np.float32)
            got = dev.read(block.forward(dev.buffer(x))).reshape(n, hidden)
            h = oracle.swiglu("q4_k", gate.data, up.data, inner, hidden, x)
            want = oracle.matmul("q4_k", down.data, hidden, inner, h).reshape(n, hidden)
            err = np.abs(got - want).max() / np.sqrt((want * want).mean())
            assert err < 5e-5, (n, rank, err)
        # the same block with the reduction fused into the down projection: partial sums stored into
        # their rows' owners, added there, the sums stored into every rank's copy (one to 300 tokens:
        # the small-M kernel, the token groups, the tensor-core kernel)
        pushed = shard.ShardedFFN(dev, gate, up, down, rank, world, exchange="push")
        for n in (1, 5, 12, 300):
            x = rng.standard_normal((n, hidden)).astype(np.float32)
            got = dev.read(pushed.forward(dev.buffer(x))).reshape(n, hidden)
            h = oracle.swiglu("q4_k", gate.data, up.data, inner, hidden, x)
            want = oracle.matmul("q4_k", down.data, hidden, inner, h).reshape(n, hidden)
            err = np.abs(got - want).max() / np.sqrt((want * want).mean())
            assert err < 5e-5, ("push ffn", n, rank, err)
        # the row-sharded product with the all-gather fused into its epilogue: every rank's copy of
        # the shared result must hold every rank's rows (uneven shards: 1000 rows over two ranks)
        rows, cols = 1000, 1024
        t = Tensor("q4_k", (rows, cols), oracle.quantize("q4_k", (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)))
        sharded = shard.RowShardedPush(dev, t, rank, world, max_tokens=40)
        for n in (1, 5, 40, 2, 40):
            x = rng.standard_normal((n, cols)).astype(np.float32)
            got = dev.read(sharded.matmul(dev.buffer(x))).reshape(n, rows)
            want = oracle.matmul("q4_k", t.data, rows, cols, x)
            err = np.abs(got - want).max() / np.sqrt((want * want).mean())
            assert err < 2e-5, ("push", n, rank, err)
        dev.sync()
        # a peer that never arrives: rank 0 alone enters the all-reduce; its bounded wait runs out,
        # the kernel ends, and the next sync reports the time-out.  The context stays usable.
        dist.barrier()
        if rank == 0:
            from dwim_b200 import DeviceError
            buf = dev.buffer(np.ones(8, np.float32))
            peer(buf, 8)
            try:
                dev.sync()
                raise AssertionError("the lone all-reduce did not time out")
            except DeviceError as e:
                assert e.code == -6, e
            dev.sync()                                   # the status was cleared: usable again
            assert np.array_equal(dev.read(dev.buffer(np.arange(4, dtype=np.float32))), np.arange(4, dtype=np.float32))
        # a context used from a thread that never chose a device (its current device is GPU 0): every
        # entry point works on the context's own device
        import threading
        seen = {}

        def from_thread():
            try:
                d2 = B200(rank)
                v = np.arange(4096, dtype=np.float32) + rank
                seen["ok"] = bool(np.array_equal(d2.read(d2.buffer(v)), v) and np.array_equal(dev.read(dev.buffer(v)), v))
                d2.close()
            except Exception as e:   # noqa: BLE001
                seen["ok"] = repr(e)
        th = threading.Thread(target=from_thread)
        th.start()
        th.join()
        assert seen.get("ok") is True, seen
        dist.barrier()
        queue.put((rank, "ok"))
    except Exception as e:   # noqa: BLE001 - reported to the parent
        queue.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_peer_allreduce_on_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on the box")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue, port, world = ctx.Queue(), _free_port(), 2
    procs = [ctx.Process(target=_rank, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results
