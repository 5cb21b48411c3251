"""Sharding over the GPUs of one node: a weight matrix by rows, and the
feed-forward block tensor-parallel (rows of gate/up, columns of down).

The reference engine is single-GPU (gpu/cuda/mod.rs:230 opens device 0 and
nothing else); this is new.  Output rows of ``out[t] = W . x[t]`` are
independent, so rank ``r`` of ``world`` holds rows ``[begin_r, end_r)`` of W —
cut at multiples of ``align`` rows, blocks untouched — multiplies them, and one
all-gather re-assembles the token-major result on every rank:

    rank r:   part_r[t, :] = W[begin_r:end_r] . x[t]            (its own GPU)
    exchange: parts = all_gather(part_r)       [world, n, part_rows]
    assemble: out[t, begin_r:end_r] = parts[r, t, :end_r-begin_r]

``plan`` and ``assemble`` are the host-side statement of that layout (the
device does ``assemble`` with ``B200.gather_rows``); ``RowSharded`` runs it
with one process per GPU over ``torch.distributed`` (NCCL).
"""
from __future__ import annotations

import numpy as np

from .device import B200, shard_rows
from .tensor import Tensor


def plan(rows: int, world: int, align: int = 16):
    """[(begin, end)] per rank; rank 0 holds the most rows."""
    return [shard_rows(rows, r, world, align) for r in range(world)]


def part_rows(rows: int, world: int, align: int = 16) -> int:
    """Rows of the common (padded) slice every rank contributes to the all-gather."""
    b, e = shard_rows(rows, 0, world, align)
    return e - b


def assemble(parts: np.ndarray, n: int, rows: int, world: int, align: int = 16) -> np.ndarray:
    """Token-major [n, rows] from the gathered [world, n, part_rows] slices."""
    pr = part_rows(rows, world, align)
    parts = np.asarray(parts).reshape(world, n, pr)
    out = np.empty((n, rows), parts.dtype)
    for r, (b, e) in enumerate(plan(rows, world, align)):
        out[:, b:e] = parts[r, :, : e - b]
    return out


class RowSharded:
    """A weight matrix split by output rows over the ranks of a process group.

    Every rank constructs it with the same host ``Tensor`` (or only its own
    slice via ``local=``) and calls ``matmul`` with the same activations; each
    call leaves the full result in ``out`` on every rank.
    """

    def __init__(self, dev: B200, tensor: Tensor | None, rank: int, world: int, align: int = 16, group=None,
                 local: Tensor | None = None, shape=None):
        import torch
        self.dev, self.rank, self.world, self.align, self.group = dev, rank, world, align, group
        self.rows, self.cols = tensor.shape if tensor is not None else shape
        self.begin, self.end = shard_rows(self.rows, rank, world, align)
        self.part_rows = part_rows(self.rows, world, align)
        mine = local if local is not None else tensor.slice_rows(self.begin, self.end)
        assert mine.shape == (self.end - self.begin, self.cols)
        self.weight = dev.upload(mine)
        self._torch = torch
        self._device = torch.device("cuda", torch.cuda.current_device())
        self._stream = torch.cuda.ExternalStream(dev.stream, device=self._device)
        self._parts = None      # torch tensor [world * n * part_rows], and its device views
        self._views = None
        self._short = None

    def _buffers(self, n: int):
        if self._parts is None or self._parts.numel() != self.world * n * self.part_rows:
            t = self._torch
            my_rows = self.end - self.begin
            # allocated and zeroed on the library's own stream, which is the one that writes them next
            with t.cuda.stream(self._stream):
                self._parts = t.zeros(self.world * n * self.part_rows, dtype=t.float32, device=self._device)
                # a short last shard computes into a buffer of its own and is padded into the common slice
                self._short = None if my_rows == self.part_rows else t.zeros(n * my_rows, dtype=t.float32, device=self._device)
            mine = self._parts[self.rank * n * self.part_rows:(self.rank + 1) * n * self.part_rows]
            local = self.dev.wrap((mine if self._short is None else self._short).data_ptr(), n * my_rows)
            self._views = (mine, local, self.dev.wrap(self._parts.data_ptr(), self._parts.numel()))
        return self._views

    def matmul(self, out, x) -> None:
        """out[t] = W . x[t] on every rank; ``out`` has n * rows floats."""
        import torch.distributed as dist
        n = len(x) // self.cols
        mine, local, parts = self._buffers(n)
        self.dev.matmul(local, self.weight, x)
        my_rows = self.end - self.begin
        with self._torch.cuda.stream(self._stream):
            if self._short is not None:
                mine.view(n, self.part_rows)[:, :my_rows] = self._short.view(n, my_rows)
            dist.all_gather_into_tensor(self._parts, mine, group=self.group)
        self.dev.touch(parts)               # written by the collective, not by the library
        self.dev.gather_rows(out, parts, n, self.rows, self.world, self.align)


class RowShardedPush:
    """The same split with the exchange fused into the product: every rank's
    kernel stores its rows of the token-major result into every rank's copy of a
    shared output from its epilogue (``B200.matmul_gather``: plain stores, over
    NVLink for the peers' copies), and one barrier kernel tells every rank that
    all slices have landed.  No collective library call, no re-assembly pass.

    ``matmul`` returns the device buffer that holds the full result on this
    rank.  Two buffers alternate: the result of a call stays valid until the
    call after the next."""

    def __init__(self, dev: B200, tensor: Tensor | None, rank: int, world: int, max_tokens: int, align: int = 16,
                 group=None, local: Tensor | None = None, shape=None):
        import torch.distributed as dist
        self.dev, self.rank, self.world, self.align = dev, rank, world, align
        self.rows, self.cols = tensor.shape if tensor is not None else shape
        self.begin, self.end = shard_rows(self.rows, rank, world, align)
        mine = local if local is not None else tensor.slice_rows(self.begin, self.end)
        assert mine.shape == (self.end - self.begin, self.cols)
        self.weight = dev.upload(mine)
        self.max_tokens = max_tokens
        self._outs, self._turn = [], 0
        for _ in range(2):
            buf, handle = dev.shared_alloc(max_tokens * self.rows)
            handles = [None] * world
            if world > 1:
                dist.all_gather_object(handles, handle, group=group)
            else:
                handles = [handle]
            dev.shared_connect(buf, world, rank, handles)
            self._outs.append(buf)
        if world > 1:
            dist.barrier(group=group)       # nobody stores before everybody has mapped

    def matmul(self, x):
        n = len(x) // self.cols
        if n > self.max_tokens:
            raise ValueError(f"{n} tokens, the shared outputs hold {self.max_tokens}")
        out = self._outs[self._turn]
        self._turn ^= 1
        self.dev.resize(out, n * self.rows)
        if self.end > self.begin:
            self.dev.matmul_gather(out, self.weight, x, self.begin, self.rows)
        self.dev.shared_barrier(out)
        return out


# ---- the feed-forward block, tensor parallel ------------------------------------------
#
#   out[t] = down . ( silu(gate . x[t]) * (up . x[t]) )
#
# (inference/qwen35/mod.rs:652-654: swiglu, then matmul_add with the down
# projection).  gate and up are split by output rows, down by the same indices
# along its K, so the intermediate of a rank is exactly the K slice its part
# of down multiplies and never leaves the GPU; the ranks' partial sums of
# ``out`` are added by one all-reduce (NCCL, or for a few tokens the library's own
# over peer memory, ``PeerReduce``).  The cuts fall on multiples of 256 rows:
# whole blocks of down's rows (the k-quant formats pack 256 weights of K).

FFN_ALIGN = 256


def ffn_cuts(inner: int, world: int):
    """[(begin, end)] of the intermediate dimension per rank, at multiples of 256."""
    return plan(inner, world, FFN_ALIGN)


def ffn_shard(gate: Tensor, up: Tensor, down: Tensor, rank: int, world: int):
    """Rank ``rank``'s parts (gate rows, up rows, down columns) of the block."""
    inner = gate.rows
    if up.shape != gate.shape or down.cols != inner or down.rows != gate.cols:
        raise ValueError(f"not a feed-forward block: gate {gate.shape}, up {up.shape}, down {down.shape}")
    b, e = ffn_cuts(inner, world)[rank]
    groups = range(b // FFN_ALIGN, e // FFN_ALIGN)
    return gate.slice_rows(b, e), up.slice_rows(b, e), down.select_column_groups(FFN_ALIGN, groups)


class PeerReduce:
    """The library's small all-reduce over peer memory (``B200.peer_allreduce``),
    set up for a process group: every rank creates its mailbox, the handles
    travel through ``torch.distributed`` (any backend), every rank maps its
    peers'.  One per device; vectors of up to ``cap`` floats."""

    def __init__(self, dev: B200, rank: int, world: int, cap: int, group=None):
        import torch.distributed as dist
        self.dev, self.cap = dev, cap
        mine = dev.peer_create(world, rank, cap)
        handles = [None] * world
        dist.all_gather_object(handles, mine, group=group)
        dev.peer_connect(handles)
        dist.barrier(group=group)          # nobody writes before everybody has mapped

    def __call__(self, buf, n: int) -> None:
        self.dev.peer_allreduce(buf, n)


class ShardedFFN:
    """The feed-forward block over the ranks of a process group (one process
    per GPU).  ``forward`` leaves the block's full output on every rank."""

    def __init__(self, dev: B200, gate: Tensor, up: Tensor, down: Tensor, rank: int = 0, world: int = 1, group=None,
                 peer: PeerReduce | None = None, exchange: str = "nccl"):
        """``exchange``: how the ranks' partial sums of the down projection are added.
        "push": the product's epilogue stores each partial sum into its row's owner
        (``B200.matmul_scatter``), the owners add and store the sums into every rank's
        copy of the result (``B200.reduce_gather``): no collective library call.
        "nccl": one all-reduce after the product (or ``peer``, the library's small
        all-reduce, for vectors it holds)."""
        import torch
        self.dev, self.rank, self.world, self.group = dev, rank, world, group
        self.exchange = exchange
        self.peer = peer                   # sums of up to peer.cap floats go through it instead of NCCL
        self.hidden, self.inner = gate.cols, gate.rows
        g, u, d = ffn_shard(gate, up, down, rank, world)
        self.my_inner = g.rows
        self.gate, self.up, self.down = dev.upload(g), dev.upload(u), dev.upload(d)
        self._torch = torch
        self._device = torch.device("cuda", torch.cuda.current_device())
        self._stream = torch.cuda.ExternalStream(dev.stream, device=self._device)

    # Activation buffers are shared by every block of the same shape on a device (a
    # decoder's layers use one residual stream, not one per layer): the all-reduce
    # then always sees the same buffer, which NCCL has set up once.
    _shared: dict = {}

    def _buffers(self, n: int):
        key = (id(self.dev), n, self.hidden, self.my_inner)
        bufs = ShardedFFN._shared.get(key)
        if bufs is None:
            t = self._torch
            with t.cuda.stream(self._stream):      # zeroed on the stream that writes it next
                out_t = t.zeros(n * self.hidden, dtype=t.float32, device=self._device)
            bufs = (out_t, self.dev.wrap(out_t.data_ptr(), n * self.hidden), self.dev.alloc(n * self.my_inner),
                    self.dev.alloc(n * self.my_inner))
            ShardedFFN._shared[key] = bufs
        self._out_t = bufs[0]
        return bufs

    _shared_push: dict = {}

    def _push_buffers(self, n: int):
        """The shared slots and result of the "push" exchange, one set per shape and
        device, created by every rank at the same point (their handles are exchanged)."""
        key = (id(self.dev), n, self.hidden, self.world)
        bufs = ShardedFFN._shared_push.get(key)
        if bufs is None:
            import torch.distributed as dist
            per = -(-self.hidden // self.world)
            made = []
            for length in (self.world * n * per, n * self.hidden):
                buf, handle = self.dev.shared_alloc(length)
                handles = [None] * self.world
                if self.world > 1:
                    dist.all_gather_object(handles, handle, group=self.group)
                else:
                    handles = [handle]
                self.dev.shared_connect(buf, self.world, self.rank, handles)
                made.append(buf)
            if self.world > 1:
                dist.barrier(group=self.group)
            bufs = (made[0], made[1], self.dev.alloc(n * max(self.my_inner, 1)), self.dev.alloc(n * max(self.my_inner, 1)))
            ShardedFFN._shared_push[key] = bufs
        return bufs

    def forward(self, x):
        """The block applied to ``x`` (n * hidden floats): returns the device
        buffer of n * hidden floats, valid until the next ``forward`` of any
        block of this shape on the device."""
        n = len(x) // self.hidden
        if self.exchange == "push":
            slots, out, h, scratch = self._push_buffers(n)
            if self.my_inner:
                self.dev.swiglu(h, self.gate, self.up, x, scratch)
                self.dev.matmul_scatter(slots, self.down, h)
            self.dev.shared_barrier(slots)
            self.dev.reduce_gather(out, slots, n, self.hidden)
            self.dev.shared_barrier(out)
            return out
        out_t, out, h, scratch = self._buffers(n)
        if self.my_inner:
            self.dev.swiglu(h, self.gate, self.up, x, scratch)
            self.dev.matmul(out, self.down, h)
        else:
            with self._torch.cuda.stream(self._stream):
                out_t.zero_()
        if self.world > 1:
            if self.peer is not None and n * self.hidden <= self.peer.cap:
                self.peer(out, n * self.hidden)
            else:
                import torch.distributed as dist
                with self._torch.cuda.stream(self._stream):
                    dist.all_reduce(out_t, group=self.group)
                self.dev.touch(out)         # written by the collective, not by the library
        return out
