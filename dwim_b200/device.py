"""``B200``: the engine's ``Device`` operator interface (gpu/mod.rs:176-401)
for the quantized matrix product, over the C ABI of ``libdwim_b200.so``.

Method names, argument order and meaning follow the trait: ``upload``,
``alloc``, ``resize``, ``read``, ``write``, ``matmul``, ``matmul_add``,
``swiglu``, ``name``, ``memory``, ``batch``.  Where the trait's methods panic
(a bad shape, a driver error) these raise ``DeviceError``.
"""
from __future__ import annotations

import ctypes as C
import weakref

import numpy as np

from . import _lib
from .tensor import Tensor, format_id, row_bytes


class DeviceError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{_lib.ERROR_NAMES.get(code, code)}: {message}")
        self.code = code


class Buffer:
    """A vector of f32 activations in device memory (``Device::Buffer``)."""

    def __init__(self, dev: "B200", handle: int):
        self._dev, self._h = dev, handle
        self._fin = weakref.finalize(self, dev._free_buffer, handle)

    def __len__(self) -> int:
        return int(self._dev._L.dwim_b200_buffer_len(self._h))

    @property
    def ptr(self) -> int:
        """Device address of the data."""
        return int(self._dev._L.dwim_b200_buffer_ptr(self._h) or 0)


class Weight:
    """A weight matrix in device memory (``Device::Weight``)."""

    def __init__(self, dev: "B200", handle: int, fmt: int, shape):
        self._dev, self._h, self.fmt, self.shape = dev, handle, fmt, tuple(shape)
        self._fin = weakref.finalize(self, dev._free_weight, handle)


class B200:
    def __init__(self, device: int = 0, stream: int | None = None):
        """Opens GPU ``device``.  ``stream``: a ``cudaStream_t`` (as an integer,
        e.g. ``torch.cuda.current_stream().cuda_stream``) to run on instead of a
        stream of the context's own; 0 is the legacy default stream."""
        self._L = _lib.lib()
        h = C.c_void_p()
        if stream is None:
            rc = self._L.dwim_b200_open(device, C.byref(h))
        else:
            rc = self._L.dwim_b200_open_on_stream(device, stream, C.byref(h))
        if rc != 0:
            raise DeviceError(rc, (self._L.dwim_b200_last_error(None) or b"").decode())
        self._ctx = h.value
        self._closed = False
        self._fin = weakref.finalize(self, self._L.dwim_b200_close, self._ctx)

    # -- plumbing ---------------------------------------------------------
    def _check(self, rc: int):
        if rc != 0:
            raise DeviceError(rc, (self._L.dwim_b200_last_error(self._ctx) or b"").decode())

    def _free_buffer(self, handle):
        if not self._closed:
            self._L.dwim_b200_buffer_free(self._ctx, handle)

    def _free_weight(self, handle):
        if not self._closed:
            self._L.dwim_b200_weight_free(self._ctx, handle)

    def close(self):
        if not self._closed:
            self._closed = True
            self._fin()

    # -- the trait ----------------------------------------------------------
    def name(self) -> str:
        buf = C.create_string_buffer(256)
        self._check(self._L.dwim_b200_name(self._ctx, buf, 256))
        return buf.value.decode()

    def memory(self) -> int:
        free = C.c_uint64()
        self._check(self._L.dwim_b200_memory(self._ctx, C.byref(free)))
        return free.value

    def batch(self) -> int:
        return int(self._L.dwim_b200_batch(self._ctx))

    def upload(self, tensor: Tensor) -> Weight:
        h = C.c_void_p()
        data = tensor.data
        self._check(self._L.dwim_b200_upload(self._ctx, tensor.fmt, tensor.rows, tensor.cols,
                                             data.ctypes.data, data.size, C.byref(h)))
        return Weight(self, h.value, tensor.fmt, tensor.shape)

    def alloc(self, length: int) -> Buffer:
        h = C.c_void_p()
        self._check(self._L.dwim_b200_alloc(self._ctx, length, C.byref(h)))
        return Buffer(self, h.value)

    def wrap(self, device_ptr: int, length: int) -> Buffer:
        """A buffer over device memory the caller owns (e.g. a torch tensor)."""
        h = C.c_void_p()
        self._check(self._L.dwim_b200_wrap(self._ctx, device_ptr, length, C.byref(h)))
        return Buffer(self, h.value)

    def touch(self, buf: Buffer) -> None:
        """Tells the library that someone else wrote ``buf`` (a kernel of the
        caller's, a collective): its cached operand form is dropped."""
        self._check(self._L.dwim_b200_touch(self._ctx, buf._h))

    def touch_bf16(self, buf: Buffer) -> None:
        """``touch`` by a writer that vouches every value it wrote is exactly a bf16."""
        self._check(self._L.dwim_b200_touch_bf16(self._ctx, buf._h))

    def activation_precision(self, mode: str) -> None:
        """``"exact"`` (the default: f32 activations as two f16 columns) or ``"f16"`` (one column, the
        precision of the reference's CUDA device: worst error 3e-3 instead of 2e-6, twice the rate) for
        products of more than eight tokens."""
        self._check(self._L.dwim_b200_activation_precision(self._ctx, {"exact": 0, "f16": 1}[mode]))

    def resize(self, buf: Buffer, length: int) -> None:
        self._check(self._L.dwim_b200_resize(self._ctx, buf._h, length))

    def read(self, buf: Buffer, out: np.ndarray | None = None) -> np.ndarray:
        n = len(buf)
        if out is None:
            out = np.empty(n, np.float32)
        assert out.dtype == np.float32 and out.size == n and out.flags.c_contiguous
        self._check(self._L.dwim_b200_read(self._ctx, buf._h, out.ctypes.data, n))
        return out

    def write(self, buf: Buffer, data) -> None:
        data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        self._check(self._L.dwim_b200_write(self._ctx, buf._h, data.ctypes.data, data.size))

    def write_bf16(self, buf: Buffer, bits) -> None:
        """Writes bf16 bit patterns (uint16); the buffer holds their f32 values."""
        bits = np.ascontiguousarray(bits, dtype=np.uint16).reshape(-1)
        self._check(self._L.dwim_b200_write_bf16(self._ctx, buf._h, bits.ctypes.data, bits.size))

    def buffer(self, data) -> Buffer:
        """alloc + write, as the reference tests' helper (gpu/tests.rs:142-146)."""
        data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        buf = self.alloc(data.size)
        self.write(buf, data)
        return buf

    def matmul(self, out: Buffer, w: Weight, x: Buffer) -> None:
        self._check(self._L.dwim_b200_matmul(self._ctx, out._h, w._h, x._h))

    def matmul_add(self, x: Buffer, w: Weight, input: Buffer, scratch: Buffer | None = None) -> None:
        self._check(self._L.dwim_b200_matmul_add(self._ctx, x._h, w._h, input._h, scratch._h if scratch else None))

    def swiglu(self, out: Buffer, gate: Weight, up: Weight, x: Buffer, scratch: Buffer) -> None:
        self._check(self._L.dwim_b200_swiglu(self._ctx, out._h, gate._h, up._h, x._h, scratch._h))

    def normalize(self, out: Buffer, x: Buffer, weight: Buffer, length: int, eps: float) -> None:
        """``Device::normalize``: ``out = rmsnorm(x[:length]) * weight``."""
        self._check(self._L.dwim_b200_normalize(self._ctx, out._h, x._h, weight._h, length, eps))

    def argmax(self, logits: Buffer, length: int) -> np.ndarray:
        """First index of the largest of every ``length`` logits (uint32 per row)."""
        n = len(logits) // length if length else 0
        out = np.zeros(n, np.uint32)
        self._check(self._L.dwim_b200_argmax(self._ctx, logits._h, length, out.ctypes.data_as(C.POINTER(C.c_uint32)), n))
        return out

    def matmul_static(self, out: Buffer, w: Weight, x: Buffer) -> None:
        """``matmul`` for up to 8 tokens that allocates nothing: the operand
        scratch is a fixed array inside the library, shared by every call on
        the GPU.  For callers that must not allocate device memory."""
        rows, cols = w.shape
        n = len(x) // cols
        if len(x) != n * cols or len(out) != n * rows:
            raise DeviceError(_lib.EINVAL, f"matmul_static: x of {len(x)} and out of {len(out)} floats for a [{rows}, {cols}] matrix")
        self._check(self._L.dwim_b200_matmul_static(self._ctx, out.ptr, w._h, x.ptr, n))

    # -- beside the trait -----------------------------------------------------
    def sync(self) -> None:
        self._check(self._L.dwim_b200_sync(self._ctx))

    def dequantize(self, w: Weight) -> np.ndarray:
        """``Tensor::dequantize`` (gpu/mod.rs:138-168), computed on the device."""
        out = np.empty(w.shape, np.float32)
        self._check(self._L.dwim_b200_dequantize(self._ctx, w._h, out.ctypes.data, out.size))
        return out

    def quantize(self, fmt, weights) -> Tensor:
        """Quantizes an f32 ``[rows, cols]`` matrix to GGUF blocks on the device."""
        fmt = format_id(fmt)
        weights = np.ascontiguousarray(weights, dtype=np.float32)
        rows, cols = weights.shape
        out = np.empty(rows * row_bytes(fmt, cols), np.uint8)
        self._check(self._L.dwim_b200_quantize(self._ctx, fmt, rows, cols, weights.ctypes.data,
                                               out.ctypes.data, out.size))
        return Tensor(fmt, (rows, cols), out)

    def gather_rows(self, out: Buffer, parts: Buffer, n: int, rows: int, world: int, align: int) -> None:
        self._check(self._L.dwim_b200_gather_rows(self._ctx, out._h, parts._h, n, rows, world, align))

    # -- a result shared by the ranks of a group (one process per GPU) -----------
    def shared_alloc(self, length: int):
        """This rank's copy of a buffer the group shares, and its inter-process
        handle (``bytes``), to be exchanged among the ranks."""
        nb = int(self._L.dwim_b200_peer_handle_bytes())
        h, hb = C.c_void_p(), C.create_string_buffer(nb)
        self._check(self._L.dwim_b200_shared_alloc(self._ctx, length, C.byref(h), hb, nb))
        return Buffer(self, h.value), hb.raw

    def shared_connect(self, buf: Buffer, world: int, rank: int, handles) -> None:
        """Maps the peers' copies of ``buf``; ``handles`` in rank order."""
        nb = int(self._L.dwim_b200_peer_handle_bytes())
        blob = b"".join(bytes(h)[:nb].ljust(nb, b"\0") for h in handles)
        self._check(self._L.dwim_b200_shared_connect(self._ctx, buf._h, world, rank, blob, nb))

    def shared_connect_local(self, buf: Buffer, world: int, rank: int, copies) -> None:
        """``shared_connect`` for ranks of one process: ``copies`` are the ranks' buffers in rank order."""
        arr = (C.c_void_p * world)(*[None if c is None else c._h for c in copies])
        self._check(self._L.dwim_b200_shared_connect_local(self._ctx, buf._h, world, rank, arr))

    def matmul_gather(self, out: Buffer, w: Weight, x: Buffer, row_begin: int, total_rows: int) -> None:
        """The row-sharded product, its rows stored into every rank's copy of ``out``."""
        self._check(self._L.dwim_b200_matmul_gather(self._ctx, out._h, w._h, x._h, row_begin, total_rows))

    def shared_barrier(self, buf: Buffer) -> None:
        self._check(self._L.dwim_b200_shared_barrier(self._ctx, buf._h))

    def matmul_scatter(self, slots: Buffer, w: Weight, x: Buffer) -> None:
        """The K-sharded product, every partial sum stored into its row's owner's slot."""
        self._check(self._L.dwim_b200_matmul_scatter(self._ctx, slots._h, w._h, x._h))

    def reduce_gather(self, out: Buffer, slots: Buffer, n: int, rows: int) -> None:
        """This rank's rows summed over the slots, the sums stored into every rank's copy of ``out``."""
        self._check(self._L.dwim_b200_reduce_gather(self._ctx, out._h, slots._h, n, rows))

    # -- the small all-reduce over peer memory (one process per GPU) ------------
    def peer_create(self, world: int, rank: int, cap: int) -> bytes:
        """Allocates this rank's mailbox for vectors of up to ``cap`` floats;
        returns its inter-process handle, to be exchanged among the ranks."""
        nb = int(self._L.dwim_b200_peer_handle_bytes())
        h = C.create_string_buffer(nb)
        self._check(self._L.dwim_b200_peer_create(self._ctx, world, rank, cap, h, nb))
        return h.raw

    def peer_connect(self, handles) -> None:
        """Maps the ranks' mailboxes; ``handles`` in rank order."""
        nb = int(self._L.dwim_b200_peer_handle_bytes())
        blob = b"".join(bytes(h)[:nb].ljust(nb, b"\0") for h in handles)
        self._check(self._L.dwim_b200_peer_connect(self._ctx, blob, nb))

    def peer_allreduce(self, buf: Buffer, n: int | None = None) -> None:
        """The first ``n`` floats of ``buf`` become their sum over the ranks."""
        self._check(self._L.dwim_b200_peer_allreduce(self._ctx, buf._h, len(buf) if n is None else n))

    @property
    def stream(self) -> int:
        return int(self._L.dwim_b200_stream(self._ctx) or 0)

    @property
    def launches(self) -> int:
        return int(self._L.dwim_b200_launches(self._ctx))

    def timer_begin(self) -> None:
        self._check(self._L.dwim_b200_timer_begin(self._ctx))

    def timer_end(self) -> float:
        ms = C.c_float()
        self._check(self._L.dwim_b200_timer_end(self._ctx, C.byref(ms)))
        return ms.value


def shard_rows(rows: int, rank: int, world: int, align: int = 16):
    """Rows [begin, end) of rank ``rank`` when a matrix is split by output rows."""
    b, e = C.c_size_t(), C.c_size_t()
    rc = _lib.lib().dwim_b200_shard_rows(rows, rank, world, align, C.byref(b), C.byref(e))
    if rc != 0:
        raise DeviceError(rc, "bad shard arguments")
    return b.value, e.value
