"""dwim_b200: the dwim engine's block-quantized matrix product (GGUF Q4_K,
Q6_K, Q8_0 weights x f32/bf16 activations), hand-written for NVIDIA B200.

``B200`` mirrors the engine's ``Device`` trait for this path; ``Tensor`` is the
host-side weight container.  The arithmetic lives in ``libdwim_b200.so``
(CUDA, sm_100a), built in place by ``python -m dwim_b200.build``.
"""
from ._lib import Q4_K, Q6_K, Q8_0
from .device import B200, Buffer, DeviceError, Weight, shard_rows
from .tensor import Tensor, format_id, row_bytes

__all__ = ["B200", "Buffer", "DeviceError", "Weight", "Tensor", "Q4_K", "Q6_K", "Q8_0", "format_id", "row_bytes",
           "shard_rows"]
