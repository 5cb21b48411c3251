"""Loads ``libdwim_b200.so`` and declares the C ABI of ``include/dwim_b200.h``.

There is no fallback: if the library has not been built, importing a symbol
from here raises, and nothing in the package computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libdwim_b200.so"

Q8_0, Q4_K, Q6_K, BF16 = 8, 12, 14, 30

OK, EINVAL, EFORMAT, ENOMEM, ECUDA, ENODEV, ETIMEOUT = 0, -1, -2, -3, -4, -5, -6
ERROR_NAMES = {EINVAL: "EINVAL", EFORMAT: "EFORMAT", ENOMEM: "ENOMEM", ECUDA: "ECUDA", ENODEV: "ENODEV",
               ETIMEOUT: "ETIMEOUT"}

_vp, _sz = C.c_void_p, C.c_size_t
_f32p, _u16p = C.POINTER(C.c_float), C.POINTER(C.c_uint16)

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "dwim_b200_open": (C.c_int, [C.c_int, C.POINTER(_vp)]),
    "dwim_b200_open_on_stream": (C.c_int, [C.c_int, _vp, C.POINTER(_vp)]),
    "dwim_b200_close": (C.c_int, [_vp]),
    "dwim_b200_last_error": (C.c_char_p, [_vp]),
    "dwim_b200_name": (C.c_int, [_vp, C.c_char_p, _sz]),
    "dwim_b200_memory": (C.c_int, [_vp, C.POINTER(C.c_uint64)]),
    "dwim_b200_batch": (_sz, [_vp]),
    "dwim_b200_sync": (C.c_int, [_vp]),
    "dwim_b200_stream": (_vp, [_vp]),
    "dwim_b200_status": (C.c_int, [_vp, C.POINTER(C.c_uint32)]),
    "dwim_b200_launches": (C.c_uint64, [_vp]),
    "dwim_b200_timer_begin": (C.c_int, [_vp]),
    "dwim_b200_timer_end": (C.c_int, [_vp, _f32p]),
    "dwim_b200_alloc": (C.c_int, [_vp, _sz, C.POINTER(_vp)]),
    "dwim_b200_wrap": (C.c_int, [_vp, _vp, _sz, C.POINTER(_vp)]),
    "dwim_b200_resize": (C.c_int, [_vp, _vp, _sz]),
    "dwim_b200_touch": (C.c_int, [_vp, _vp]),
    "dwim_b200_touch_bf16": (C.c_int, [_vp, _vp]),
    "dwim_b200_activation_precision": (C.c_int, [_vp, C.c_int]),
    "dwim_b200_write": (C.c_int, [_vp, _vp, _vp, _sz]),
    "dwim_b200_write_bf16": (C.c_int, [_vp, _vp, _vp, _sz]),
    "dwim_b200_read": (C.c_int, [_vp, _vp, _vp, _sz]),
    "dwim_b200_buffer_free": (C.c_int, [_vp, _vp]),
    "dwim_b200_buffer_len": (_sz, [_vp]),
    "dwim_b200_buffer_ptr": (_vp, [_vp]),
    "dwim_b200_row_bytes": (_sz, [C.c_int, _sz]),
    "dwim_b200_upload": (C.c_int, [_vp, C.c_int, _sz, _sz, _vp, _sz, C.POINTER(_vp)]),
    "dwim_b200_weight_free": (C.c_int, [_vp, _vp]),
    "dwim_b200_weight_shape": (C.c_int, [_vp, C.POINTER(C.c_int), C.POINTER(_sz), C.POINTER(_sz)]),
    "dwim_b200_dequantize": (C.c_int, [_vp, _vp, _vp, _sz]),
    "dwim_b200_quantize": (C.c_int, [_vp, C.c_int, _sz, _sz, _vp, _vp, _sz]),
    "dwim_b200_matmul": (C.c_int, [_vp, _vp, _vp, _vp]),
    "dwim_b200_matmul_add": (C.c_int, [_vp, _vp, _vp, _vp, _vp]),
    "dwim_b200_swiglu": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "dwim_b200_normalize": (C.c_int, [_vp, _vp, _vp, _vp, _sz, C.c_float]),
    "dwim_b200_argmax": (C.c_int, [_vp, _vp, _sz, C.POINTER(C.c_uint32), _sz]),
    "dwim_b200_matmul_static": (C.c_int, [_vp, _vp, _vp, _vp, _sz]),
    "dwim_b200_shared_alloc": (C.c_int, [_vp, _sz, C.POINTER(_vp), _vp, _sz]),
    "dwim_b200_shared_connect_local": (C.c_int, [_vp, _vp, C.c_int, C.c_int, _vp]),
    "dwim_b200_shared_connect": (C.c_int, [_vp, _vp, C.c_int, C.c_int, _vp, _sz]),
    "dwim_b200_matmul_gather": (C.c_int, [_vp, _vp, _vp, _vp, _sz, _sz]),
    "dwim_b200_shared_barrier": (C.c_int, [_vp, _vp]),
    "dwim_b200_matmul_scatter": (C.c_int, [_vp, _vp, _vp, _vp]),
    "dwim_b200_reduce_gather": (C.c_int, [_vp, _vp, _vp, _sz, _sz]),
    "dwim_b200_shard_rows": (C.c_int, [_sz, C.c_int, C.c_int, _sz, C.POINTER(_sz), C.POINTER(_sz)]),
    "dwim_b200_gather_rows": (C.c_int, [_vp, _vp, _vp, _sz, _sz, C.c_int, _sz]),
    "dwim_b200_peer_handle_bytes": (_sz, []),
    "dwim_b200_peer_create": (C.c_int, [_vp, C.c_int, C.c_int, _sz, _vp, _sz]),
    "dwim_b200_peer_connect": (C.c_int, [_vp, _vp, _sz]),
    "dwim_b200_peer_allreduce": (C.c_int, [_vp, _vp, _sz]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dwim_b200.build` "
                "(there is no CPU fallback)")
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)   # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib
