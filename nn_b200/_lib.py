"""ctypes binding of libnnq_b200.so (the C ABI declared in include/nnq.h).

The library is the product; there is no fallback. If the shared object is missing and
cannot be built, or a GPU call is made without a usable device, this raises.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

_lib = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_int64 = ctypes.c_int64
c_size_t = ctypes.c_size_t

# symbol -> (restype, argtypes); kept in step with include/nnq.h (tests/test_abi.py checks it)
SIGNATURES = {
    "nnq_version": (c_int, []),
    "nnq_status_str": (ctypes.c_char_p, [c_int]),
    "nnq_format_geometry": (c_int, [c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int)]),
    "nnq_init": (c_int, [c_int, ctypes.POINTER(c_void_p)]),
    "nnq_destroy": (None, [c_void_p]),
    "nnq_last_error": (ctypes.c_char_p, [c_void_p]),
    "nnq_set_path": (c_int, [c_void_p, c_int]),
    "nnq_device_status": (c_int, [c_void_p, c_void_p]),
    "nnq_weight_create": (c_int, [c_void_p, c_int, c_void_p, c_size_t, c_void_p, c_size_t, c_int64, c_int64,
                                  ctypes.POINTER(c_void_p)]),
    "nnq_weight_create_shard": (c_int, [c_void_p, c_int, c_void_p, c_size_t, c_void_p, c_size_t, c_int64, c_int64,
                                        c_int, c_int, c_int, ctypes.POINTER(c_void_p)]),
    "nnq_weight_destroy": (None, [c_void_p]),
    "nnq_weight_info": (c_int, [c_void_p, ctypes.POINTER(c_int), ctypes.POINTER(c_int64), ctypes.POINTER(c_int64),
                                ctypes.POINTER(c_size_t), ctypes.POINTER(c_size_t)]),
    "nnq_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "nnq_dequantize_raw": (c_int, [c_void_p, c_int, c_void_p, c_size_t, c_void_p, c_size_t, c_int64, c_void_p,
                                   ctypes.POINTER(c_int64), c_void_p]),
    "nnq_quantize": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_size_t, c_void_p, c_size_t,
                             ctypes.POINTER(c_int64), c_void_p]),
    "nnq_int8_quantize_per_channel": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nnq_int8_dequantize_per_channel": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "nnq_int8_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int, c_int64, c_void_p,
                                c_void_p, c_int, c_void_p]),
    "nnq_group_quantize": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nnq_group_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64, c_void_p, c_void_p]),
    "nnq_gq_create_per_group": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64, c_void_p,
                                        ctypes.POINTER(c_void_p)]),
    "nnq_gq_create_gptq": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p,
                                   ctypes.POINTER(c_void_p)]),
    "nnq_gq_info": (c_int, [c_void_p, ctypes.POINTER(c_int64), ctypes.POINTER(c_int64), ctypes.POINTER(c_int),
                            ctypes.POINTER(c_int64), ctypes.POINTER(c_int64), ctypes.POINTER(c_int)]),
    "nnq_gq_dequantize": (c_int, [c_void_p, c_void_p, c_void_p]),
    "nnq_gq_linear": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p]),
    "nnq_gq_destroy": (None, [c_void_p]),
    "nnq_gptq_unpack_qweight": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "nnq_gptq_unpack_qzeros": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "nnq_gptq_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "nnq_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p]),
    "nnq_linear_host": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int]),
    "nnq_linear_batch": (c_int, [c_void_p, c_int, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int, c_int64,
                                 ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int, c_void_p]),
    "nnq_linear_batch_host": (c_int, [c_void_p, c_int, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int, c_int64,
                                      ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int]),
    "nnq_launch_count": (c_int64, [c_void_p]),
    "nnq_comm_create": (c_int, [c_void_p, c_int, c_int, c_size_t, ctypes.POINTER(c_void_p)]),
    "nnq_comm_get_handle": (c_int, [c_void_p, c_void_p]),
    "nnq_comm_open_peers": (c_int, [c_void_p, c_void_p]),
    "nnq_comm_all_reduce": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p]),
    "nnq_comm_set_spin_limit": (c_int, [c_void_p, ctypes.c_uint]),
    "nnq_comm_local_buffer": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "nnq_comm_open_local_peers": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "nnq_comm_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p]),
    "nnq_comm_destroy": (None, [c_void_p]),
    "nnq_decoder_create": (c_int, [c_void_p, c_void_p, ctypes.POINTER(c_void_p)]),
    "nnq_decoder_set_layer": (c_int, [c_void_p, c_int] + [c_void_p] * 11),
    "nnq_decoder_set_head": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "nnq_decoder_set_comm": (c_int, [c_void_p, c_void_p]),
    "nnq_decoder_reset": (c_int, [c_void_p, c_int, c_int, c_void_p]),
    "nnq_decoder_step": (c_int, [c_void_p, c_void_p]),
    "nnq_decoder_prefill": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "nnq_decoder_state": (c_int, [c_void_p, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int), c_void_p]),
    "nnq_decoder_buffers": (c_int, [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p),
                                    ctypes.POINTER(c_void_p)]),
    "nnq_decoder_destroy": (None, [c_void_p]),
    "nnq_plan_create": (c_int, [c_void_p, c_int, c_int, c_int, ctypes.POINTER(c_void_p)]),
    "nnq_plan_add": (c_int, [c_void_p, c_int, ctypes.POINTER(c_void_p), c_void_p, ctypes.POINTER(c_void_p),
                             ctypes.POINTER(c_void_p)]),
    "nnq_plan_add_reduced": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nnq_plan_finalize": (c_int, [c_void_p]),
    "nnq_plan_run": (c_int, [c_void_p, c_void_p]),
    "nnq_plan_reset": (c_int, [c_void_p, c_void_p]),
    "nnq_plan_set_spin_limit": (c_int, [c_void_p, ctypes.c_uint]),
    "nnq_plan_info": (c_int, [c_void_p, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int),
                              ctypes.POINTER(c_size_t), ctypes.POINTER(c_size_t)]),
    "nnq_plan_dependency": (c_int, [c_void_p, c_int, ctypes.POINTER(c_int)]),
    "nnq_plan_geometry": (c_int, [c_int, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int)]),
    "nnq_plan_destroy": (None, [c_void_p]),
    "nnq_moe_create": (c_int, [c_void_p, c_int, c_int, c_int, c_int, ctypes.c_float, c_void_p, c_void_p, c_int, c_int,
                               c_void_p, c_size_t, c_void_p, c_size_t, c_void_p, c_void_p, c_size_t, c_void_p,
                               c_size_t, c_void_p, ctypes.POINTER(c_void_p)]),
    "nnq_moe_create_shard": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, ctypes.c_float, c_void_p,
                                     c_void_p, c_int, c_int, c_void_p, c_size_t, c_void_p, c_size_t, c_void_p,
                                     c_void_p, c_size_t, c_void_p, c_size_t, c_void_p, ctypes.POINTER(c_void_p)]),
    "nnq_moe_destroy": (None, [c_void_p]),
    "nnq_moe_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    "nnq_moe_forward_static": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    "nnq_moe_forward_routed": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nnq_moe_gather_rows": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "nnq_moe_combine_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "nnq_moe_route": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
}


def path() -> str:
    return _build.LIB


def load():
    """Load (building first if the sources are newer) and type the C ABI."""
    global _lib
    if _lib is not None:
        return _lib
    if _build.stale():
        _build.build()
    if not os.path.exists(_build.LIB):
        raise RuntimeError(f"{_build.LIB} is missing and could not be built")
    lib = ctypes.CDLL(_build.LIB)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
