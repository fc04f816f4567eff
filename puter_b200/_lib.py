"""ctypes loader for libputer_b200.so (the C ABI declared in include/puter_b200.h).

Loading fails loudly: there is no Python or CPU fallback behind these entry points.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libputer_b200.so")

STATUS_BYTES = 1024


class CUDAStatus(ctypes.Structure):
    _fields_ = [("code", ctypes.c_int), ("message", ctypes.c_char * STATUS_BYTES)]


vp, u32, u64, i64, cint, dbl, flt = (ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int64, ctypes.c_int,
                                     ctypes.c_double, ctypes.c_float)
SP = ctypes.POINTER(CUDAStatus)

_GATED = ["swiglu", "geglu", "glu", "reglu", "siglu", "geglu_tanh", "seglu", "linglu"]

# name -> (restype, argtypes); mirrors include/puter_b200.h one to one
SIGNATURES = {
    "cuda_status_clear": (None, [SP]),
    "cuda_status_set": (None, [SP, cint, ctypes.c_char_p]),
    "cuda_open_device": (cint, [ctypes.POINTER(vp), SP]),
    "cuda_open_device_index": (cint, [cint, ctypes.POINTER(vp), SP]),
    "cuda_close_device": (None, [vp]),
    "cuda_device_total_memory": (ctypes.c_longlong, [vp]),
    "cuda_device_capability_major": (cint, [vp]),
    "cuda_buffer_alloc": (vp, [vp, ctypes.c_longlong]),
    "cuda_buffer_release": (None, [vp]),
    "cuda_buffer_device_ptr": (vp, [vp]),
    "cuda_buffer_wrap": (vp, [vp, vp, ctypes.c_longlong]),
    "cuda_buffer_ipc_export": (cint, [vp, ctypes.c_char_p, SP]),
    "cuda_buffer_ipc_import": (vp, [vp, ctypes.c_char_p, ctypes.c_longlong, SP]),
    "cuda_memcpy_async_h2d": (cint, [vp, vp, ctypes.c_longlong, vp, SP]),
    "cuda_memcpy_async_d2h": (cint, [vp, vp, ctypes.c_longlong, vp, SP]),
    "cuda_memcpy_async_d2d": (cint, [vp, vp, ctypes.c_longlong, vp, SP]),
    "cuda_stream_synchronize": (cint, [vp, SP]),
    "cuda_default_context": (vp, []),
    "cuda_context_upload_stream": (vp, [vp]),
    "cuda_context_default_stream": (vp, [vp]),
    "cuda_context_set_stream": (cint, [vp, vp, SP]),
    "cuda_context_reset_stream": (cint, [vp, SP]),
    "cuda_context_set_exact": (cint, [vp, cint, SP]),
    "cuda_context_take_error": (cint, [vp, ctypes.POINTER(cint), SP]),
    "cuda_context_launch_count": (ctypes.c_ulonglong, [vp]),
    "cuda_host_alloc": (vp, [ctypes.c_longlong]),
    "cuda_host_free": (None, [vp]),
    "cuda_dispatch_convert": (cint, [vp, cint, cint, vp, vp, u64, u64, SP]),
    "cuda_convert_host": (cint, [vp, cint, cint, vp, u64, vp, u64, SP]),
    "cuda_dispatch_unary_elementwise": (cint, [vp, cint, cint, vp, vp, u32, u64, SP]),
    "cuda_dispatch_binary_elementwise": (cint, [vp, cint, cint, vp, vp, vp, u32, u64, SP]),
    "cuda_dispatch_gated_residual": (cint, [vp, cint, vp, vp, vp, vp, u32, u32, u32, u32, u32, u64, SP]),
    "cuda_dispatch_rmsnorm": (cint, [vp, cint, vp, vp, vp, u32, u32, flt, u64, SP]),
    "cuda_dispatch_layernorm": (cint, [vp, cint, vp, vp, vp, vp, u32, u32, flt, u64, SP]),
    "cuda_dispatch_layernorm_residual": (cint, [vp, cint, vp, vp, vp, vp, vp, u32, u32, flt, u64, SP]),
    "cuda_dispatch_softmax": (cint, [vp, cint, vp, vp, u32, u32, u64, SP]),
    "cuda_dispatch_log_softmax": (cint, [vp, cint, vp, vp, u32, u32, u64, SP]),
    "cuda_dispatch_last_token": (cint, [vp, cint, vp, vp, u32, u32, u32, u64, SP]),
    "cuda_dispatch_adaptive_rmsnorm": (cint, [vp, cint, vp, vp, vp, u32, u32, u32, u32, dbl, u64, SP]),
    "cuda_dispatch_modulated_layernorm": (cint, [vp, cint, vp, vp, vp, u32, u32, u32, u32, u32, dbl, u64, SP]),
    "cuda_dispatch_rmsnorm_f64": (cint, [vp, cint, vp, vp, vp, u32, u32, dbl, u64, SP]),
    "cuda_dispatch_add_rmsnorm_gated_residual": (cint, [vp, cint, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, dbl, u32, u32, u32, u64, SP]),
    "cuda_dispatch_add_rmsnorm_gated_residual_gather": (cint, [vp, cint, vp, vp, vp, vp, vp, ctypes.POINTER(vp), ctypes.POINTER(vp), u32, u32, u32,
                                                               u32, dbl, u32, u32, u32, u64, SP]),
    "cuda_dispatch_swiglu_gather": (cint, [vp, cint, ctypes.POINTER(vp), u32, u32, vp, vp, u32, u64, SP]),
    "cuda_dispatch_rope": (cint, [vp, cint, vp, vp, u32, u32, u32, u32, flt, flt, flt, flt, u32, u32, u32, u64, SP]),
    "cuda_dispatch_rope_f64": (cint, [vp, cint, vp, vp, u32, u32, u32, dbl, i64, u32, u32, dbl, dbl, dbl, u32, u64, SP]),
    "cuda_dispatch_rope_pairs": (cint, [vp, cint, vp, vp, vp, vp, u32, u64, SP]),
    "cuda_dispatch_kv_page_write": (cint, [vp, cint, vp, vp, vp, vp, vp, u32, u32, u32, u32, u64, u64, SP]),
    "cuda_dispatch_kv_page_gather": (cint, [vp, cint, vp, vp, vp, u32, u32, u32, u32, u64, u64, SP]),
    "cuda_dispatch_rope_kv_page_write": (cint, [vp, cint, cint, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, dbl, u32, u32,
                                                dbl, dbl, dbl, u32, u64, SP]),
    "cuda_dispatch_multi_head_attention": (cint, [vp, cint, cint, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, u64, SP]),
    "cuda_dispatch_flash_attention": (cint, [vp, cint, vp, vp, vp, vp, u32, u32, u32, u32, u64, SP]),
    "cuda_dispatch_flash_attention_causal": (cint, [vp, cint, vp, vp, vp, vp, u32, u32, u32, u32, u32, u64, SP]),
    "cuda_dispatch_rope_attention_prefill": (cint, [vp, cint, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, dbl, i64, u32, dbl, dbl,
                                                    dbl, u32, u64, SP]),
    "cuda_dispatch_paged_decode_attention": (cint, [vp, cint, cint, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32,
                                                    u32, u64, SP]),
}
SIGNATURES["cuda_dispatch_paged_decode_attention_noalloc"] = SIGNATURES["cuda_dispatch_paged_decode_attention"]
for _g in _GATED:
    SIGNATURES[f"cuda_dispatch_{_g}"] = (cint, [vp, cint, vp, vp, vp, u32, u64, SP])
    SIGNATURES[f"cuda_dispatch_{_g}_packed"] = (cint, [vp, cint, vp, vp, u32, u32, u64, SP])

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library and binds every declared entry point; raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m puter_b200.csrc.build` (there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
