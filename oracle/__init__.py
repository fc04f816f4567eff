"""CPU oracle for the puter hot path — TEST INFRASTRUCTURE, not product code.

A ctypes front end over ``libputer_oracle.so`` (built from ``puter_oracle.cpp``,
a C++ restatement of the scalar Go code of puter's ``device/cpu`` backend and
``convert`` package).  Only the tests, the smoke check and the ``cpu_baseline`` /
``--impl reference`` legs of the benchmark may import this package; the shipped
library never does.

Arrays are numpy; 16-bit and 8-bit float formats travel as raw ``uint16`` /
``uint8`` bit patterns so that comparisons are bit-exact.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libputer_oracle.so")

# dtype codes = CUDAElementDType (device/cuda/internal/bridge/core.h:26-33)
F32, F16, BF16, F64, E4M3, E5M2 = 0, 1, 2, 3, 4, 5
_NP = {F32: np.float32, F16: np.uint16, BF16: np.uint16, E4M3: np.uint8, E5M2: np.uint8}

# unary op codes = CUDAUnaryFloat32Op (core.h:35-70); gated variants in oracle order
RELU, TANH, SIGMOID, SILU, GELU, GELU_TANH = 0, 12, 13, 14, 22, 29
UNARY_CODES = {"Relu": 0, "Exp": 8, "Log": 9, "Tanh": 12, "Sigmoid": 13, "Silu": 14, "Swish": 15, "Softsign": 16, "ELU": 17, "SELU": 18,
               "LeakyReLU": 19, "HardSigmoid": 20, "HardSwish": 21, "Gelu": 22, "Log1p": 23, "Expm1": 24, "CELU": 25, "Softplus": 26,
               "Mish": 27, "LogSigmoid": 28, "GeluTanh": 29, "HardTanh": 30, "HardGelu": 31, "QuickGelu": 32, "TanhShrink": 33}
SWIGLU, GEGLU, GLU, REGLU, SIGLU, GEGLU_TANH, SEGLU, LINGLU = 0, 1, 2, 3, 4, 5, 6, 7
ADD, SUB, MUL, DIV, MAX, MIN = 0, 1, 2, 3, 4, 5


def build(force: bool = False) -> str:
    """Compile the oracle library in place (g++, a few seconds)."""
    src = os.path.join(_HERE, "puter_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libputer_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_fast_exp32.restype = ctypes.c_float
        _lib.oracle_fast_exp32.argtypes = [ctypes.c_float]
        _lib.oracle_fast_tanh32.restype = ctypes.c_float
        _lib.oracle_fast_tanh32.argtypes = [ctypes.c_float]
        _lib.oracle_fast_silu32.restype = ctypes.c_float
        _lib.oracle_fast_silu32.argtypes = [ctypes.c_float]
        _lib.oracle_fast_exp64.restype = ctypes.c_double
        _lib.oracle_fast_exp64.argtypes = [ctypes.c_double]
    return _lib


def set_threads(n: int) -> None:
    lib().oracle_set_threads(ctypes.c_int(n))


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def _ll(x):
    return ctypes.c_longlong(int(x))


def _check(rc: int, what: str):
    if rc != 0:
        raise ValueError(f"oracle {what}: status {rc}")


def np_dtype(dt: int):
    return _NP[dt]


def convert(src: np.ndarray, src_dt: int, dst_dt: int) -> np.ndarray:
    """convert package (convert/bf16_f32.go, f16_f32.go, fp8_f32.go)."""
    src = np.ascontiguousarray(src, dtype=_NP[src_dt])
    dst = np.empty(src.shape, dtype=_NP[dst_dt])
    _check(lib().oracle_convert(src_dt, dst_dt, _p(src), _p(dst), _ll(src.size)), "convert")
    return dst


def to_f32(a: np.ndarray, dt: int) -> np.ndarray:
    return a.astype(np.float32) if dt == F32 else convert(a, dt, F32)


def from_f32(a: np.ndarray, dt: int) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a.copy() if dt == F32 else convert(a, F32, dt)


def unary(op: int, dt: int, src: np.ndarray) -> np.ndarray:
    src = np.ascontiguousarray(src, dtype=_NP[dt])
    dst = np.empty_like(src)
    _check(lib().oracle_unary(op, dt, _p(src), _p(dst), _ll(src.size)), "unary")
    return dst


def softmax_rows(dt: int, x: np.ndarray, log: bool = False) -> np.ndarray:
    """device.Activation.Softmax / LogSoftmax applied to every row of a [rows, cols] array."""
    x = np.ascontiguousarray(x, dtype=_NP[dt])
    rows, cols = x.shape
    out = np.empty_like(x)
    _check(lib().oracle_softmax_rows(dt, _p(x), _p(out), _ll(rows), _ll(cols), ctypes.c_int(int(log))), "softmax_rows")
    return out


def last_token(x: np.ndarray, batch: int, seq: int, hidden: int) -> np.ndarray:
    """device.Shape.LastToken on a [batch, seq, hidden] array of any element type."""
    x = np.ascontiguousarray(x)
    out = np.empty((batch, hidden), dtype=x.dtype)
    _check(lib().oracle_last_token(_p(x), _p(out), _ll(batch), _ll(seq), _ll(hidden * x.dtype.itemsize)), "last_token")
    return out


def gated_tensors(op: int, dt: int, gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate = np.ascontiguousarray(gate, dtype=_NP[dt])
    up = np.ascontiguousarray(up, dtype=_NP[dt])
    dst = np.empty_like(gate)
    _check(lib().oracle_gated_tensors(op, dt, _p(dst), _p(gate), _p(up), _ll(gate.size)), "gated_tensors")
    return dst


def gated_packed(op: int, dt: int, packed: np.ndarray, batch: int, half: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=_NP[dt])
    dst = np.empty(batch * half, dtype=_NP[dt])
    _check(lib().oracle_gated_packed(op, dt, _p(dst), _p(packed), _ll(batch), _ll(half)), "gated_packed")
    return dst.reshape(batch, half)


def binary(op: int, dt: int, left: np.ndarray, right: np.ndarray) -> np.ndarray:
    left = np.ascontiguousarray(left, dtype=_NP[dt])
    right = np.ascontiguousarray(right, dtype=_NP[dt])
    dst = np.empty_like(left)
    _check(lib().oracle_binary(op, dt, _p(left), _p(right), _p(dst), _ll(left.size)), "binary")
    return dst


def rmsnorm(dt: int, x: np.ndarray, scale: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=_NP[dt])
    scale = np.ascontiguousarray(scale, dtype=_NP[dt])
    rows, cols = x.shape
    out = np.empty_like(x)
    _check(lib().oracle_rmsnorm(dt, _p(x), _p(scale), _p(out), _ll(rows), _ll(cols), ctypes.c_double(eps)), "rmsnorm")
    return out


def layernorm(dt: int, x: np.ndarray, scale: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """device.LayerNorm.LayerNorm (epsilon fixed at 1e-5 by the reference)."""
    x = np.ascontiguousarray(x, dtype=_NP[dt])
    scale = np.ascontiguousarray(scale, dtype=_NP[dt])
    bias = np.ascontiguousarray(bias, dtype=_NP[dt])
    rows, cols = x.shape
    out = np.empty_like(x)
    _check(lib().oracle_layernorm(dt, _p(x), _p(scale), _p(bias), _p(out), _ll(rows), _ll(cols)), "layernorm")
    return out


def adaptive_rmsnorm(dt: int, x: np.ndarray, modulation: np.ndarray, rows_per_batch: int, mod_cols: int, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=_NP[dt])
    modulation = np.ascontiguousarray(modulation, dtype=_NP[dt])
    rows, cols = x.shape
    out = np.empty_like(x)
    _check(lib().oracle_adaptive_rmsnorm(dt, _p(x), _p(modulation), _p(out), _ll(rows), _ll(cols), _ll(rows_per_batch), _ll(mod_cols),
                                         ctypes.c_double(eps)), "adaptive_rmsnorm")
    return out


def modulated_layernorm(dt: int, x: np.ndarray, modulation: np.ndarray, rows_per_batch: int, mod_cols: int, eps: float,
                        set_index: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=_NP[dt])
    modulation = np.ascontiguousarray(modulation, dtype=_NP[dt])
    rows, cols = x.shape
    out = np.empty_like(x)
    _check(lib().oracle_modulated_layernorm(dt, _p(x), _p(modulation), _p(out), _ll(rows), _ll(cols), _ll(rows_per_batch), _ll(mod_cols),
                                            ctypes.c_double(eps), _ll(set_index)), "modulated_layernorm")
    return out


def gated_residual(dt, residual, branch, modulation, rows, last_dim, rows_per_batch, mod_cols, set_index):
    residual = np.ascontiguousarray(residual, dtype=_NP[dt])
    branch = np.ascontiguousarray(branch, dtype=_NP[dt])
    modulation = np.ascontiguousarray(modulation, dtype=_NP[dt])
    out = np.empty_like(residual)
    _check(
        lib().oracle_gated_residual(dt, _p(residual), _p(branch), _p(modulation), _p(out), _ll(rows), _ll(last_dim),
                                    _ll(rows_per_batch), _ll(mod_cols), _ll(set_index)),
        "gated_residual",
    )
    return out


def rope(dt, x, seq_len, num_heads, head_dim, base=10000.0, start=0, mode=0, scaling=0, factor=1.0, low=0.0,
         high=0.0, orig_ctx=0):
    """device.RoPE.RoPE; x is [seq, heads, head_dim]; mode 0 interleaved / 1 half; scaling 1 = llama3."""
    x = np.ascontiguousarray(x, dtype=_NP[dt])
    out = np.empty_like(x)
    _check(
        lib().oracle_rope(dt, _p(x), _p(out), _ll(seq_len), _ll(num_heads), _ll(head_dim), ctypes.c_double(base),
                          _ll(start), ctypes.c_int(mode), ctypes.c_int(scaling), ctypes.c_double(factor),
                          ctypes.c_double(low), ctypes.c_double(high), _ll(orig_ctx)),
        "rope",
    )
    return out


def rope_pairs(x, cos, sin):
    x = np.ascontiguousarray(x, dtype=np.float32)
    cos = np.ascontiguousarray(cos, dtype=np.float32)
    sin = np.ascontiguousarray(sin, dtype=np.float32)
    out = np.empty_like(x)
    _check(lib().oracle_rope_pairs(_p(out), _p(x), _p(cos), _p(sin), _ll(cos.size)), "rope_pairs")
    return out


def page_write(dt, storage, values, page_ids, offsets, page_count, page_size, inner, storage_offset=0):
    storage = np.ascontiguousarray(storage, dtype=_NP[dt])
    values = np.ascontiguousarray(values, dtype=_NP[dt])
    page_ids = np.ascontiguousarray(page_ids, dtype=np.int32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    out = storage.copy()
    _check(
        lib().oracle_page_write(dt, _p(out), _p(values), _p(page_ids), _p(offsets), _p(out), _ll(page_count),
                                _ll(page_size), _ll(inner), _ll(page_ids.size), _ll(storage_offset)),
        "page_write",
    )
    return out


def page_gather(dt, storage, page_table, page_count, page_size, inner, out_rows, storage_offset=0):
    storage = np.ascontiguousarray(storage, dtype=_NP[dt])
    page_table = np.ascontiguousarray(page_table, dtype=np.int32)
    out_rows = min(out_rows, page_table.size * page_size)  # device/cpu/shape/page.go:188-192
    out = np.zeros((out_rows, inner), dtype=_NP[dt])
    _check(
        lib().oracle_page_gather(dt, _p(storage), _p(page_table), _p(out), _ll(page_count), _ll(page_size), _ll(inner),
                                 _ll(out_rows), _ll(storage_offset)),
        "page_gather",
    )
    return out


def stable_softmax_row(scores):
    s = np.ascontiguousarray(scores, dtype=np.float32).copy()
    lib().oracle_stable_softmax_row(_p(s), _ll(s.size))
    return s


def mha(dt, q, k, v, seq_q, seq_k, num_heads, kv_heads, head_dim, causal=True, window=0, alibi=0.0):
    q = np.ascontiguousarray(q, dtype=_NP[dt])
    k = np.ascontiguousarray(k, dtype=_NP[dt])
    v = np.ascontiguousarray(v, dtype=_NP[dt])
    out = np.zeros_like(q)
    _check(
        lib().oracle_mha(dt, _p(q), _p(k), _p(v), _p(out), _ll(seq_q), _ll(seq_k), _ll(num_heads), _ll(kv_heads),
                         _ll(head_dim), ctypes.c_int(int(causal)), _ll(window), ctypes.c_float(alibi)),
        "mha",
    )
    return out


def mha_rows(dt, q, k, v, seq_q, seq_k, num_heads, kv_heads, head_dim, rows, heads, causal=True):
    """MultiHeadAttention on listed (row, head) pairs only; returns [len(rows), head_dim]."""
    q = np.ascontiguousarray(q, dtype=_NP[dt])
    k = np.ascontiguousarray(k, dtype=_NP[dt])
    v = np.ascontiguousarray(v, dtype=_NP[dt])
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    heads = np.ascontiguousarray(heads, dtype=np.int32)
    out = np.zeros_like(q)
    _check(
        lib().oracle_mha_rows(dt, _p(q), _p(k), _p(v), _p(out), _ll(seq_q), _ll(seq_k), _ll(num_heads), _ll(kv_heads),
                              _ll(head_dim), ctypes.c_int(int(causal)), _p(rows), _p(heads), _ll(rows.size)),
        "mha_rows",
    )
    o3 = out.reshape(seq_q, num_heads, head_dim)
    return o3[rows, heads, :].copy()


def sdpa(dt, q, k, v, seq_q, seq_k, depth, value_dim, causal=False):
    q = np.ascontiguousarray(q, dtype=_NP[dt])
    k = np.ascontiguousarray(k, dtype=_NP[dt])
    v = np.ascontiguousarray(v, dtype=_NP[dt])
    out = np.zeros((seq_q, value_dim), dtype=_NP[dt])
    _check(
        lib().oracle_sdpa(dt, _p(q), _p(k), _p(v), _p(out), _ll(seq_q), _ll(seq_k), _ll(depth), _ll(value_dim),
                          ctypes.c_int(int(causal))),
        "sdpa",
    )
    return out


def paged_decode(dt, kv_dt, q, k_pages, v_pages, page_table, ctx_lens, page_size, num_heads, kv_heads, head_dim,
                 k_scale=None, v_scale=None):
    """page_gather(K), page_gather(V), MultiHeadAttention(seqQ=1) per sequence."""
    q = np.ascontiguousarray(q, dtype=_NP[dt])
    k_pages = np.ascontiguousarray(k_pages, dtype=_NP[kv_dt])
    v_pages = np.ascontiguousarray(v_pages, dtype=_NP[kv_dt])
    page_table = np.ascontiguousarray(page_table, dtype=np.int32)
    ctx_lens = np.ascontiguousarray(ctx_lens, dtype=np.int32)
    batch, max_pages = page_table.shape
    inner = kv_heads * head_dim
    page_count = k_pages.size // (page_size * inner)
    out = np.zeros_like(q)
    ks = None if k_scale is None else np.ascontiguousarray(k_scale, dtype=np.float32)
    vs = None if v_scale is None else np.ascontiguousarray(v_scale, dtype=np.float32)
    _check(
        lib().oracle_paged_decode(dt, kv_dt, _p(q), _p(k_pages), _p(v_pages), _p(page_table), _p(ctx_lens),
                                  _p(ks) if ks is not None else None, _p(vs) if vs is not None else None, _p(out),
                                  _ll(batch), _ll(max_pages), _ll(page_count), _ll(page_size), _ll(num_heads),
                                  _ll(kv_heads), _ll(head_dim)),
        "paged_decode",
    )
    return out
