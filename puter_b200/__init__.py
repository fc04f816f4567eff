"""puter_b200 — B200 (sm_100a) kernels for puter's LLM-execution hot path behind its device operator API.

The product is ``libputer_b200.so`` (C ABI in ``include/puter_b200.h``).  This Python package is the thin
plumbing used by the tests and the benchmark: a ctypes binding (``_lib``) and ``Device``, which mirrors the
method names and argument order of ``device/interface.go`` over torch tensors (torch only provides device
memory, streams and process groups).
"""
from . import dtypes
from .device import (Device, DeviceError, FlashAttentionConfig, ModulatedLayerNormConfig, MultiHeadAttentionConfig, RMSNormConfig,
                     RoPEConfig)

__all__ = ["Device", "DeviceError", "RMSNormConfig", "RoPEConfig", "MultiHeadAttentionConfig", "FlashAttentionConfig", "ModulatedLayerNormConfig",
           "dtypes"]
