"""``Device``: the hot-path subset of puter's ``device.Backend`` over the C ABI.

Method names, argument order and error behaviour follow ``device/interface.go``; configs follow
``device/config.go``.  Tensor arguments are CUDA ``torch.Tensor`` objects used purely as device memory
(their ``data_ptr`` is wrapped in a non-owning ``CUDABufferRef``); dims and the element ``format`` are passed
explicitly, as in the Go interface.  A failing call raises ``DeviceError`` — the counterpart of the panic in
the reference's void methods (device/cuda/compute_host.go:42-46).  Zero-sized problems are silent no-ops.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

from . import _lib, dtypes

# op codes (include/puter_b200.h)
UNARY = {"ReLU": 0, "Exp": 8, "Log": 9, "Tanh": 12, "Sigmoid": 13, "Silu": 14, "Swish": 15, "Softsign": 16, "ELU": 17, "SELU": 18,
         "LeakyReLU": 19, "HardSigmoid": 20, "HardSwish": 21, "Gelu": 22, "Log1p": 23, "Expm1": 24, "CELU": 25, "Softplus": 26,
         "Mish": 27, "LogSigmoid": 28, "GeluTanh": 29, "HardTanh": 30, "HardGelu": 31, "QuickGelu": 32, "TanhShrink": 33}
BINARY = {"Add": 0, "Sub": 1, "Mul": 2, "Div": 3, "Max": 4, "Min": 5}
GATED = {"SwiGLU": "swiglu", "GeGLU": "geglu", "GLU": "glu", "ReGLU": "reglu", "SiGLU": "siglu", "GeGLUTanh": "geglu_tanh",
         "SeGLU": "seglu", "LinGLU": "linglu"}

RoPEModeInterleaved, RoPEModeHalf = 0, 1
RoPEScalingNone, RoPEScalingLlama3 = 0, 1


class DeviceError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


@dataclass
class RMSNormConfig:  # device/config.go:82-92
    Epsilon: float = 1e-5


@dataclass
class ModulatedLayerNormConfig:  # device/config.go:94-109
    Epsilon: float = 1e-6
    Set: int = 0


@dataclass
class RoPEConfig:  # device/config.go:123-134; defaults device/cpu/rope/config.go:7-15
    BaseFreq: float = 10000.0
    StartPosition: int = 0
    Mode: int = RoPEModeInterleaved
    Scaling: int = RoPEScalingNone
    ScalingFactor: float = 1.0
    LowFreqFactor: float = 0.0
    HighFreqFactor: float = 0.0
    OriginalContext: int = 0


@dataclass
class FlashAttentionConfig:  # device/config.go:278-281
    BlockSize: int = 64
    Causal: bool = False


@dataclass
class MultiHeadAttentionConfig:  # device/config.go:283-290
    NumHeads: int = 1
    HeadDim: int = 1
    Causal: bool = False
    WindowSize: int = 0
    ALiBiSlope: float = 0.0
    KVHeadCount: int = 0


class SharedBuffer:
    """Device memory that the per-GPU processes of one box can all address (CUDA IPC): allocated by ``Device.alloc_shared`` or
    mapped from a peer's ``handle`` by ``Device.open_shared``.  ``torch.as_tensor(buf, device="cuda")`` views it as bytes."""

    def __init__(self, dev, ref, nbytes, handle=None):
        self._dev, self.ref, self.nbytes, self.handle = dev, ref, nbytes, handle
        self.ptr = int(dev.lib.cuda_buffer_device_ptr(ref))
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 2}

    def close(self):
        if self.ref is not None:
            self._dev.lib.cuda_buffer_release(self.ref)
            self.ref = None


class Device:
    """One context on one GPU.  ``Device()`` opens the current torch CUDA device."""

    def __init__(self, ordinal: int | None = None, follow_torch_stream: bool = True):
        import torch

        self._torch = torch
        self.lib = _lib.load()
        if ordinal is None:
            ordinal = torch.cuda.current_device() if torch.cuda.is_available() else 0
        self.ordinal = ordinal
        self._status = _lib.CUDAStatus()
        ref = ctypes.c_void_p()
        rc = self.lib.cuda_open_device_index(ordinal, ctypes.byref(ref), ctypes.byref(self._status))
        if rc != 0 or not ref.value:
            raise DeviceError(rc, self._status.message.decode(errors="replace"))
        self.ref = ref
        self.follow_torch_stream = follow_torch_stream
        self._stream = None  # stream last handed to the library
        self._refs = {}      # (address, bytes) -> CUDABufferRef

    # ---- plumbing -------------------------------------------------------------------------------------
    def close(self):
        if getattr(self, "ref", None):
            for r in self._refs.values():
                self.lib.cuda_buffer_release(r)
            self._refs.clear()
            self.lib.cuda_close_device(self.ref)
            self.ref = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != 0:
            raise DeviceError(self._status.code, self._status.message.decode(errors="replace"))

    def _enter(self):
        if self.follow_torch_stream:
            s = self._torch.cuda.current_stream(self.ordinal).cuda_stream
            if s != self._stream:  # the library keeps the stream until told otherwise: only a change costs a call
                self.lib.cuda_context_set_stream(self.ref, ctypes.c_void_p(s), ctypes.byref(self._status))
                self._stream = s

    def _ref(self, t):
        """Non-owning CUDABufferRef of a tensor's memory.  Handles are cached by (address, size): a serving loop passes the
        same buffers every step, and a handle is only a (pointer, size) record, so reuse is safe for as long as the
        address range stays valid for the call that uses it."""
        if t is None:
            return None
        assert t.is_cuda and t.is_contiguous(), "device tensors must be contiguous CUDA memory"
        key = (t.data_ptr(), t.numel() * t.element_size())
        r = self._refs.get(key)
        if r is None:
            r = ctypes.c_void_p(self.lib.cuda_buffer_wrap(self.ref, ctypes.c_void_p(key[0]), key[1]))
            self._refs[key] = r
        return r

    def _call(self, name, tensors, build_args):
        self._enter()
        if len(self._refs) >= 4096:  # bound the cache (between calls only): handles are cheap to rebuild
            for old in self._refs.values():
                self.lib.cuda_buffer_release(old)
            self._refs.clear()
        args = build_args([self._ref(t) for t in tensors])
        rc = getattr(self.lib, name)(self.ref, *args, ctypes.byref(self._status))
        self._check(rc)

    # ---- memory shared between the per-GPU processes of a box ----------------------------------------
    def alloc_shared(self, nbytes: int) -> SharedBuffer:
        ref = self.lib.cuda_buffer_alloc(self.ref, nbytes)
        if not ref:
            raise DeviceError(-7, "cuda: allocation of %d shared bytes failed" % nbytes)
        ref = ctypes.c_void_p(ref)
        handle = ctypes.create_string_buffer(64)
        self._check(self.lib.cuda_buffer_ipc_export(ref, handle, ctypes.byref(self._status)))
        return SharedBuffer(self, ref, nbytes, handle.raw)

    def open_shared(self, handle: bytes, nbytes: int) -> SharedBuffer:
        ref = self.lib.cuda_buffer_ipc_import(self.ref, ctypes.c_char_p(handle), nbytes, ctypes.byref(self._status))
        if not ref:
            raise DeviceError(self._status.code, self._status.message.decode(errors="replace"))
        return SharedBuffer(self, ctypes.c_void_p(ref), nbytes)

    def _ref_any(self, t):
        return t.ref if isinstance(t, SharedBuffer) else self._ref(t)

    def _ref_table(self, items):
        refs = [self._ref_any(t) for t in items]
        return (ctypes.c_void_p * len(refs))(*[r.value for r in refs])

    def set_exact(self, exact: bool):
        self._check(self.lib.cuda_context_set_exact(self.ref, int(exact), ctypes.byref(self._status)))

    def launch_count(self) -> int:
        return int(self.lib.cuda_context_launch_count(self.ref))

    def take_error(self) -> int:
        self._enter()
        flag = ctypes.c_int(0)
        self._check(self.lib.cuda_context_take_error(self.ref, ctypes.byref(flag), ctypes.byref(self._status)))
        return flag.value

    def synchronize(self):
        stream = self.lib.cuda_context_default_stream(self.ref)
        self._check(self.lib.cuda_stream_synchronize(ctypes.c_void_p(stream), ctypes.byref(self._status)))

    # ---- convert package ------------------------------------------------------------------------------
    def Convert(self, dst, src, count, dst_format, src_format):
        """Device-side cast (execution/shape_cast_intrinsic.go:57-114 on the host in the reference)."""
        self._call("cuda_dispatch_convert", [src, dst], lambda r: (src_format, dst_format, r[0], r[1], count, 0))

    def ConvertHost(self, dst_np, src_np, dst_format, src_format):
        """convert.<X>To<Y>(dst, src): host slices in and out (convert/bf16_f32.go:11-22 etc.).

        Unequal lengths raise DeviceError(-2) like ErrLenMismatch (convert/errors.go:10-15)."""
        self._enter()
        rc = self.lib.cuda_convert_host(self.ref, src_format, dst_format, ctypes.c_void_p(src_np.ctypes.data), src_np.size,
                                        ctypes.c_void_p(dst_np.ctypes.data), dst_np.size, ctypes.byref(self._status))
        self._check(rc)

    # ---- Activation -----------------------------------------------------------------------------------
    def _unary(self, op, dst, src, count, format):
        self._call("cuda_dispatch_unary_elementwise", [src, dst], lambda r: (UNARY[op], format, r[0], r[1], count, 0))

    def Relu(self, dst, src, count, format):  # kept beside ReLU: the earlier spelling of this mirror
        self._unary("ReLU", dst, src, count, format)

    def Softmax(self, dst, src, count, format):
        """device.Activation.Softmax (device/interface.go:65): the softmax of ONE vector of `count` elements."""
        self._call("cuda_dispatch_softmax", [src, dst], lambda r: (format, r[0], r[1], 1, count, 0))

    def LogSoftmax(self, dst, src, count, format):
        """device.Activation.LogSoftmax (device/interface.go:46)."""
        self._call("cuda_dispatch_log_softmax", [src, dst], lambda r: (format, r[0], r[1], 1, count, 0))

    def SoftmaxRows(self, dst, src, rows, cols, format, log=False):
        """The bridge's own shape (device/cuda/activation/softmax.h:10-19): an independent softmax per row."""
        self._call("cuda_dispatch_log_softmax" if log else "cuda_dispatch_softmax", [src, dst], lambda r: (format, r[0], r[1], rows, cols, 0))

    def _gated_packed(self, variant, dst, packed, batch, halfCount, format):
        # the C ABI takes (inner = halfCount, count = batch): device/cuda/compute_host.go:1215-1231
        self._call(f"cuda_dispatch_{GATED[variant]}_packed", [dst, packed], lambda r: (format, r[0], r[1], halfCount, batch, 0))

    def _gated_tensors(self, variant, dst, gate, up, count, format):
        self._call(f"cuda_dispatch_{GATED[variant]}", [dst, gate, up], lambda r: (format, r[0], r[1], r[2], count, 0))

    def SwiGLU(self, dst, packed, batch, halfCount, format):
        self._gated_packed("SwiGLU", dst, packed, batch, halfCount, format)

    def SwiGLUTensors(self, dst, gate, up, count, format):
        self._gated_tensors("SwiGLU", dst, gate, up, count, format)

    def GeGLU(self, dst, packed, batch, halfCount, format):
        self._gated_packed("GeGLU", dst, packed, batch, halfCount, format)

    def GeGLUTensors(self, dst, gate, up, count, format):
        self._gated_tensors("GeGLU", dst, gate, up, count, format)

    def GeGLUTanh(self, dst, packed, batch, halfCount, format):
        self._gated_packed("GeGLUTanh", dst, packed, batch, halfCount, format)

    def GeGLUTanhTensors(self, dst, gate, up, count, format):
        self._gated_tensors("GeGLUTanh", dst, gate, up, count, format)

    def GLU(self, dst, packed, batch, halfCount, format):
        self._gated_packed("GLU", dst, packed, batch, halfCount, format)

    def GLUTensors(self, dst, gate, up, count, format):
        self._gated_tensors("GLU", dst, gate, up, count, format)

    def ReGLU(self, dst, packed, batch, halfCount, format):
        self._gated_packed("ReGLU", dst, packed, batch, halfCount, format)

    def ReGLUTensors(self, dst, gate, up, count, format):
        self._gated_tensors("ReGLU", dst, gate, up, count, format)

    def SiGLU(self, dst, packed, batch, halfCount, format):
        self._gated_packed("SiGLU", dst, packed, batch, halfCount, format)

    def SiGLUTensors(self, dst, gate, up, count, format):
        self._gated_tensors("SiGLU", dst, gate, up, count, format)

    def SeGLU(self, dst, packed, batch, halfCount, format):
        self._gated_packed("SeGLU", dst, packed, batch, halfCount, format)

    def SeGLUTensors(self, dst, gate, up, count, format):
        self._gated_tensors("SeGLU", dst, gate, up, count, format)

    def LinGLU(self, dst, packed, batch, halfCount, format):
        self._gated_packed("LinGLU", dst, packed, batch, halfCount, format)

    def LinGLUTensors(self, dst, gate, up, count, format):
        self._gated_tensors("LinGLU", dst, gate, up, count, format)

    # ---- Elementwise ----------------------------------------------------------------------------------
    def _binary(self, op, dst, left, right, count, format):
        self._call("cuda_dispatch_binary_elementwise", [left, right, dst], lambda r: (BINARY[op], format, r[0], r[1], r[2], count, 0))

    def Add(self, dst, left, right, count, format):
        self._binary("Add", dst, left, right, count, format)

    def Sub(self, dst, left, right, count, format):
        self._binary("Sub", dst, left, right, count, format)

    def Mul(self, dst, left, right, count, format):
        self._binary("Mul", dst, left, right, count, format)

    def Div(self, dst, left, right, count, format):
        self._binary("Div", dst, left, right, count, format)

    def Max(self, dst, left, right, count, format):
        self._binary("Max", dst, left, right, count, format)

    def Min(self, dst, left, right, count, format):
        self._binary("Min", dst, left, right, count, format)

    # ---- LayerNorm ------------------------------------------------------------------------------------
    def RMSNorm(self, config: RMSNormConfig, input, scale, output, rows, lastDim, format):
        self._call("cuda_dispatch_rmsnorm_f64", [input, scale, output],
                   lambda r: (format, r[0], r[1], r[2], rows, lastDim, float(config.Epsilon), 0))

    def LayerNorm(self, input, scale, bias, output, rows, lastDim, format):
        """device.LayerNorm.LayerNorm (device/interface.go:362-366); epsilon 1e-5 as on the CPU."""
        self._call("cuda_dispatch_layernorm", [input, scale, bias, output], lambda r: (format, r[0], r[1], r[2], r[3], rows, lastDim, 0.0, 0))

    def LayerNormResidual(self, input, scale, bias, residual, output, rows, lastDim, format):
        """The catalog's fused layernorm + add (fusion/catalog.go:183-205): LayerNorm(input, scale, bias) + residual."""
        self._call("cuda_dispatch_layernorm_residual", [input, scale, bias, residual, output],
                   lambda r: (format, r[0], r[1], r[2], r[3], r[4], rows, lastDim, 0.0, 0))

    def AdaptiveRMSNorm(self, config: RMSNormConfig, input, modulation, output, rows, lastDim, rowsPerBatch, modulationCols, format):
        """device.LayerNorm.AdaptiveRMSNorm (device/interface.go:356-361)."""
        self._call("cuda_dispatch_adaptive_rmsnorm", [input, modulation, output],
                   lambda r: (format, r[0], r[1], r[2], rows, lastDim, rowsPerBatch, modulationCols, float(config.Epsilon), 0))

    def ModulatedLayerNorm(self, config: "ModulatedLayerNormConfig", input, modulation, output, rows, lastDim, rowsPerBatch, modulationCols,
                           format):
        """device.LayerNorm.ModulatedLayerNorm (device/interface.go:367-372)."""
        self._call("cuda_dispatch_modulated_layernorm", [input, modulation, output],
                   lambda r: (format, r[0], r[1], r[2], rows, lastDim, rowsPerBatch, modulationCols, int(config.Set), float(config.Epsilon), 0))

    def GatedResidual(self, residual, branch, modulation, output, rows, lastDim, rowsPerBatch, modulationCols, set, format):
        """execution/math_gated_residual_intrinsic.go:11-17 (gatedResidualDevice)."""
        self._call("cuda_dispatch_gated_residual", [residual, branch, modulation, output],
                   lambda r: (format, r[0], r[1], r[2], r[3], rows, lastDim, rowsPerBatch, modulationCols, set, 0))

    def AddRMSNormGatedResidual(self, config: RMSNormConfig, x, residual, scale, branch, modulation, hOut, normOut, gatedOut, rows,
                                lastDim, rowsPerBatch, modulationCols, set, format):
        """Fused Add -> RMSNorm (+ GatedResidual on the sum); catalog-style fusion (fusion/catalog.go:183-205)."""
        self._call("cuda_dispatch_add_rmsnorm_gated_residual", [x, residual, scale, branch, modulation, hOut, normOut, gatedOut],
                   lambda r: (format, r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7], rows, lastDim, float(config.Epsilon),
                              rowsPerBatch, modulationCols, set, 0))

    def AddRMSNormGatedResidualGather(self, config: RMSNormConfig, x, residual, scale, branch, modulation, normAll, gatedAll, world, rank,
                                      rows, lastDim, rowsPerBatch, modulationCols, set, format):
        """AddRMSNormGatedResidual whose two outputs land in every rank's gathered tensor: normAll[r] / gatedAll[r] are rank r's
        [world * rows, lastDim] tensors (torch tensors or SharedBuffers) as this process addresses them."""
        self._enter()
        args = [self._ref(t) for t in (x, residual, scale, branch, modulation)]
        rc = self.lib.cuda_dispatch_add_rmsnorm_gated_residual_gather(
            self.ref, format, *args, self._ref_table(normAll), self._ref_table(gatedAll), world, rank, rows, lastDim, float(config.Epsilon),
            rowsPerBatch, modulationCols, set, 0, ctypes.byref(self._status))
        self._check(rc)

    def SwiGLUTensorsGather(self, dstAll, world, rank, gate, up, count, format):
        """SwiGLUTensors whose output lands at element offset rank * count of every rank's gathered tensor dstAll[r]."""
        self._enter()
        rc = self.lib.cuda_dispatch_swiglu_gather(self.ref, format, self._ref_table(dstAll), world, rank, self._ref(gate), self._ref(up),
                                                  count, 0, ctypes.byref(self._status))
        self._check(rc)

    # ---- RoPE -----------------------------------------------------------------------------------------
    def RoPE(self, config: RoPEConfig, input, output, seqLen, numHeads, headDim, format):
        self._call("cuda_dispatch_rope_f64", [input, output],
                   lambda r: (format, r[0], r[1], seqLen, numHeads, headDim, float(config.BaseFreq), int(config.StartPosition),
                              int(config.Mode), int(config.Scaling), float(config.ScalingFactor), float(config.LowFreqFactor),
                              float(config.HighFreqFactor), int(config.OriginalContext), 0))

    def RoPEPairs(self, output, input, cosBuffer, sinBuffer, halfDim, format):
        self._call("cuda_dispatch_rope_pairs", [input, output, cosBuffer, sinBuffer], lambda r: (format, r[0], r[1], r[2], r[3], halfDim, 0))

    # ---- Shape ----------------------------------------------------------------------------------------
    def LastToken(self, input, output, batch, seq, hidden, format):
        """device.Shape.LastToken (device/interface.go:622): output[b] = input[b, seq - 1, :]."""
        self._call("cuda_dispatch_last_token", [input, output], lambda r: (format, r[0], r[1], batch, seq, hidden, 0))

    def IntrinsicLastToken(self, input, output, seq, hiddenBytes, outBytes, format):
        """Device hook of the shape.last_token intrinsic (execution/shape_intrinsic.go:12-19,489-543): sizes arrive in bytes."""
        es = dtypes.SIZE[format]
        if hiddenBytes % es or (hiddenBytes and outBytes % hiddenBytes):
            raise DeviceError(-2, "shape.last_token: row of %d bytes / output of %d bytes do not fit the element type" % (hiddenBytes, outBytes))
        batch = outBytes // hiddenBytes if hiddenBytes else 0
        self.LastToken(input, output, batch, seq, hiddenBytes // es, format)

    # ---- Shape: paged KV ------------------------------------------------------------------------------
    def KVPageWrite(self, storage, values, pageIDs, offsets, output, pageCount, pageSize, inner, valueRows, storageOffset, format):
        """execution/page_intrinsic.go:13-18 (pageIntrinsicDevice)."""
        same = output is storage or output.data_ptr() == storage.data_ptr()
        tensors = [storage, values, pageIDs, offsets] + ([] if same else [output])
        self._call("cuda_dispatch_kv_page_write", tensors,
                   lambda r: (format, r[0], r[1], r[2], r[3], r[0] if same else r[4], pageCount, pageSize, inner, valueRows,
                              storageOffset, 0))

    def KVPageGather(self, storage, pageTable, output, pageCount, pageSize, inner, outRows, storageOffset, format):
        self._call("cuda_dispatch_kv_page_gather", [storage, pageTable, output],
                   lambda r: (format, r[0], r[1], r[2], pageCount, pageSize, inner, outRows, storageOffset, 0))

    def RoPEKVPageWrite(self, rope: RoPEConfig, k, v, positions, pageIDs, offsets, kPages, vPages, rows, kvHeads, headDim, pageCount,
                        pageSize, maxPositions, format, kvFormat=None, kScale=None, vScale=None):
        """KV-cache producer of a decode layer in one launch: RoPE(k) at positions[row] -> [e4m3 of value / scale] -> KVPageWrite of K
        and V (in place).  No single reference counterpart; equals RoPE + Convert + KVPageWrite run one after the other."""
        kvf = format if kvFormat is None else kvFormat
        self._call("cuda_dispatch_rope_kv_page_write", [k, v, positions, pageIDs, offsets, kPages, vPages, kScale, vScale],
                   lambda r: (format, kvf, r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7], r[8], rows, kvHeads, headDim, pageCount,
                              pageSize, maxPositions, float(rope.BaseFreq), int(rope.Mode), int(rope.Scaling), float(rope.ScalingFactor),
                              float(rope.LowFreqFactor), float(rope.HighFreqFactor), int(rope.OriginalContext), 0))

    # ---- Attention ------------------------------------------------------------------------------------
    def MultiHeadAttention(self, config: MultiHeadAttentionConfig, query, key, value, output, seqQ, seqK, format):
        if config.ALiBiSlope != 0:
            raise DeviceError(-6, "attention: ALiBi is not part of this library's path (the router never sets it)")
        kv = config.KVHeadCount if config.KVHeadCount > 0 else config.NumHeads
        variant = 2 if config.WindowSize > 0 else (1 if kv != config.NumHeads else 0)
        self._call("cuda_dispatch_multi_head_attention", [query, key, value, output],
                   lambda r: (format, variant, r[0], r[1], r[2], r[3], seqQ, seqK, config.NumHeads, kv, config.HeadDim,
                              config.WindowSize, int(config.Causal), 0))

    def FlashAttention(self, config: FlashAttentionConfig, query, key, value, output, seqQ, seqK, depth, valueDim, format):
        self._call("cuda_dispatch_flash_attention_causal", [query, key, value, output],
                   lambda r: (format, r[0], r[1], r[2], r[3], seqQ, seqK, depth, valueDim, int(config.Causal), 0))

    ScaledDotProductAttention = FlashAttention

    def RoPEAttentionPrefill(self, rope: RoPEConfig | None, attn: MultiHeadAttentionConfig, query, key, value, output, batch, seqLen, format):
        """Batched prefill: per batch item RoPE(q), RoPE(k) then causal MultiHeadAttention.  rope=None: inputs already rotated."""
        kv = attn.KVHeadCount if attn.KVHeadCount > 0 else attn.NumHeads
        rc = rope or RoPEConfig()
        mode = 2 if rope is None else int(rc.Mode)
        self._call("cuda_dispatch_rope_attention_prefill", [query, key, value, output],
                   lambda r: (format, r[0], r[1], r[2], r[3], batch, seqLen, attn.NumHeads, kv, attn.HeadDim, int(attn.Causal), mode,
                              float(rc.BaseFreq), int(rc.StartPosition), int(rc.Scaling), float(rc.ScalingFactor),
                              float(rc.LowFreqFactor), float(rc.HighFreqFactor), int(rc.OriginalContext), 0))

    def PagedDecodeAttention(self, attn: MultiHeadAttentionConfig, query, kPages, vPages, pageTable, ctxLens, output, batch,
                             maxPagesPerSeq, pageCount, pageSize, format, kvFormat=None, kScale=None, vScale=None, errorFlag=None):
        """KVPageGather(K), KVPageGather(V), MultiHeadAttention(seqQ=1, causal) per sequence, without the gathers."""
        kv = attn.KVHeadCount if attn.KVHeadCount > 0 else attn.NumHeads
        kvf = format if kvFormat is None else kvFormat
        self._call("cuda_dispatch_paged_decode_attention", [query, kPages, vPages, pageTable, ctxLens, kScale, vScale, output, errorFlag],
                   lambda r: (format, kvf, r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7], r[8], batch, maxPagesPerSeq, pageCount,
                              pageSize, attn.NumHeads, kv, attn.HeadDim, 0))

    def PagedDecodeAttentionNoAlloc(self, attn: MultiHeadAttentionConfig, query, kPages, vPages, pageTable, ctxLens, output, batch,
                                    maxPagesPerSeq, pageCount, pageSize, format, kvFormat=None, kScale=None, vScale=None, errorFlag=None):
        """PagedDecodeAttention for callers that must not allocate device memory during the step: the split-KV scratch is
        the library's fixed per-GPU array (8 MiB), so larger problems raise DeviceError(-2).  Calls on one GPU must be
        stream-ordered (they share the array); make the first call on a device outside of stream capture."""
        kv = attn.KVHeadCount if attn.KVHeadCount > 0 else attn.NumHeads
        kvf = format if kvFormat is None else kvFormat
        self._call("cuda_dispatch_paged_decode_attention_noalloc",
                   [query, kPages, vPages, pageTable, ctxLens, kScale, vScale, output, errorFlag],
                   lambda r: (format, kvf, r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7], r[8], batch, maxPagesPerSeq, pageCount,
                              pageSize, attn.NumHeads, kv, attn.HeadDim, 0))


def _make_unary(name):
    def method(self, dst, src, count, format):
        self._unary(name, dst, src, count, format)

    method.__name__ = name
    method.__qualname__ = f"Device.{name}"
    method.__doc__ = f"device.Activation.{name}(dst, src, count, format) (device/interface.go:18-74)."
    return method


# one method per unary activation that has a bridge op code: Silu, Gelu, GeluTanh, Sigmoid, Tanh, ReLU, Exp, Log, ...
for _name in UNARY:
    setattr(Device, _name, _make_unary(_name))
