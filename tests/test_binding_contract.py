"""The binding contract, pinned without a GPU: what the reference's router hands to each device method
(execution/bind_test.go:937-1199, execution/shape_intrinsic_test.go:13-51) must reach the C ABI as the
arguments include/puter_b200.h declares.  A recording stand-in replaces the shared library; tensors are
address/size records."""
import ctypes
import inspect

import pytest

from puter_b200 import device as D
from puter_b200 import dtypes


class _Tensor:
    is_cuda = True

    def __init__(self, addr, nbytes):
        self.addr, self.nbytes = addr, nbytes

    def is_contiguous(self):
        return True

    def data_ptr(self):
        return self.addr

    def numel(self):
        return self.nbytes

    def element_size(self):
        return 1


class _Lib:
    """Records every C call; buffer handles are small integers that map back to the wrapped address."""

    def __init__(self):
        self.calls = []
        self.handles = {}

    def __getattr__(self, name):
        def fn(*args):
            if name == "cuda_buffer_wrap":
                h = 1000 + len(self.handles)
                self.handles[h] = (args[1].value, args[2])
                return h
            if name == "cuda_buffer_release":
                return None
            self.calls.append((name, args))
            return 0

        return fn

    def last(self):
        name, args = self.calls[-1]
        plain = []
        for a in args[1:-1]:  # drop the context handle and the status pointer
            if isinstance(a, ctypes.c_void_p):
                plain.append(("buf", self.handles[a.value][0]) if a.value in self.handles else a.value)
            else:
                plain.append(a)
        return name, plain


@pytest.fixture
def dev():
    d = D.Device.__new__(D.Device)
    d.lib = _Lib()
    d.ref = ctypes.c_void_p(1)
    d.ordinal = 0
    d.follow_torch_stream = False
    d._stream = None
    d._refs = {}
    from puter_b200 import _lib

    d._status = _lib.CUDAStatus()
    yield d
    d.ref = None  # nothing to close


def t(addr, nbytes=1 << 20):
    return _Tensor(addr, nbytes)


def test_sdpa_bind_reaches_multi_head_attention(dev):
    # bind_test.go:1042-1090: q, k, v [1, 8, 2, 4] f32, num_heads 2, head_dim 4, causal false -> seqQ = seqK = 8, KVHeadCount 2
    cfg = D.MultiHeadAttentionConfig(NumHeads=2, HeadDim=4, Causal=False, KVHeadCount=2)
    dev.MultiHeadAttention(cfg, t(0x10), t(0x20), t(0x30), t(0x40), 8, 8, dtypes.Float32)
    name, a = dev.lib.last()
    assert name == "cuda_dispatch_multi_head_attention"
    # (dtype, variant, q, k, v, out, seqQ, seqK, numHeads, kvHeads, headDim, windowSize, causal, token)
    assert a == [dtypes.Float32, 0, ("buf", 0x10), ("buf", 0x20), ("buf", 0x30), ("buf", 0x40), 8, 8, 2, 2, 4, 0, 0, 0]
    gqa = D.MultiHeadAttentionConfig(NumHeads=32, HeadDim=128, Causal=True, KVHeadCount=8)
    dev.MultiHeadAttention(gqa, t(0x10), t(0x20), t(0x30), t(0x40), 1, 77, dtypes.BFloat16)
    assert dev.lib.last()[1][:2] == [dtypes.BFloat16, 1] and dev.lib.last()[1][6:13] == [1, 77, 32, 8, 128, 0, 1]
    unset = D.MultiHeadAttentionConfig(NumHeads=4, HeadDim=8, Causal=True)  # KVHeadCount 0 means "as many as query heads"
    dev.MultiHeadAttention(unset, t(0x10), t(0x20), t(0x30), t(0x40), 3, 3, dtypes.Float32)
    assert dev.lib.last()[1][8:10] == [4, 4]
    windowed = D.MultiHeadAttentionConfig(NumHeads=4, HeadDim=8, Causal=True, WindowSize=16)
    dev.MultiHeadAttention(windowed, t(0x10), t(0x20), t(0x30), t(0x40), 3, 3, dtypes.Float32)
    assert dev.lib.last()[1][1] == 2 and dev.lib.last()[1][11] == 16


def test_rope_bind_passes_the_full_config(dev):
    # bind_test.go:937-984: x [1, 2, 2, 4] f32, position 7, Llama-3 half mode -> seqLen 2, numHeads 2, headDim 4
    cfg = D.RoPEConfig(BaseFreq=500000.0, StartPosition=7, Mode=D.RoPEModeHalf, Scaling=D.RoPEScalingLlama3, ScalingFactor=32.0,
                       LowFreqFactor=1.0, HighFreqFactor=4.0, OriginalContext=8192)
    dev.RoPE(cfg, t(0x10), t(0x20), 2, 2, 4, dtypes.Float32)
    name, a = dev.lib.last()
    assert name == "cuda_dispatch_rope_f64"
    # (dtype, in, out, seqLen, numHeads, headDim, base, start, halfMode, scaling, factor, low, high, originalContext, token)
    assert a == [dtypes.Float32, ("buf", 0x10), ("buf", 0x20), 2, 2, 4, 500000.0, 7, 1, 1, 32.0, 1.0, 4.0, 8192, 0]
    # bind_test.go:1092-1135: a device-resident position tensor decodes to StartPosition 9
    cfg.StartPosition = 9
    dev.RoPE(cfg, t(0x10), t(0x20), 2, 2, 4, dtypes.Float32)
    assert dev.lib.last()[1][7] == 9
    assert D.RoPEConfig().BaseFreq == 10000.0 and D.RoPEConfig().Mode == D.RoPEModeInterleaved  # device/cpu/rope/config.go:7-15


def test_rmsnorm_bind(dev):
    # bind_test.go:1137-1170: x [2, 4] f32, eps 1e-5 -> rows 2, lastDim 4
    dev.RMSNorm(D.RMSNormConfig(1e-5), t(0x10), t(0x20), t(0x30), 2, 4, dtypes.Float32)
    name, a = dev.lib.last()
    assert name == "cuda_dispatch_rmsnorm_f64"
    assert a == [dtypes.Float32, ("buf", 0x10), ("buf", 0x20), ("buf", 0x30), 2, 4, 1e-5, 0]


def test_swiglu_variant_by_input_count(dev):
    # bind_test.go:1172-1199: one input selects the packed method, two inputs the tensor-pair method;
    # the C side takes (inner = halfCount, count = batch) for the packed form (device/cuda/compute_host.go:1215-1231)
    dev.SwiGLU(t(0x10), t(0x20), 128, 1376, dtypes.Float32)
    name, a = dev.lib.last()
    assert name == "cuda_dispatch_swiglu_packed" and a == [dtypes.Float32, ("buf", 0x10), ("buf", 0x20), 1376, 128, 0]
    dev.SwiGLUTensors(t(0x10), t(0x20), t(0x30), 128 * 1376, dtypes.Float32)
    name, a = dev.lib.last()
    assert name == "cuda_dispatch_swiglu" and a == [dtypes.Float32, ("buf", 0x10), ("buf", 0x20), ("buf", 0x30), 128 * 1376, 0]


def test_add_bind(dev):
    dev.Add(t(0x10), t(0x20), t(0x30), 65536, dtypes.BFloat16)
    name, a = dev.lib.last()
    # (operation, dtype, left, right, out, count, token): CUDABinaryFloat32Add = 0
    assert name == "cuda_dispatch_binary_elementwise" and a == [0, dtypes.BFloat16, ("buf", 0x20), ("buf", 0x30), ("buf", 0x10), 65536, 0]


def test_last_token_hook_and_shape_method(dev):
    # shape_intrinsic_test.go:13-51: [4, 3] f32 -> seq 4, hiddenBytes 12, outBytes 12
    dev.IntrinsicLastToken(t(0x7000), t(0x7100), 4, 12, 12, dtypes.Float32)
    name, a = dev.lib.last()
    assert name == "cuda_dispatch_last_token" and a == [dtypes.Float32, ("buf", 0x7000), ("buf", 0x7100), 1, 4, 3, 0]
    # device.Shape.LastToken(input, output, batch, seq, hidden, format), device/interface.go:622
    dev.LastToken(t(0x7000), t(0x7100), 2, 3, 2, dtypes.Float32)
    assert dev.lib.last()[1] == [dtypes.Float32, ("buf", 0x7000), ("buf", 0x7100), 2, 3, 2, 0]


@pytest.mark.parametrize("method,params", [
    # argument names and order of device/interface.go (receiver and self dropped)
    ("MultiHeadAttention", ["config", "query", "key", "value", "output", "seqQ", "seqK", "format"]),
    ("RoPE", ["config", "input", "output", "seqLen", "numHeads", "headDim", "format"]),
    ("RoPEPairs", ["output", "input", "cosBuffer", "sinBuffer", "halfDim", "format"]),
    ("RMSNorm", ["config", "input", "scale", "output", "rows", "lastDim", "format"]),
    ("SwiGLU", ["dst", "packed", "batch", "halfCount", "format"]),
    ("SwiGLUTensors", ["dst", "gate", "up", "count", "format"]),
    ("Add", ["dst", "left", "right", "count", "format"]),
    ("Silu", ["dst", "src", "count", "format"]),
    ("Gelu", ["dst", "src", "count", "format"]),
    ("Softmax", ["dst", "src", "count", "format"]),
    ("LogSoftmax", ["dst", "src", "count", "format"]),
    ("LastToken", ["input", "output", "batch", "seq", "hidden", "format"]),
    ("FlashAttention", ["config", "query", "key", "value", "output", "seqQ", "seqK", "depth", "valueDim", "format"]),
    ("GatedResidual", ["residual", "branch", "modulation", "output", "rows", "lastDim", "rowsPerBatch", "modulationCols", "set", "format"]),
    ("KVPageWrite", ["storage", "values", "pageIDs", "offsets", "output", "pageCount", "pageSize", "inner", "valueRows", "storageOffset", "format"]),
    ("KVPageGather", ["storage", "pageTable", "output", "pageCount", "pageSize", "inner", "outRows", "storageOffset", "format"]),
])
def test_method_signatures_follow_the_go_interface(method, params):
    got = [p for p in inspect.signature(getattr(D.Device, method)).parameters if p != "self"]
    assert got == params
