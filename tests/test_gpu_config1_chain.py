"""BASELINE config 1: a Llama-style decoder-layer op chain (no GEMMs) in fp32, each op through the C ABI vs device/cpu semantics.

Shapes: batch 1, seq 128, hidden 512, 8 heads x head_dim 64, seed 0; RMSNorm gamma ~ U(0.5,1.5), eps 1e-5; RoPE theta 1e4 on
q,k [S=128, H=8, D=64]; causal attention (scale 1/8 == 1/sqrt(64)); SwiGLU on gate,up [128,1376]; residual add.
Parity target: <= 1e-5 relative per op output (near-zero floor as device/cpu/parity/parity.go:47,86-92).
"""
import numpy as np
import pytest

import oracle as O
from gpu_util import dev, empty, host, rel_err

pytestmark = pytest.mark.gpu


def test_config1_fp32_chain():
    import puter_b200

    O.build()
    d = puter_b200.Device()
    S, HID, H, D_, I = 128, 512, 8, 64, 1376
    rng = np.random.default_rng(0)
    x = rng.standard_normal((S, HID)).astype(np.float32)
    gamma = rng.uniform(0.5, 1.5, HID).astype(np.float32)
    q = rng.standard_normal((S, H, D_)).astype(np.float32)
    k = rng.standard_normal((S, H, D_)).astype(np.float32)
    v = rng.standard_normal((S, H * D_)).astype(np.float32)
    gate = rng.standard_normal((S, I)).astype(np.float32)
    up = rng.standard_normal((S, I)).astype(np.float32)
    F = O.F32
    report = {}

    # RMSNorm
    want_n = O.rmsnorm(F, x, gamma, 1e-5)
    o = empty(x.nbytes)
    d.RMSNorm(puter_b200.RMSNormConfig(1e-5), dev(x), dev(gamma), o, S, HID, F)
    got_n = host(o, np.float32, x.shape)
    report["rmsnorm"] = rel_err(got_n, want_n)

    # RoPE on q and k (interleaved default, and half mode)
    for mode in (0, 1):
        cfg = puter_b200.RoPEConfig(BaseFreq=10000.0, Mode=mode)
        for name, t in (("q", q), ("k", k)):
            want = O.rope(F, t, S, H, D_, base=10000.0, mode=mode)
            o = empty(t.nbytes)
            d.RoPE(cfg, dev(t), o, S, H, D_, F)
            got = host(o, np.float32, t.shape)
            assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
            report[f"rope_{name}_{mode}"] = float(np.abs(got - want).max())
    qr = O.rope(F, q, S, H, D_, base=10000.0)
    kr = O.rope(F, k, S, H, D_, base=10000.0)

    # causal attention on the rotated q, k
    want_a = O.mha(F, qr.reshape(S, H * D_), kr.reshape(S, H * D_), v, S, S, H, H, D_, True)
    o = empty(v.nbytes)
    d.MultiHeadAttention(puter_b200.MultiHeadAttentionConfig(NumHeads=H, HeadDim=D_, Causal=True), dev(qr), dev(kr), dev(v), o, S, S, F)
    got_a = host(o, np.float32, v.shape)
    report["attention"] = rel_err(got_a, want_a)

    # SwiGLU (two-tensor form) and the residual add
    want_s = O.gated_tensors(O.SWIGLU, F, gate, up)
    o = empty(gate.nbytes)
    d.SwiGLUTensors(o, dev(gate), dev(up), gate.size, F)
    got_s = host(o, np.float32, gate.shape)
    report["swiglu"] = rel_err(got_s, want_s)
    want_r = O.binary(O.ADD, F, x, want_a)
    o = empty(x.nbytes)
    d.Add(o, dev(x), dev(got_a), x.size, F)
    got_r = host(o, np.float32, x.shape)
    report["residual"] = rel_err(got_r, want_r)

    for name in ("rmsnorm", "attention", "swiglu", "residual"):
        assert report[name] <= 1e-5, report
    assert np.array_equal(got_s.view(np.uint32), want_s.view(np.uint32))  # the polynomial exp is reproduced bit for bit
