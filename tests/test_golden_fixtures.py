"""The committed golden file (tests/golden/golden.npz, made by tests/golden/make_golden.py): the oracle must still reproduce it
bit for bit (CPU), and the kernels must match it through the C ABI (GPU)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
G = np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))


def test_oracle_still_reproduces_the_golden_file():
    import make_golden

    fresh = make_golden.cases()
    assert sorted(fresh) == sorted(G.files)
    for name in G.files:
        a, b = np.ascontiguousarray(fresh[name]), np.ascontiguousarray(G[name])
        assert a.dtype == b.dtype and a.shape == b.shape, name
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), name


def test_reference_literals_in_the_golden_file():
    import oracle as O

    got = O.gated_residual(O.F32, G["ref_gated_residual_res"], np.ones(12, np.float32), G["ref_gated_residual_mod"], 4, 3, 2, 9, 0)
    assert np.array_equal(got, G["ref_gated_residual_want"])
    got = O.mha(O.F32, np.zeros((1, 4), np.float32), np.zeros((3, 2), np.float32), G["ref_decode_v"], 1, 3, 2, 1, 2, True)
    assert np.array_equal(got.ravel(), G["ref_decode_want"])
    for row, want in zip(G["ref_softmax_in"], G["ref_softmax_want"]):
        assert np.array_equal(O.stable_softmax_row(row), want)


@pytest.mark.gpu
def test_kernels_match_the_golden_file():
    import oracle as O
    import puter_b200
    from gpu_util import dev, empty, host, rel_err

    d = puter_b200.Device()
    F, B = O.F32, O.BF16

    def run(fn, nbytes, np_dtype, shape=None):
        out = empty(nbytes)
        fn(out)
        return host(out, np_dtype, shape)

    x32, y32, xb, yb = G["x32"], G["y32"], G["xb"], G["yb"]
    n = x32.size
    same = lambda a, b: np.array_equal(np.ascontiguousarray(a).view(np.uint8).ravel(), np.ascontiguousarray(b).view(np.uint8).ravel())
    assert same(run(lambda o: d.Silu(o, dev(x32), n, F), n * 4, np.float32), G["silu_f32"])
    assert same(run(lambda o: d.GeluTanh(o, dev(x32), n, F), n * 4, np.float32), G["gelu_tanh_f32"])
    assert np.allclose(run(lambda o: d.Gelu(o, dev(x32), n, F), n * 4, np.float32), G["gelu_f32"], rtol=1e-5, atol=1e-9)
    assert same(run(lambda o: d.Silu(o, dev(xb), n, B), n * 2, np.uint16), G["silu_bf16"])
    assert same(run(lambda o: d.SwiGLUTensors(o, dev(x32), dev(y32), n, F), n * 4, np.float32), G["swiglu_f32"])
    sw = run(lambda o: d.SwiGLUTensors(o, dev(xb), dev(yb), n, B), n * 2, np.uint16)
    assert np.abs(sw.astype(np.int32) - G["swiglu_bf16"].astype(np.int32)).max() <= 1
    assert same(run(lambda o: d.Add(o, dev(xb), dev(yb), n, B), n * 2, np.uint16), G["add_bf16"])
    got = run(lambda o: d.RMSNorm(puter_b200.RMSNormConfig(1e-5), dev(x32), dev(G["gamma"]), o, 8, 128, F), n * 4, np.float32, (8, 128))
    assert rel_err(got, G["rmsnorm_f32"]) <= 1e-6
    cfg = puter_b200.RoPEConfig(500000.0, 3, 1, 1, 32.0, 1.0, 4.0, 8192)
    got = run(lambda o: d.RoPE(cfg, dev(x32), o, 8, 2, 64, F), n * 4, np.float32)
    assert np.abs(got - G["rope_f32_llama3_half"]).max() <= 1e-5 * np.abs(G["rope_f32_llama3_half"]).max()
    f = G["conv_src_f32"]
    for name, dt in (("bf16", O.BF16), ("f16", O.F16), ("e4m3", O.E4M3), ("e5m2", O.E5M2)):
        want = G[f"conv_f32_to_{name}"]
        assert same(run(lambda o: d.Convert(o, dev(f), f.size, dt, F), want.nbytes, want.dtype), want)
    for name, dt, src in (("bf16", O.BF16, np.arange(65536, dtype=np.uint16)), ("e4m3", O.E4M3, np.arange(256, dtype=np.uint8))):
        want = G[f"conv_{name}_all"]
        assert same(run(lambda o: d.Convert(o, dev(src), src.size, F, dt), want.nbytes, np.float32), want)
    mh = puter_b200.MultiHeadAttentionConfig(NumHeads=4, HeadDim=32, Causal=True, KVHeadCount=2)
    got = run(lambda o: d.MultiHeadAttention(mh, dev(G["att_q"]), dev(G["att_k"]), dev(G["att_v"]), o, 16, 24, F), G["mha_f32"].nbytes,
              np.float32, G["mha_f32"].shape)
    assert rel_err(got, G["mha_f32"]) <= 1e-5
    qb, kb, vb = (O.from_f32(G[k], B) for k in ("att_q", "att_k", "att_v"))
    got = run(lambda o: d.MultiHeadAttention(mh, dev(qb), dev(kb), dev(vb), o, 16, 24, B), G["mha_bf16"].nbytes, np.uint16, G["mha_bf16"].shape)
    assert same(got, G["mha_bf16"])
    dc = puter_b200.MultiHeadAttentionConfig(NumHeads=8, HeadDim=128, Causal=True, KVHeadCount=2)
    got = run(lambda o: d.PagedDecodeAttention(dc, dev(G["dec_q"]), dev(G["dec_k"]), dev(G["dec_v"]), dev(G["dec_table"]), dev(G["dec_ctx"]), o,
                                               3, 7, G["dec_k"].shape[0], 16, B), G["dec_out"].nbytes, np.uint16, G["dec_out"].shape)
    assert np.abs(O.to_f32(got, B) - O.to_f32(G["dec_out"], B)).max() <= 2e-2
