"""Parity at the stated sizes of configurations 4 and 5, on the very tensors bench.py times (bench_inputs is shared).

Config 4: the whole B = 64 batch (contexts U[512, 32768], page 16, permuted page table, bf16 and e4m3 KV) runs on the GPU;
the CPU oracle (page_gather + MultiHeadAttention, device/cpu/attention/typed_compute.go:142-237,
device/cpu/shape/page_generic.go:30-50) runs on a sample that holds the longest and the shortest sequence and six others.
Config 5: 16384 x 4096 / 14336 through the fused Add + RMSNorm + GatedResidual kernel and SwiGLUTensors; the oracle
(device/cpu/layernorm/compute.go:364-374 and the unfused ops) runs on a row sample.
"""
import numpy as np
import pytest

import bench_inputs as BI
import oracle as O
from gpu_util import empty, host, ulp16_diff

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def d():
    import puter_b200

    O.build()
    return puter_b200.Device()


@pytest.fixture(scope="module")
def batch():
    return BI.DecodeBatch()


def _sample(batch):
    rng = np.random.default_rng(99)
    picked = [int(np.argmax(batch.ctx)), int(np.argmin(batch.ctx))]
    for i in rng.permutation(batch.batch):
        if len(picked) == 8:
            break
        if int(i) not in picked:
            picked.append(int(i))
    return picked


@pytest.mark.parametrize("fp8", [False, True], ids=["bf16kv", "e4m3kv"])
def test_config4_paged_decode_full_size(d, batch, fp8):
    import puter_b200
    import torch

    assert batch.batch == 64 and batch.ctx.min() >= 512 and batch.ctx.max() <= 32768
    kv_dt = O.E4M3 if fp8 else O.BF16
    st = BI.upload_decode(d, batch, range(batch.batch), fp8)
    out = torch.zeros(batch.batch, BI.HQ * BI.DIM, dtype=torch.int16, device="cuda")
    cfg = puter_b200.MultiHeadAttentionConfig(NumHeads=BI.HQ, HeadDim=BI.DIM, Causal=True, KVHeadCount=BI.HKV)
    d.PagedDecodeAttention(cfg, st["q"], st["k"], st["v"], st["table"], st["ctx"], out, batch.batch, st["max_pages"], st["total_pages"],
                           BI.PAGE, O.BF16, kvFormat=kv_dt, kScale=st.get("k_scale"), vScale=st.get("v_scale"))
    got = out.cpu().numpy().view(np.uint16)
    assert d.take_error() == 0

    picked = _sample(batch)
    es = 1 if fp8 else 2
    qs, ks, vs = [], [], []
    for i in picked:
        q, k, v = batch.sequence(i)
        if fp8:
            k, v = batch.scaled_for_fp8(k, v)
        kb, vb = O.from_f32(k, kv_dt), O.from_f32(v, kv_dt)
        # paged-KV indexing is bit-exact: gathering sequence i out of the permuted pool gives back exactly its rows
        rows = batch.rows(i)
        for pool, want in ((st["k"], kb), (st["v"], vb)):
            g = empty(rows * BI.INNER * es)
            d.KVPageGather(pool, st["table"][i].contiguous(), g, st["total_pages"], BI.PAGE, BI.INNER, rows, 0, kv_dt)
            assert np.array_equal(host(g, want.dtype, want.shape), want), f"gathered pages of sequence {i} differ"
        qs.append(O.from_f32(q, O.BF16))  # the bench's numpy rounding and the convert package's agree on the query rows
        ks.append(kb)
        vs.append(vb)
    assert d.take_error() == 0
    assert np.array_equal(np.stack(qs), st["q_host"].numpy().view(np.uint16)[picked])

    # the oracle on a pool that holds only the sampled sequences, pages in order
    pages = [int(batch.pages_per[i]) for i in picked]
    table = np.zeros((len(picked), max(pages)), np.int32)
    at = 0
    for r, n in enumerate(pages):
        table[r, :n] = np.arange(at, at + n)
        at += n
    kmini = np.concatenate(ks).reshape(at, BI.PAGE, BI.INNER)
    vmini = np.concatenate(vs).reshape(at, BI.PAGE, BI.INNER)
    O.set_threads(O.max_threads())
    want = O.paged_decode(O.BF16, kv_dt, np.stack(qs), kmini, vmini, table, batch.ctx[picked], BI.PAGE, BI.HQ, BI.HKV, BI.DIM,
                          batch.k_scale if fp8 else None, batch.v_scale if fp8 else None)
    g = got[picked]
    err = np.abs(O.to_f32(g, O.BF16) - O.to_f32(want, O.BF16))
    assert err.max() <= 2e-2, float(err.max())
    if fp8:
        assert err.mean() <= 2e-3, float(err.mean())
    else:
        assert (g == want).mean() > 0.95, float((g == want).mean())
    # every row of the batch was written and is finite
    f = O.to_f32(got, O.BF16)
    assert np.isfinite(f).all() and (np.abs(f).max(axis=1) > 0).all()


def test_config5_chain_full_size(d):
    import puter_b200
    import torch

    inp = BI.ChainInputs()
    assert (inp.T, inp.C, inp.I) == (16384, 4096, 14336)
    t = BI.upload_chain(inp, 0, inp.T)
    T, C, I = inp.T, inp.C, inp.I
    h = torch.empty(T, C, dtype=torch.int16, device="cuda")
    n = torch.empty(T, C, dtype=torch.int16, device="cuda")
    g = torch.empty(T, C, dtype=torch.int16, device="cuda")
    s = torch.empty(T, I, dtype=torch.int16, device="cuda")
    d.AddRMSNormGatedResidual(puter_b200.RMSNormConfig(1e-6), t["x"], t["r"], t["gamma"], t["branch"], t["mod"], h, n, g, T, C,
                              inp.rows_per_batch, 3 * C, 0, O.BF16)
    d.SwiGLUTensors(s, t["gate"], t["up"], T * I, O.BF16)
    assert d.take_error() == 0

    rpb = inp.rows_per_batch
    rng = np.random.default_rng(5)
    rows = sorted(set([b * rpb for b in range(inp.B)] + [b * rpb + rpb - 1 for b in range(inp.B)] + [int(r) for r in rng.integers(0, T, 24)]))
    src = inp.rows(rows)
    idx = torch.tensor(rows, device="cuda")
    got = {k: v[idx].cpu().numpy().view(np.uint16) for k, v in (("h", h), ("n", n), ("g", g), ("s", s))}
    want_h = O.binary(O.ADD, O.BF16, src["x"], src["r"])
    want_n = O.rmsnorm(O.BF16, want_h, inp.gamma, 1e-6)
    want_g = np.stack([O.gated_residual(O.BF16, want_h[j:j + 1], src["branch"][j:j + 1], inp.mod[r // rpb:r // rpb + 1], 1, C, 1, 3 * C, 0)
                       .reshape(C) for j, r in enumerate(rows)])
    want_s = O.gated_tensors(O.SWIGLU, O.BF16, src["gate"], src["up"])
    assert np.array_equal(got["h"], want_h)
    assert np.array_equal(got["g"], want_g)
    assert ulp16_diff(got["n"], want_n).max() <= 1
    assert ulp16_diff(got["s"], want_s).max() <= 1
    assert (got["n"] == want_n).mean() > 0.98 and (got["s"] == want_s).mean() > 0.98
