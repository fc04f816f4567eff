"""GPU parity: attention family through the C ABI vs the CPU oracle (and the reference's literal fixtures)."""
import numpy as np
import pytest

import oracle as O
from gpu_util import dev, empty, host, rel_err

pytestmark = pytest.mark.gpu
ES = {O.F32: 4, O.F16: 2, O.BF16: 2, O.E4M3: 1}


@pytest.fixture(scope="module")
def d():
    import puter_b200

    O.build()
    return puter_b200.Device()


def run_mha(d, dt, q, k, v, sq, sk, hq, hkv, dim, causal=True, window=0):
    import puter_b200

    out = empty(q.size * ES[dt])
    cfg = puter_b200.MultiHeadAttentionConfig(NumHeads=hq, HeadDim=dim, Causal=causal, WindowSize=window, KVHeadCount=hkv)
    d.MultiHeadAttention(cfg, dev(q), dev(k), dev(v), out, sq, sk, dt)
    return host(out, O.np_dtype(dt), (sq, hq * dim))


def test_decode_gqa_causal_known_answer(d):
    # device/metal/attention/multihead_parity_darwin_test.go:16-37
    q = np.zeros((1, 4), np.float32)
    k = np.zeros((3, 2), np.float32)
    v = np.array([[1, 10], [2, 20], [3, 30]], np.float32)
    got = run_mha(d, O.F32, q, k, v, 1, 3, 2, 1, 2)
    assert np.abs(got.ravel() - np.array([2, 20, 2, 20], np.float32)).max() <= 4e-6  # <= 2 ULP as in the reference test


def test_prefill_gqa_3x3_fixture(d):
    # device/metal/attention/multihead_parity_darwin_test.go:39-72 (<= 8 ULP vs CPU there)
    q = np.array([0.25, -0.50, 0.75, 0.10, -0.30, 0.20, 0.40, -0.80, 0.60, 0.90, -0.20, 0.35], np.float32).reshape(3, 4)
    k = np.array([0.10, 0.20, -0.40, 0.30, 0.50, -0.70], np.float32).reshape(3, 2)
    v = np.array([1, 10, 2, 20, 3, 30], np.float32).reshape(3, 2)
    want = O.mha(O.F32, q, k, v, 3, 3, 2, 1, 2, True)
    got = run_mha(d, O.F32, q, k, v, 3, 3, 2, 1, 2)
    assert rel_err(got, want) <= 1e-6


def test_softmax_infinity_rows_through_attention(d):
    # device/cpu/attention/softmax_test.go:10-40, reached through scores: q.k = +Inf for chosen keys
    big = np.float32(3e38)
    q = np.array([[big, 0]], np.float32)
    k = np.array([[1, 0], [big, 0], [0.5, 0]], np.float32)  # only the dot with key 1 overflows to +Inf
    v = np.array([[1, 1], [5, 7], [9, 9]], np.float32)
    want = O.mha(O.F32, q, k, v, 1, 3, 1, 1, 2, False)
    got = run_mha(d, O.F32, q, k, v, 1, 3, 1, 1, 2, causal=False)
    assert np.array_equal(got, want) and got.ravel().tolist() == [5, 7]


@pytest.mark.parametrize("sq,sk,hq,hkv,dim,causal,window", [(128, 128, 8, 8, 64, True, 0), (7, 64, 4, 2, 16, True, 0),
                                                            (33, 33, 6, 3, 40, False, 0), (1, 1024, 4, 1, 128, True, 0),
                                                            (64, 64, 2, 2, 32, True, 9), (5, 3, 2, 1, 8, True, 0)])
def test_mha_f32_matches_cpu_within_1e5(d, sq, sk, hq, hkv, dim, causal, window):
    rng = np.random.default_rng(sq * sk + dim)
    q = rng.standard_normal((sq, hq * dim)).astype(np.float32)
    k = rng.standard_normal((sk, hkv * dim)).astype(np.float32)
    v = rng.standard_normal((sk, hkv * dim)).astype(np.float32)
    want = O.mha(O.F32, q, k, v, sq, sk, hq, hkv, dim, causal, window)
    got = run_mha(d, O.F32, q, k, v, sq, sk, hq, hkv, dim, causal, window)
    assert rel_err(got, want) <= 1e-5
    assert (got.view(np.uint32) != want.view(np.uint32)).mean() < 0.01  # same operation order: almost always bit-equal


@pytest.mark.parametrize("dt", [O.BF16, O.F16])
@pytest.mark.parametrize("sq,sk,hq,hkv,dim", [(16, 16, 4, 2, 64), (9, 40, 2, 1, 32), (64, 64, 8, 8, 16)])
def test_mha_16bit_exact_path_reproduces_rounded_scores(d, dt, sq, sk, hq, hkv, dim):
    rng = np.random.default_rng(sq + sk)
    q = O.from_f32(rng.standard_normal((sq, hq * dim)).astype(np.float32), dt)
    k = O.from_f32(rng.standard_normal((sk, hkv * dim)).astype(np.float32), dt)
    v = O.from_f32(rng.standard_normal((sk, hkv * dim)).astype(np.float32), dt)
    want = O.mha(dt, q, k, v, sq, sk, hq, hkv, dim, True)
    got = run_mha(d, dt, q, k, v, sq, sk, hq, hkv, dim)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dt", [O.F32, O.BF16, O.F16])
@pytest.mark.parametrize("sq,sk,depth,vd,causal", [(2, 2, 3, 4, False), (64, 64, 32, 32, True), (17, 50, 24, 40, False), (128, 128, 64, 64, True)])
def test_flash_attention_single_head(d, dt, sq, sk, depth, vd, causal):
    import puter_b200

    rng = np.random.default_rng(sq * depth)
    q = O.from_f32(rng.standard_normal((sq, depth)).astype(np.float32), dt)
    k = O.from_f32(rng.standard_normal((sk, depth)).astype(np.float32), dt)
    v = O.from_f32(rng.standard_normal((sk, vd)).astype(np.float32), dt)
    want = O.sdpa(dt, q, k, v, sq, sk, depth, vd, causal)
    out = empty(sq * vd * ES[dt])
    d.FlashAttention(puter_b200.FlashAttentionConfig(Causal=causal), dev(q), dev(k), dev(v), out, sq, sk, depth, vd, dt)
    got = host(out, O.np_dtype(dt), (sq, vd))
    if dt == O.F32:
        assert rel_err(got, want) <= 1e-5
    else:
        assert np.abs(O.to_f32(got, dt) - O.to_f32(want, dt)).max() <= 2e-2
    assert (got.view(np.uint8) != want.view(np.uint8)).mean() < 0.01


def make_paged(rng, batch, ctx_lens, page_size, hkv, dim, kv_dt, extra_pages=3):
    pages_per = [(c + page_size - 1) // page_size for c in ctx_lens]
    total = sum(pages_per) + extra_pages
    max_pages = max(max(pages_per), 1)
    perm = rng.permutation(total).astype(np.int32)
    table = np.zeros((batch, max_pages), np.int32)
    at = 0
    for b, n in enumerate(pages_per):
        table[b, :n] = perm[at:at + n]
        at += n
    kf = rng.standard_normal((total, page_size, hkv * dim)).astype(np.float32)
    vf = rng.standard_normal((total, page_size, hkv * dim)).astype(np.float32)
    ks = vs = None
    if kv_dt == O.E4M3:
        ks = rng.uniform(0.01, 0.1, hkv).astype(np.float32)
        vs = rng.uniform(0.01, 0.1, hkv).astype(np.float32)
        kq = O.from_f32((kf.reshape(total, page_size, hkv, dim) / ks[None, None, :, None]).reshape(kf.shape), O.E4M3)
        vq = O.from_f32((vf.reshape(total, page_size, hkv, dim) / vs[None, None, :, None]).reshape(vf.shape), O.E4M3)
    else:
        kq, vq = O.from_f32(kf, kv_dt), O.from_f32(vf, kv_dt)
    return table, kq, vq, ks, vs, total, max_pages


@pytest.mark.parametrize("dt,kv_dt", [(O.BF16, O.BF16), (O.F16, O.F16), (O.BF16, O.E4M3)])
@pytest.mark.parametrize("ctx_lens,page_size,hq,hkv", [([1], 16, 32, 8), ([3, 17, 0, 512, 100], 16, 32, 8), ([700, 33], 16, 8, 8),
                                                       ([250, 1, 77], 16, 16, 1), ([90, 300], 32, 12, 4), ([45, 130], 4, 8, 2),
                                                       ([2048, 1500, 16, 999], 16, 32, 8), ([64, 65], 16, 48, 16)])
def test_paged_decode_matches_gather_then_mha(d, dt, kv_dt, ctx_lens, page_size, hq, hkv):
    import puter_b200

    dim = 128
    batch = len(ctx_lens)
    rng = np.random.default_rng(sum(ctx_lens) + page_size + hq)
    table, kq, vq, ks, vs, total, max_pages = make_paged(rng, batch, ctx_lens, page_size, hkv, dim, kv_dt)
    q = O.from_f32(rng.standard_normal((batch, hq * dim)).astype(np.float32), dt)
    ctx = np.array(ctx_lens, np.int32)
    want = O.paged_decode(dt, kv_dt, q, kq, vq, table, ctx, page_size, hq, hkv, dim, ks, vs)
    sentinel = np.full(q.shape, 0x5151, np.uint16)
    out = dev(sentinel)
    cfg = puter_b200.MultiHeadAttentionConfig(NumHeads=hq, HeadDim=dim, Causal=True, KVHeadCount=hkv)
    d.PagedDecodeAttention(cfg, dev(q), dev(kq), dev(vq), dev(table), dev(ctx), out, batch, max_pages, total, page_size, dt,
                           kvFormat=kv_dt, kScale=None if ks is None else dev(ks), vScale=None if vs is None else dev(vs))
    got = host(out, np.uint16, q.shape)
    assert d.take_error() == 0
    for b, c in enumerate(ctx_lens):
        if c == 0:
            assert np.array_equal(got[b], sentinel[b])  # empty context: row untouched
        else:
            err = np.abs(O.to_f32(got[b], dt) - O.to_f32(want[b], dt)).max()
            assert err <= 2e-2, (b, c, err)
    live = np.array(ctx_lens) > 0
    if kv_dt == dt:
        assert (got[live] != want[live]).mean() < 0.05  # rounded scores are reproduced: nearly all outputs bit-equal
    else:
        # fp8 pages are multiplied as stored; q and the softmax weights enter as two e4m3 terms (~8 significant bits)
        err = np.abs(O.to_f32(got[live], dt) - O.to_f32(want[live], dt))
        assert err.mean() <= 2e-3


@pytest.mark.parametrize("kv_dt", [O.BF16, O.E4M3])
@pytest.mark.parametrize("ctx_lens,hq,hkv", [([2048, 1500, 16, 999], 32, 8), ([3000], 4, 4), ([90, 300, 40], 16, 2)])
def test_paged_decode_merge_paths_agree(d, monkeypatch, kv_dt, ctx_lens, hq, hkv):
    """A sequence spread over several workers is merged by its owners together under a cooperative launch (a share each, one
    of two routines depending on the number of owners) and by the last warp to arrive under a plain launch.  The plain launch
    is what a refused cooperative launch falls back to; PUTER_DECODE_NO_COOPERATIVE selects it.  All routes weight the same
    partials: the results agree to the last bits of the float32 sums and meet the same bound against the oracle."""
    import puter_b200

    dim, page_size, dt = 128, 16, O.BF16
    batch = len(ctx_lens)
    rng = np.random.default_rng(sum(ctx_lens) + hq)
    table, kq, vq, ks, vs, total, max_pages = make_paged(rng, batch, ctx_lens, page_size, hkv, dim, kv_dt)
    q = O.from_f32(rng.standard_normal((batch, hq * dim)).astype(np.float32), dt)
    ctx = np.array(ctx_lens, np.int32)
    want = O.to_f32(O.paged_decode(dt, kv_dt, q, kq, vq, table, ctx, page_size, hq, hkv, dim, ks, vs), dt)
    cfg = puter_b200.MultiHeadAttentionConfig(NumHeads=hq, HeadDim=dim, Causal=True, KVHeadCount=hkv)
    args = (cfg, dev(q), dev(kq), dev(vq), dev(table), dev(ctx))
    kw = dict(kvFormat=kv_dt, kScale=None if ks is None else dev(ks), vScale=None if vs is None else dev(vs))
    results = []
    for plain in (False, True, False):
        if plain:
            monkeypatch.setenv("PUTER_DECODE_NO_COOPERATIVE", "1")
        else:
            monkeypatch.delenv("PUTER_DECODE_NO_COOPERATIVE", raising=False)
        out = dev(np.full(q.shape, 0x5151, np.uint16))
        d.PagedDecodeAttention(*args, out, batch, max_pages, total, page_size, dt, **kw)
        results.append(host(out, np.uint16, q.shape))
        assert d.take_error() == 0
    coop, plain, again = results
    assert np.array_equal(coop, again)  # the plain launch left the arrival counters at zero, and each route is deterministic
    assert np.abs(O.to_f32(coop, dt) - want).max() <= 2e-2
    assert np.abs(O.to_f32(plain, dt) - want).max() <= 2e-2
    assert (coop != plain).mean() < 0.02  # different summation trees over the same partials: rare last-bit differences only


def test_paged_decode_step_replays_from_a_cuda_graph(d):
    """A decode step is one (cooperative) kernel launch with no host synchronisation and no allocation once the workspace
    has its size: it can be captured into a CUDA graph and replayed, with the same bits as the eager call."""
    import puter_b200
    import torch

    dim, page_size, hq, hkv, dt = 128, 16, 32, 8, O.BF16
    ctx_lens = [2048, 1500, 16, 999]
    batch = len(ctx_lens)
    rng = np.random.default_rng(77)
    table, kq, vq, _, _, total, max_pages = make_paged(rng, batch, ctx_lens, page_size, hkv, dim, dt)
    q = O.from_f32(rng.standard_normal((batch, hq * dim)).astype(np.float32), dt)
    cfg = puter_b200.MultiHeadAttentionConfig(NumHeads=hq, HeadDim=dim, Causal=True, KVHeadCount=hkv)
    args = (cfg, dev(q), dev(kq), dev(vq), dev(table), dev(np.array(ctx_lens, np.int32)))
    eager = dev(np.zeros(q.shape, np.uint16))
    replayed = dev(np.zeros(q.shape, np.uint16))
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        # the eager call sizes the workspace and moves the context to this stream before the capture begins
        d.PagedDecodeAttention(*args, eager, batch, max_pages, total, page_size, dt)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            d.PagedDecodeAttention(*args, replayed, batch, max_pages, total, page_size, dt)
    assert not host(replayed, np.uint16, q.shape).any()  # capturing ran nothing
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert np.array_equal(host(replayed, np.uint16, q.shape), host(eager, np.uint16, q.shape))
    assert d.take_error() == 0


def test_paged_decode_flags_bad_page_ids_and_long_contexts(d):
    import puter_b200

    rng = np.random.default_rng(5)
    hq, hkv, dim, ps = 8, 2, 128, 16
    table, kq, vq, _, _, total, max_pages = make_paged(rng, 2, [40, 40], ps, hkv, dim, O.BF16)
    q = O.from_f32(rng.standard_normal((2, hq * dim)).astype(np.float32), O.BF16)
    cfg = puter_b200.MultiHeadAttentionConfig(NumHeads=hq, HeadDim=dim, Causal=True, KVHeadCount=hkv)
    bad = table.copy()
    bad[0, 1] = total + 100
    out = empty(q.nbytes)
    d.PagedDecodeAttention(cfg, dev(q), dev(kq), dev(vq), dev(bad), dev(np.array([40, 40], np.int32)), out, 2, max_pages, total, ps, O.BF16)
    assert d.take_error() == 1
    d.PagedDecodeAttention(cfg, dev(q), dev(kq), dev(vq), dev(table), dev(np.array([40, 4000], np.int32)), out, 2, max_pages, total, ps, O.BF16)
    assert d.take_error() == 1
    with pytest.raises(puter_b200.DeviceError):  # unsupported head_dim is refused, not approximated
        bad_cfg = puter_b200.MultiHeadAttentionConfig(NumHeads=8, HeadDim=64, Causal=True, KVHeadCount=2)
        d.PagedDecodeAttention(bad_cfg, dev(q), dev(kq), dev(vq), dev(table), dev(np.array([40, 40], np.int32)), out, 2, max_pages, total, ps, O.BF16)


@pytest.mark.parametrize("dt", [O.BF16, O.F16])
@pytest.mark.parametrize("sk,hq,hkv", [(1, 8, 2), (100, 32, 8), (3000, 4, 4)])
def test_mha_decode_fast_path_seqq1(d, dt, sk, hq, hkv):
    rng = np.random.default_rng(sk)
    dim = 128
    q = O.from_f32(rng.standard_normal((1, hq * dim)).astype(np.float32), dt)
    k = O.from_f32(rng.standard_normal((sk, hkv * dim)).astype(np.float32), dt)
    v = O.from_f32(rng.standard_normal((sk, hkv * dim)).astype(np.float32), dt)
    want = O.mha(dt, q, k, v, 1, sk, hq, hkv, dim, True)
    got = run_mha(d, dt, q, k, v, 1, sk, hq, hkv, dim)
    assert np.abs(O.to_f32(got, dt) - O.to_f32(want, dt)).max() <= 2e-2
    d.set_exact(True)
    try:
        assert np.array_equal(run_mha(d, dt, q, k, v, 1, sk, hq, hkv, dim), want)
    finally:
        d.set_exact(False)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("batch,seq,hq,hkv,dim", [(2, 40, 4, 2, 64), (1, 130, 8, 2, 128), (2, 256, 8, 2, 128)])
def test_rope_attention_prefill_small(d, mode, batch, seq, hq, hkv, dim):
    import puter_b200

    dt = O.BF16
    rng = np.random.default_rng(seq + mode)
    q = O.from_f32(rng.standard_normal((batch, seq, hq * dim)).astype(np.float32), dt)
    k = O.from_f32(rng.standard_normal((batch, seq, hkv * dim)).astype(np.float32), dt)
    v = O.from_f32(rng.standard_normal((batch, seq, hkv * dim)).astype(np.float32), dt)
    out = empty(q.nbytes)
    rope = puter_b200.RoPEConfig(BaseFreq=500000.0, Mode=mode)
    attn = puter_b200.MultiHeadAttentionConfig(NumHeads=hq, HeadDim=dim, Causal=True, KVHeadCount=hkv)
    d.RoPEAttentionPrefill(rope, attn, dev(q), dev(k), dev(v), out, batch, seq, dt)
    got = host(out, np.uint16, q.shape)
    for b in range(batch):
        qr = O.rope(dt, q[b], seq, hq, dim, base=500000.0, mode=mode)
        kr = O.rope(dt, k[b], seq, hkv, dim, base=500000.0, mode=mode)
        want = O.mha(dt, qr, kr, v[b], seq, seq, hq, hkv, dim, True)
        assert np.abs(O.to_f32(got[b], dt) - O.to_f32(want.reshape(seq, -1), dt)).max() <= 2e-2


@pytest.mark.parametrize("dt", [O.BF16, O.F16])
@pytest.mark.parametrize("seq,hq,hkv,causal", [(128, 1, 1, True), (256, 4, 2, True), (384, 2, 2, False), (1024, 8, 2, True), (200, 4, 1, True)])
def test_tensor_core_prefill_through_mha_entry(d, dt, seq, hq, hkv, causal):
    """bf16/f16 self-attention with head_dim 128 runs on the tcgen05 kernel; compared with the CPU semantics."""
    dim = 128
    rng = np.random.default_rng(seq + hq)
    q = O.from_f32(rng.standard_normal((seq, hq * dim)).astype(np.float32), dt)
    k = O.from_f32(rng.standard_normal((seq, hkv * dim)).astype(np.float32), dt)
    v = O.from_f32(rng.standard_normal((seq, hkv * dim)).astype(np.float32), dt)
    want = O.mha(dt, q, k, v, seq, seq, hq, hkv, dim, causal)
    got = run_mha(d, dt, q, k, v, seq, seq, hq, hkv, dim, causal=causal)
    assert d.take_error() == 0
    err = np.abs(O.to_f32(got, dt) - O.to_f32(want, dt))
    assert err.max() <= 2e-2, (float(err.max()), np.unravel_index(err.argmax(), err.shape))
    assert err.mean() <= 2e-3


def test_prefill_config3_full_size_on_a_row_sample(d):
    """Config 3 at full size (B=4, S=4096, 32/8 heads, head_dim 128, RoPE theta 5e5 fused): sampled rows vs the oracle."""
    import puter_b200
    import torch

    B, S, HQ, HKV, D_ = 4, 4096, 32, 8, 128
    dt = O.BF16
    rng = np.random.default_rng(1)
    q = O.from_f32(rng.standard_normal((B, S, HQ * D_), dtype=np.float32), dt)
    k = O.from_f32(rng.standard_normal((B, S, HKV * D_), dtype=np.float32), dt)
    v = O.from_f32(rng.standard_normal((B, S, HKV * D_), dtype=np.float32), dt)
    out = empty(q.nbytes)
    rope = puter_b200.RoPEConfig(BaseFreq=500000.0, Mode=1)
    attn = puter_b200.MultiHeadAttentionConfig(NumHeads=HQ, HeadDim=D_, Causal=True, KVHeadCount=HKV)
    d.RoPEAttentionPrefill(rope, attn, dev(q), dev(k), dev(v), out, B, S, dt)
    got = host(out, np.uint16, q.shape)
    assert d.take_error() == 0
    worst = 0.0
    for b in (0, 3):
        qr = O.rope(dt, q[b], S, HQ, D_, base=500000.0, mode=1)
        kr = O.rope(dt, k[b], S, HKV, D_, base=500000.0, mode=1)
        rows = np.concatenate([np.arange(8), np.arange(S - 8, S), rng.integers(0, S, 48)]).astype(np.int32)
        heads = rng.integers(0, HQ, rows.size).astype(np.int32)
        want = O.mha_rows(dt, qr, kr, v[b], S, S, HQ, HKV, D_, rows, heads, causal=True)
        g = got[b].reshape(S, HQ, D_)[rows, heads, :]
        worst = max(worst, float(np.abs(O.to_f32(g, dt) - O.to_f32(want, dt)).max()))
    assert worst <= 2e-2, worst
    # size-independent property: row 0 attends only to key 0, so out[0] == v[0] of its KV head, exactly
    v0 = v[:, 0, :].reshape(B, HKV, D_)
    assert np.array_equal(got[:, 0, :].reshape(B, HQ, D_), np.repeat(v0, HQ // HKV, axis=1))


@pytest.mark.parametrize("batch,seq,hq,hkv,causal,mode", [(3, 1000, 16, 4, True, 1), (3, 1000, 16, 4, True, 0), (2, 640, 32, 8, False, None),
                                                        (5, 520, 32, 8, True, 1)])
def test_prefill_persistent_grid_many_items_per_cta(d, batch, seq, hq, hkv, causal, mode):
    """More (batch, head, row block) items than SMs, ragged last tiles, with and without fused RoPE: every CTA of the persistent
    grid runs several items back to back (barrier phases, K/V ring and staging tile carried across items).  Checked on a row
    sample of every batch item against the CPU semantics."""
    import puter_b200

    dim, dt = 128, O.BF16
    rng = np.random.default_rng(seq + hq + (mode or 7))
    q = O.from_f32(rng.standard_normal((batch, seq, hq * dim), dtype=np.float32), dt)
    k = O.from_f32(rng.standard_normal((batch, seq, hkv * dim), dtype=np.float32), dt)
    v = O.from_f32(rng.standard_normal((batch, seq, hkv * dim), dtype=np.float32), dt)
    out = empty(q.nbytes)
    rope = None if mode is None else puter_b200.RoPEConfig(BaseFreq=500000.0, Mode=mode)
    cfg = puter_b200.MultiHeadAttentionConfig(NumHeads=hq, HeadDim=dim, Causal=causal, KVHeadCount=hkv)
    d.RoPEAttentionPrefill(rope, cfg, dev(q), dev(k), dev(v), out, batch, seq, dt)
    got = O.to_f32(host(out, np.uint16, (batch, seq, hq, dim)), dt)
    assert d.take_error() == 0
    rows = np.array([0, 1, 127, 128, 255, 256, 300, seq // 2, seq - 129, seq - 2, seq - 1], np.int32)
    for b in range(batch):
        qb, kb = q[b], k[b]
        if mode is not None:
            qb = O.rope(dt, qb, seq, hq, dim, base=500000.0, mode=mode).reshape(seq, hq * dim)
            kb = O.rope(dt, kb, seq, hkv, dim, base=500000.0, mode=mode).reshape(seq, hkv * dim)
        r = np.repeat(rows, hq)
        h = np.tile(np.arange(hq, dtype=np.int32), rows.size)
        want = O.to_f32(O.mha_rows(dt, qb, kb, v[b], seq, seq, hq, hkv, dim, r, h, causal), dt)
        assert np.abs(got[b, r, h] - want).max() <= 2e-2
