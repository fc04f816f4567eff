"""The allocation-free paged-decode entry point (for callers that may not call cudaMalloc while a decode step runs:
pre-planned serving arenas, latency-critical sections, runtimes that forbid driver allocations after start-up).

Calls cuda_dispatch_paged_decode_attention_noalloc through the C ABI twice in a row, on two different problems, and
checks each result against the regular entry point (bit for bit: both run the same kernels over the same split).  The
scratch array is shared by all calls and keeps the previous call's contents, so the second call also proves that stale
contents do no harm.  Also checked: free device memory does not move across calls, and the documented size limit.
Collected last on purpose.
"""
import numpy as np
import pytest

import oracle as O
from gpu_util import dev, empty, host
from test_gpu_attention import make_paged

pytestmark = pytest.mark.gpu


def _problem(seed, ctx_lens, hq, hkv, kv_dt):
    rng = np.random.default_rng(seed)
    dim, ps = 128, 16
    table, kq, vq, ks, vs, total, max_pages = make_paged(rng, len(ctx_lens), ctx_lens, ps, hkv, dim, kv_dt)
    q = O.from_f32(rng.standard_normal((len(ctx_lens), hq * dim)).astype(np.float32), O.BF16)
    return dict(q=q, k=kq, v=vq, table=table, ctx=np.array(ctx_lens, np.int32), ks=ks, vs=vs, total=total, max_pages=max_pages,
                hq=hq, hkv=hkv, dim=dim, ps=ps, kv_dt=kv_dt)


def _run(d, p, noalloc):
    import puter_b200

    cfg = puter_b200.MultiHeadAttentionConfig(NumHeads=p["hq"], HeadDim=p["dim"], Causal=True, KVHeadCount=p["hkv"])
    out = empty(p["q"].nbytes, fill=0)
    fn = d.PagedDecodeAttentionNoAlloc if noalloc else d.PagedDecodeAttention
    fn(cfg, dev(p["q"]), dev(p["k"]), dev(p["v"]), dev(p["table"]), dev(p["ctx"]), out, len(p["ctx"]), p["max_pages"], p["total"],
       p["ps"], O.BF16, kvFormat=p["kv_dt"], kScale=None if p["ks"] is None else dev(p["ks"]),
       vScale=None if p["vs"] is None else dev(p["vs"]))
    return host(out, np.uint16, p["q"].shape)


def test_noalloc_entry_matches_regular_entry_on_two_calls_in_a_row():
    import puter_b200
    import torch

    O.build()
    d = puter_b200.Device()
    first = _problem(101, [3000, 17, 640, 2049, 1], 32, 8, O.BF16)
    second = _problem(202, [90, 5000, 333], 16, 4, O.E4M3)  # different shape and KV type: stale scratch must not matter
    got1 = _run(d, first, noalloc=True)
    got2 = _run(d, second, noalloc=True)
    want1 = _run(d, first, noalloc=False)
    want2 = _run(d, second, noalloc=False)
    assert d.take_error() == 0
    # both entry points run the same kernels over the same split of the work and merge the partials in the same order,
    # so the results are not merely close: they are the same bits
    assert np.array_equal(got1, want1) and np.array_equal(got2, want2)
    # and against the CPU oracle, like the regular entry point's own test
    ref = O.paged_decode(O.BF16, O.BF16, first["q"], first["k"], first["v"], first["table"], first["ctx"], 16, 32, 8, 128)
    assert np.abs(O.to_f32(got1, O.BF16) - O.to_f32(ref, O.BF16)).max() <= 2e-2

    # the property the entry point exists for: with every buffer of a step already on the device, further calls leave the
    # amount of free device memory exactly where it was (no cudaMalloc / cudaFree behind the caller's back)
    cfg = puter_b200.MultiHeadAttentionConfig(NumHeads=32, HeadDim=128, Causal=True, KVHeadCount=8)
    bufs = [dev(first[k]) for k in ("q", "k", "v", "table", "ctx")]
    out = empty(first["q"].nbytes, fill=0)
    args = (cfg, *bufs, out, len(first["ctx"]), first["max_pages"], first["total"], 16, O.BF16)
    d.PagedDecodeAttentionNoAlloc(*args)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        d.PagedDecodeAttentionNoAlloc(*args)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert np.array_equal(host(out, np.uint16, first["q"].shape), want1)


def test_noalloc_entry_refuses_problems_beyond_its_fixed_scratch():
    import puter_b200
    import torch

    d = puter_b200.Device()
    p = _problem(7, [16] * 600, 32, 8, O.BF16)  # 600 sequences x 32 heads do not fit the 8 MiB array
    with pytest.raises(puter_b200.DeviceError) as e:
        _run(d, p, noalloc=True)
    assert e.value.code == -2 and "fixed" in e.value.message
    assert _run(d, p, noalloc=False).shape == p["q"].shape  # the regular entry point still takes it
    # the documented limit for 32 query heads over 8 KV heads on a 148-SM GPU: 355 sequences fit, 356 do not
    if torch.cuda.get_device_properties(0).multi_processor_count == 148:
        ok = _problem(8, [16] * 355, 32, 8, O.BF16)
        assert np.array_equal(_run(d, ok, noalloc=True), _run(d, ok, noalloc=False))
        over = _problem(9, [16] * 356, 32, 8, O.BF16)
        with pytest.raises(puter_b200.DeviceError) as e:
            _run(d, over, noalloc=True)
        assert e.value.code == -2
    assert d.take_error() == 0
