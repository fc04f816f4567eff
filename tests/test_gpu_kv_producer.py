"""KV-cache producer (RoPE(k) -> [e4m3 quantise] -> paged write of K and V in one launch) against the composition of the
reference ops restated by the oracle: rope at each row's position, convert, page write."""
import numpy as np
import pytest

import oracle as O
from gpu_util import dev, empty, host

pytestmark = pytest.mark.gpu


def reference(dt, kv_dt, k, v, positions, page_ids, offsets, k_pool, v_pool, heads, dim, page_size, mode, base, k_scale, v_scale):
    rows = k.shape[0]
    k_rot = np.empty_like(k)
    for r in range(rows):  # one row at its own position
        k_rot[r] = O.rope(dt, k[r].copy(), 1, heads, dim, base=base, start=int(positions[r]), mode=mode).reshape(-1)
    def quant(x, scale):
        if kv_dt != O.E4M3:
            return x
        f = O.to_f32(x, dt).reshape(rows, heads, dim) / scale.reshape(1, heads, 1).astype(np.float32)
        return O.convert(f.astype(np.float32).reshape(-1), O.F32, O.E4M3).reshape(rows, heads * dim)
    kq, vq = quant(k_rot, k_scale), quant(v, v_scale)
    pages = k_pool.shape[0]
    inner = heads * dim
    ko = O.page_write(kv_dt, k_pool.reshape(-1), kq.reshape(-1), page_ids, offsets, pages, page_size, inner)
    vo = O.page_write(kv_dt, v_pool.reshape(-1), vq.reshape(-1), page_ids, offsets, pages, page_size, inner)
    return ko, vo


@pytest.mark.parametrize("dt", [O.BF16, O.F16])
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("mode", [0, 1])
def test_producer_equals_rope_convert_page_write(dt, fp8, mode):
    import puter_b200

    d = puter_b200.Device()
    rng = np.random.default_rng(7 + mode + 2 * fp8)
    rows, heads, dim, page_size, pages, max_pos = 37, 4, 128, 16, 9, 4096
    kv_dt = O.E4M3 if fp8 else dt
    k = O.from_f32(rng.standard_normal((rows, heads * dim)).astype(np.float32), dt)
    v = O.from_f32(rng.standard_normal((rows, heads * dim)).astype(np.float32), dt)
    positions = rng.integers(0, max_pos, rows).astype(np.int32)
    slots = rng.permutation(pages * page_size)[:rows]
    page_ids, offsets = (slots // page_size).astype(np.int32), (slots % page_size).astype(np.int32)
    es = 1 if fp8 else 2
    pool_dtype = np.uint8 if fp8 else np.uint16
    k_pool = rng.integers(0, 120, (pages, page_size, heads * dim)).astype(pool_dtype)  # previous contents must survive elsewhere
    v_pool = rng.integers(0, 120, (pages, page_size, heads * dim)).astype(pool_dtype)
    k_scale = rng.uniform(0.01, 0.1, heads).astype(np.float32)
    v_scale = rng.uniform(0.01, 0.1, heads).astype(np.float32)
    want_k, want_v = reference(dt, kv_dt, k, v, positions, page_ids, offsets, k_pool, v_pool, heads, dim, page_size, mode, 500000.0,
                               k_scale, v_scale)
    kp, vp = dev(k_pool), dev(v_pool)
    cfg = puter_b200.RoPEConfig(BaseFreq=500000.0, Mode=mode)
    d.RoPEKVPageWrite(cfg, dev(k), dev(v), dev(positions), dev(page_ids), dev(offsets), kp, vp, rows, heads, dim, pages, page_size, max_pos,
                      dt, kv_dt, dev(k_scale) if fp8 else None, dev(v_scale) if fp8 else None)
    got_k = host(kp, pool_dtype).reshape(-1)
    got_v = host(vp, pool_dtype).reshape(-1)
    assert d.take_error() == 0
    assert np.array_equal(got_v, np.asarray(want_v).view(pool_dtype).reshape(-1))
    assert np.array_equal(got_k, np.asarray(want_k).view(pool_dtype).reshape(-1))


def test_producer_skips_bad_rows_and_raises_the_flag():
    import puter_b200

    d = puter_b200.Device()
    rng = np.random.default_rng(3)
    rows, heads, dim, page_size, pages = 4, 2, 64, 16, 2
    k = O.from_f32(rng.standard_normal((rows, heads * dim)).astype(np.float32), O.BF16)
    pool = np.full((pages, page_size, heads * dim), 0x1234, np.uint16)
    kp, vp = dev(pool), dev(pool.copy())
    positions = np.array([0, 1, 99999, 3], np.int32)          # row 2: position beyond the table
    page_ids = np.array([0, 7, 1, 1], np.int32)               # row 1: page out of range
    offsets = np.array([0, 0, 0, 5], np.int32)
    d.RoPEKVPageWrite(puter_b200.RoPEConfig(), dev(k), dev(k), dev(positions), dev(page_ids), dev(offsets), kp, vp, rows, heads, dim, pages,
                      page_size, 1024, O.BF16)
    got = host(vp, np.uint16).reshape(pages, page_size, heads * dim)
    assert d.take_error() != 0
    assert np.array_equal(got[0, 0], k[0]) and np.array_equal(got[1, 5], k[3])
    untouched = np.ones((pages, page_size), bool)
    untouched[0, 0] = untouched[1, 5] = False
    assert (got[untouched] == 0x1234).all()
