"""The seeded input generators shared by bench.py and the full-size GPU parity tests (no GPU needed)."""
import numpy as np

import bench_inputs as BI
import oracle as O
from puter_b200 import sharding


def test_numpy_bf16_rounding_equals_the_convert_package_rule():
    rng = np.random.default_rng(0)
    bits = rng.integers(0, 2**32, 1 << 18, dtype=np.uint64).astype(np.uint32)
    bits[:8] = [0, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00001, 0xFF800001, 0x3F808000, 0x3F818000]
    f = bits.view(np.float32)
    assert np.array_equal(BI.bf16_bits(f), O.convert(f, O.F32, O.BF16))
    b = rng.integers(0, 65536, 4096).astype(np.uint16)
    assert np.array_equal(BI.bf16_to_f32(b).view(np.uint32), O.convert(b, O.BF16, O.F32).view(np.uint32))


def test_decode_batch_is_the_seeded_configuration():
    d = BI.DecodeBatch()
    assert d.batch == 64 and d.ctx.min() >= 512 and d.ctx.max() <= 32768
    ref = np.random.default_rng(2).integers(512, 32768, 64, endpoint=True)
    assert np.array_equal(d.ctx, ref)
    assert sorted(d.perm.tolist()) == list(range(d.total_pages))  # page table = a permutation of the physical pages
    assert d.total_pages == int(((ref + 15) // 16).sum())
    assert ((d.k_scale >= 0.01) & (d.k_scale <= 0.1)).all() and ((d.v_scale >= 0.01) & (d.v_scale <= 0.1)).all()
    # a sequence's draws do not depend on how they are asked for
    small = BI.DecodeBatch(ctx_min=20, ctx_max=90, batch=5)
    q, k, v = small.sequence(3)
    q2, k2, v2 = small.sequence(3)
    assert np.array_equal(k, k2) and np.array_equal(q, q2) and k.shape == (small.rows(3), BI.INNER)
    assert abs(float(k.mean())) < 0.02 and abs(float(k.std()) - 1) < 0.02
    assert not np.array_equal(small.sequence(2)[1][:16], k[:16])


def test_shard_tables_keep_sequences_disjoint_and_complete():
    d = BI.DecodeBatch()
    for world in (1, 2, 4, 8):
        owned = sharding.lpt_assign(d.ctx, world)
        assert sorted(i for o in owned for i in o) == list(range(64))
        for o in owned:
            table, count = d.shard_tables(o)
            assert count == int(d.pages_per[o].sum()) or world == 1
            used = np.concatenate([table[r, :d.pages_per[i]] for r, i in enumerate(o)])
            assert sorted(used.tolist()) == list(range(len(used))) or world == 1  # a permutation of the shard's pool
            assert len(set(used.tolist())) == len(used) and used.max() < count
        total = sum(d.algorithmic_bytes(o) for o in owned)
        assert total == d.algorithmic_bytes()
    # E[bytes] of the stated configuration: about 4.4 GB in bf16, half of it in e4m3
    assert 3.5e9 < d.algorithmic_bytes() < 5.5e9 and d.algorithmic_bytes(esize=1) < 0.51 * d.algorithmic_bytes() + 1e6


def test_chain_blocks_and_row_lookup_agree():
    c = BI.ChainInputs(T=512, C=64, I=96, B=2)
    b1 = c.block(1)
    rows = c.rows([256, 300, 511, 0])
    assert np.array_equal(rows["x"][0], b1["x"][0]) and np.array_equal(rows["gate"][1], b1["gate"][44])
    assert np.array_equal(rows["up"][2], b1["up"][255]) and np.array_equal(rows["r"][3], c.block(0)["r"][0])
    g = BI.bf16_to_f32(c.gamma)
    assert g.min() >= 0.5 and g.max() <= 1.5
    assert c.algorithmic_bytes() == 2 * 5 * 512 * 64 + 2 * 3 * 512 * 96
    full = BI.ChainInputs()
    assert full.algorithmic_bytes() == 2 * (5 * 16384 * 4096) + 2 * (3 * 16384 * 14336)


def test_prefill_items_and_flops():
    p = BI.PrefillInputs(B=2, S=64)
    it = p.item(1)
    assert it["q"].shape == (64, 32 * 128) and it["k"].shape == (64, 8 * 128) and it["q"].dtype == np.uint16
    assert np.array_equal(it["v"], p.item(1)["v"]) and not np.array_equal(it["v"], p.item(0)["v"])
    assert BI.PrefillInputs().flops() == 4 * 4 * 32 * 128 * (4096 * 4097 // 2)
