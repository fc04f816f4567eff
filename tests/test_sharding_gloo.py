"""Host-side multi-GPU logic on CPU: partition helpers, and a world_size-2 gloo run of the sharded config-5 chain and the
sharded decode step, with the CPU oracle standing in for the kernels (the collective and the bookkeeping are what is tested)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from puter_b200 import sharding  # noqa: E402


def test_row_shard_covers_everything_once():
    for total in (0, 1, 7, 16384, 1000):
        for world in (1, 2, 3, 4, 8):
            blocks = [sharding.row_shard(total, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == total
            assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            sizes = [e - s for s, e in blocks]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.row_shard(10, 2, 2)


def test_modulation_rows():
    assert sharding.modulation_rows(0, 16384, 4096) == (0, 4, 4096)
    assert sharding.modulation_rows(8192, 16384, 4096) == (2, 2, 4096)
    assert sharding.modulation_rows(6144, 8192, 4096) == (1, 1, 2048)
    with pytest.raises(ValueError):
        sharding.modulation_rows(1000, 9000, 4096)


def test_lpt_assign_balances_context_lengths():
    rng = np.random.default_rng(2)
    ctx = rng.integers(512, 32768, 64, endpoint=True)
    for world in (1, 2, 4, 8):
        owned = sharding.lpt_assign(ctx, world)
        assert sorted(i for o in owned for i in o) == list(range(64))
        loads = [int(ctx[o].sum()) for o in owned]
        assert max(loads) <= 1.002 * (sum(loads) / world)  # 1.3 % at 8 ranks before the exchange refinement


def test_lpt_assign_refinement_never_loses_to_plain_lpt_and_is_deterministic():
    def plain_lpt(costs, world):
        loads = [0] * world
        for c in sorted((int(c) for c in costs), reverse=True):
            loads[loads.index(min(loads))] += c
        return max(loads)

    rng = np.random.default_rng(7)
    for trial in range(40):
        n = int(rng.integers(1, 80))
        world = int(rng.integers(1, 9))
        costs = rng.integers(1, 40000, n)
        owned = sharding.lpt_assign(costs, world)
        assert owned == sharding.lpt_assign(costs, world)  # same input, same partition
        assert sorted(i for o in owned for i in o) == list(range(n))
        assert all(o == sorted(o) for o in owned)
        assert max(int(costs[o].sum()) if o else 0 for o in owned) <= plain_lpt(costs, world)
    assert sharding.lpt_assign([], 3) == [[], [], []]
    assert sharding.lpt_assign([5], 2) == [[0], []]


def test_prefill_units():
    for world in (1, 2, 4, 8):
        units = [u for r in range(world) for u in sharding.prefill_units(4, 8, world, r)]
        assert sorted(units) == [(b, h) for b in range(4) for h in range(8)]
        assert len(sharding.prefill_units(4, 8, world, 0)) == 32 // world


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    import oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    O.set_threads(1)
    # ---- config-5 chain on sharded token rows, outputs all-gathered ----
    T, C, I, B = 64, 128, 192, 4
    rpb = T // B
    rng = np.random.default_rng(3)  # every rank generates the full inputs and takes its block
    mk = lambda *s: O.from_f32(rng.standard_normal(s).astype(np.float32), O.BF16)
    x, r, br = mk(T, C), mk(T, C), mk(T, C)
    gamma = O.from_f32(rng.uniform(0.5, 1.5, C).astype(np.float32), O.BF16)
    mod = O.from_f32(rng.uniform(0, 1, (B, 3 * C)).astype(np.float32), O.BF16)
    gate, up = mk(T, I), mk(T, I)
    s, e = sharding.row_shard(T, world, rank)
    first, nb, local_rpb = sharding.modulation_rows(s, e, rpb)
    h = O.binary(O.ADD, O.BF16, x[s:e], r[s:e])
    n_loc = O.rmsnorm(O.BF16, h, gamma, 1e-6)
    g_loc = O.gated_residual(O.BF16, h, br[s:e], mod[first:first + nb], e - s, C, local_rpb, 3 * C, 0).reshape(e - s, C)
    s_loc = O.gated_tensors(O.SWIGLU, O.BF16, gate[s:e], up[s:e])
    gathered = []
    for loc in (n_loc, g_loc, s_loc):
        t = torch.from_numpy(loc.astype(np.int32))  # gloo has no 16-bit integer collectives; widen the bit patterns
        full = torch.empty((T,) + tuple(t.shape[1:]), dtype=torch.int32)
        dist.all_gather_into_tensor(full, t)
        gathered.append(full.numpy().astype(np.uint16))
    # ---- decode: sequences assigned by context length, outputs gathered by index ----
    ctx = np.array([40, 300, 17, 90, 210, 64], np.int32)
    owned = sharding.lpt_assign(ctx, world)[rank]
    hq, hkv, dim, ps = 4, 2, 128, 16
    rng2 = np.random.default_rng(7)
    q = O.from_f32(rng2.standard_normal((len(ctx), hq * dim)).astype(np.float32), O.BF16)
    outs = np.zeros((len(ctx), hq * dim), np.int32)
    for i in owned:  # each rank holds only the pages of its own sequences
        rs = np.random.default_rng(100 + i)
        pages = (ctx[i] + ps - 1) // ps
        k = O.from_f32(rs.standard_normal((pages, ps, hkv * dim)).astype(np.float32), O.BF16)
        v = O.from_f32(rs.standard_normal((pages, ps, hkv * dim)).astype(np.float32), O.BF16)
        table = rs.permutation(pages).astype(np.int32)[None, :]
        outs[i] = O.paged_decode(O.BF16, O.BF16, q[i:i + 1], k, v, table, ctx[i:i + 1], ps, hq, hkv, dim)[0]
    tt = torch.from_numpy(outs)
    dist.all_reduce(tt)  # disjoint rows: the sum is the gather (0.5 MB at full size)
    if rank == 0:
        np.savez(os.path.join(out_dir, f"w{world}.npz"), n=gathered[0], g=gathered[1], s=gathered[2], dec=tt.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_world_size_2_matches_world_size_1(tmp_path):
    import torch.multiprocessing as mp

    results = {}
    for world, port in ((1, 29611), (2, 29612)):
        mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
        results[world] = np.load(os.path.join(tmp_path, f"w{world}.npz"))
    for key in ("n", "g", "s", "dec"):
        assert np.array_equal(results[1][key], results[2][key]), key
    assert results[2]["dec"].any()
