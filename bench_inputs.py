"""Seeded synthetic inputs of the benchmark configurations, shared by bench.py and the full-size parity tests.

Everything is drawn from ``numpy.random.default_rng`` (PCG64): N(0,1) = ``standard_normal(float32)``, U(a,b) =
``uniform``.  Large tensors are cut into independent streams (one per sequence, batch item or row block, seeded
``default_rng([seed, index])``) so that a rank of a multi-GPU run can generate exactly its shard, generation can run
on several host threads, and the oracle side of a test can regenerate a few units without the rest.

    config 3  PrefillInputs   seed 1   q,k,v ~ N(0,1) -> bf16, per batch item
    config 4  DecodeBatch     seed 2   ctx ~ U[512, 32768], page table = random permutation, q,K,V ~ N(0,1) -> bf16
                                        (or e4m3 bytes of value / per-head scale, scale ~ U(0.01, 0.1)), per sequence
    config 5  ChainInputs     seed 3   x, r, branch, gate, up ~ N(0,1) -> bf16 per block of token rows;
                                        gamma ~ U(0.5, 1.5), modulation ~ U(0, 1)

The module itself is pure numpy.  The ``upload_*`` helpers place a shard in device memory through torch (device
memory and copies) and this library's own converter / page-write kernels.
"""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

HQ, HKV, DIM, PAGE = 32, 8, 128, 16
INNER = HKV * DIM


def host_threads() -> int:
    return max(1, min(16, os.cpu_count() or 1))


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even (bits + 0x7FFF + lsb); NaN -> (bits >> 16) | 0x40."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    if nan.any():
        r[nan] = ((u[nan] >> np.uint32(16)) | np.uint32(0x40)).astype(np.uint16)
    return r


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# ------------------------------------------------------------------------------------------------------------------
# config 4: paged decode attention
# ------------------------------------------------------------------------------------------------------------------
class DecodeBatch:
    """The seeded decode batch.  Small members (context lengths, page permutation, scales) are built eagerly; the
    per-sequence tensors are generated on demand from the stream ``default_rng([seed, 1 + i])``: first the query row
    [HQ*DIM], then K rows, then V rows, each [pages_i * PAGE, HKV*DIM] (the slack rows of the last page hold data too,
    as a live pool would)."""

    def __init__(self, seed: int = 2, batch: int = 64, ctx_min: int = 512, ctx_max: int = 32768, slack_pages: int = 0):
        self.seed, self.batch = seed, batch
        rng = np.random.default_rng(seed)
        self.ctx = rng.integers(ctx_min, ctx_max, batch, endpoint=True).astype(np.int32)
        self.pages_per = ((self.ctx.astype(np.int64) + PAGE - 1) // PAGE).astype(np.int64)
        self.total_pages = int(self.pages_per.sum()) + slack_pages
        self.page_start = np.concatenate([[0], np.cumsum(self.pages_per)]).astype(np.int64)
        self.perm = rng.permutation(self.total_pages).astype(np.int32)  # page table = a random permutation of the pool
        self.k_scale = rng.uniform(0.01, 0.1, HKV).astype(np.float32)
        self.v_scale = rng.uniform(0.01, 0.1, HKV).astype(np.float32)

    # ---- geometry ----
    def global_pages(self, i: int) -> np.ndarray:
        """Physical page ids of sequence i in the whole-batch pool."""
        return self.perm[self.page_start[i]:self.page_start[i + 1]]

    def shard_tables(self, seqs) -> tuple[np.ndarray, int]:
        """Page table [len(seqs), maxPages] and page count of a pool that holds only `seqs`: each page keeps its relative
        position among the shard's pages, so the shard's table is again a random permutation of its (smaller) pool."""
        seqs = list(seqs)
        ids = np.concatenate([self.global_pages(i) for i in seqs]) if seqs else np.zeros(0, np.int32)
        if len(seqs) == self.batch:
            local, count = ids, self.total_pages
        else:
            local = np.empty(ids.size, np.int32)
            local[np.argsort(ids, kind="stable")] = np.arange(ids.size, dtype=np.int32)
            count = int(ids.size)
        max_pages = int(max([self.pages_per[i] for i in seqs] + [1]))
        table = np.zeros((len(seqs), max_pages), np.int32)
        at = 0
        for row, i in enumerate(seqs):
            n = int(self.pages_per[i])
            table[row, :n] = local[at:at + n]
            at += n
        return table, max(count, 1)

    def algorithmic_bytes(self, seqs=None, esize: int = 2) -> int:
        """K and V of every live token once, q and out rows, page-table entries [, scales]."""
        idx = np.arange(self.batch) if seqs is None else np.asarray(list(seqs), dtype=np.int64)
        ctx = self.ctx[idx].astype(np.int64)
        kv = int(ctx.sum()) * INNER * 2 * esize
        qo = len(idx) * HQ * DIM * (2 + 2)
        return kv + qo + 4 * int(self.pages_per[idx].sum()) + (2 * HKV * 4 if esize == 1 else 0)

    # ---- data ----
    def rows(self, i: int) -> int:
        return int(self.pages_per[i]) * PAGE

    def fill_sequence(self, i: int, q_out: np.ndarray, k_out: np.ndarray, v_out: np.ndarray) -> None:
        """Writes the float32 draws of sequence i into caller-owned buffers (q [HQ*DIM], k/v [rows(i), INNER])."""
        rng = np.random.default_rng([self.seed, 1 + i])
        rng.standard_normal(out=q_out, dtype=np.float32)
        rng.standard_normal(out=k_out, dtype=np.float32)
        rng.standard_normal(out=v_out, dtype=np.float32)

    def sequence(self, i: int):
        """(q, k, v) of sequence i as fresh float32 arrays."""
        n = self.rows(i)
        q = np.empty(HQ * DIM, np.float32)
        k = np.empty((n, INNER), np.float32)
        v = np.empty((n, INNER), np.float32)
        self.fill_sequence(i, q, k, v)
        return q, k, v

    def scaled_for_fp8(self, k: np.ndarray, v: np.ndarray):
        """value / per-KV-head scale in float32 (one IEEE division), the number the e4m3 byte is rounded from."""
        ks = np.repeat(self.k_scale, DIM)[None, :]
        vs = np.repeat(self.v_scale, DIM)[None, :]
        return (k / ks).astype(np.float32), (v / vs).astype(np.float32)


def upload_decode(dev, batch: DecodeBatch, seqs, fp8: bool, threads: int | None = None):
    """Builds the device-resident state of a decode step for the sequences `seqs` (a rank's shard, or all of them).

    Returns a dict: k, v (page pools, uint8 views of bf16 / e4m3), table, ctx, q (device) plus their pinned host copies
    table_host, ctx_host, q_host, and total_pages, max_pages.  The float32 draws are generated on host threads into reused
    pinned buffers, copied up, rounded to the storage type by this library's converter and scattered into the pool pages
    named by the page table."""
    import torch

    from puter_b200 import dtypes as D

    seqs = list(seqs)
    threads = threads or host_threads()
    table, count = batch.shard_tables(seqs)
    esize = 1 if fp8 else 2
    page_bytes = PAGE * INNER * esize
    kpool = torch.empty(count * page_bytes, dtype=torch.uint8, device="cuda")
    vpool = torch.empty(count * page_bytes, dtype=torch.uint8, device="cuda")
    if count * page_bytes:
        kpool.zero_()
        vpool.zero_()
    q_host = torch.empty(len(seqs), HQ * DIM, dtype=torch.int16).pin_memory()
    max_rows = max([batch.rows(i) for i in seqs] + [PAGE])
    nbuf = max(2, min(threads, len(seqs), 4))
    stage = [dict(q=torch.empty(HQ * DIM, dtype=torch.float32).pin_memory(),
                  k=torch.empty(max_rows, INNER, dtype=torch.float32).pin_memory(),
                  v=torch.empty(max_rows, INNER, dtype=torch.float32).pin_memory(),
                  ev=torch.cuda.Event()) for _ in range(nbuf)]
    dk = torch.empty(max_rows * INNER, dtype=torch.float32, device="cuda")
    dv = torch.empty(max_rows * INNER, dtype=torch.float32, device="cuda")
    tk = torch.empty(max_rows * INNER * esize, dtype=torch.uint8, device="cuda")
    tv = torch.empty(max_rows * INNER * esize, dtype=torch.uint8, device="cuda")
    ks_row = torch.from_numpy(np.repeat(batch.k_scale, DIM)).cuda()  # per-column divisor of a [rows, INNER] tile
    vs_row = torch.from_numpy(np.repeat(batch.v_scale, DIM)).cuda()
    table_dev = torch.from_numpy(table).cuda()
    store = D.Float8E4M3 if fp8 else D.BFloat16

    def gen(slot, i):
        s = stage[slot]
        n = batch.rows(i)
        batch.fill_sequence(i, s["q"].numpy(), s["k"].numpy()[:n], s["v"].numpy()[:n])
        return slot, i, n

    with ThreadPoolExecutor(nbuf) as pool:
        pending = []
        order = list(enumerate(seqs))
        nxt = 0

        def submit():
            nonlocal nxt
            if nxt < len(order):
                row, i = order[nxt]
                slot = nxt % nbuf
                stage[slot]["ev"].synchronize()  # the previous upload out of this slot has finished
                pending.append((row, pool.submit(gen, slot, i)))
                nxt += 1

        for _ in range(nbuf):
            submit()
        while pending:
            row, fut = pending.pop(0)
            slot, i, n = fut.result()
            s = stage[slot]
            q_host[row].copy_(torch.from_numpy(bf16_bits(s["q"].numpy()).view(np.int16)))
            dk[:n * INNER].copy_(s["k"][:n].view(-1), non_blocking=True)
            dv[:n * INNER].copy_(s["v"][:n].view(-1), non_blocking=True)
            s["ev"].record()
            if fp8:
                dk[:n * INNER].view(n, INNER).div_(ks_row)
                dv[:n * INNER].view(n, INNER).div_(vs_row)
            dev.Convert(tk, dk, n * INNER, store, D.Float32)
            dev.Convert(tv, dv, n * INNER, store, D.Float32)
            pages = table_dev[row, :n // PAGE].long()
            kpool.view(count, page_bytes)[pages] = tk[:n * INNER * esize].view(-1, page_bytes)
            vpool.view(count, page_bytes)[pages] = tv[:n * INNER * esize].view(-1, page_bytes)
            submit()
    torch.cuda.synchronize()
    ctx = np.ascontiguousarray(batch.ctx[seqs]) if seqs else np.zeros(0, np.int32)
    out = dict(k=kpool, v=vpool, total_pages=count, max_pages=table.shape[1],
               table_host=torch.from_numpy(table).pin_memory(), ctx_host=torch.from_numpy(ctx.copy()).pin_memory(), q_host=q_host)
    out["table"], out["ctx"], out["q"] = table_dev, out["ctx_host"].cuda(), q_host.cuda()
    if fp8:
        out["k_scale"] = torch.from_numpy(batch.k_scale).cuda()
        out["v_scale"] = torch.from_numpy(batch.v_scale).cuda()
    return out


# ------------------------------------------------------------------------------------------------------------------
# config 5: add + RMSNorm + gated residual, SwiGLU
# ------------------------------------------------------------------------------------------------------------------
class ChainInputs:
    """x, r, branch [T, C] and gate, up [T, I] in blocks of `BLOCK` token rows (stream ``default_rng([seed, 1 + block])``,
    drawn in that order), gamma [C] and modulation [B, 3C] from ``default_rng(seed)``.  All rounded to bf16."""

    T, C, I, B, BLOCK = 16384, 4096, 14336, 4, 256

    def __init__(self, seed: int = 3, T: int | None = None, C: int | None = None, I: int | None = None, B: int | None = None):
        self.seed = seed
        self.T, self.C, self.I, self.B = T or self.T, C or self.C, I or self.I, B or self.B
        assert self.T % self.BLOCK == 0 and self.T % self.B == 0
        self.rows_per_batch = self.T // self.B
        rng = np.random.default_rng(seed)
        self.gamma = bf16_bits(rng.uniform(0.5, 1.5, self.C).astype(np.float32))
        self.mod = bf16_bits(rng.uniform(0.0, 1.0, (self.B, 3 * self.C)).astype(np.float32))

    def block(self, blk: int, scratch: dict | None = None) -> dict:
        """bf16 bit patterns of the rows [blk*BLOCK, (blk+1)*BLOCK): dict x, r, branch [BLOCK, C], gate, up [BLOCK, I]."""
        rng = np.random.default_rng([self.seed, 1 + blk])
        out = {}
        for name, cols in (("x", self.C), ("r", self.C), ("branch", self.C), ("gate", self.I), ("up", self.I)):
            buf = None if scratch is None else scratch.get(name)
            if buf is None:
                buf = np.empty((self.BLOCK, cols), np.float32)
                if scratch is not None:
                    scratch[name] = buf
            rng.standard_normal(out=buf, dtype=np.float32)
            out[name] = bf16_bits(buf)
        return out

    def rows(self, row_ids) -> dict:
        """The same tensors restricted to the listed global rows (for the oracle side of a test)."""
        row_ids = np.asarray(row_ids, dtype=np.int64)
        res = {k: [] for k in ("x", "r", "branch", "gate", "up")}
        cache = {}
        for rid in row_ids:
            blk = int(rid // self.BLOCK)
            if blk not in cache:
                cache = {blk: self.block(blk)}
            for k in res:
                res[k].append(cache[blk][k][rid % self.BLOCK])
        return {k: np.stack(v) for k, v in res.items()}

    def algorithmic_bytes(self) -> int:
        return 2 * (3 * self.T * self.C + 2 * self.T * self.C) + 2 * (3 * self.T * self.I)


def upload_chain(inp: ChainInputs, row_start: int, row_end: int, threads: int | None = None) -> dict:
    """Device tensors (int16 views of bf16) of the token rows [row_start, row_end), generated block by block on host threads."""
    import torch

    assert row_start % inp.BLOCK == 0 and row_end % inp.BLOCK == 0
    rows = row_end - row_start
    threads = threads or host_threads()
    dev_t = {k: torch.empty(rows, inp.C if k in ("x", "r", "branch") else inp.I, dtype=torch.int16, device="cuda")
             for k in ("x", "r", "branch", "gate", "up")}
    blocks = list(range(row_start // inp.BLOCK, row_end // inp.BLOCK))
    nthr = max(1, min(threads, len(blocks)))
    scratch = [dict() for _ in range(nthr)]
    free = list(range(nthr))

    def gen(blk, slot):
        return blk, slot, inp.block(blk, scratch[slot])

    with ThreadPoolExecutor(nthr) as pool:
        futs = []
        it = iter(blocks)
        for _ in range(nthr):
            b = next(it, None)
            if b is not None:
                futs.append(pool.submit(gen, b, free.pop()))
        while futs:
            blk, slot, data = futs.pop(0).result()
            r0 = blk * inp.BLOCK - row_start
            for k, a in data.items():
                dev_t[k][r0:r0 + inp.BLOCK].copy_(torch.from_numpy(a.view(np.int16)))
            b = next(it, None)
            if b is not None:
                futs.append(pool.submit(gen, b, slot))
    dev_t["gamma"] = torch.from_numpy(inp.gamma.view(np.int16)).cuda()
    dev_t["mod"] = torch.from_numpy(inp.mod.view(np.int16)).cuda()
    torch.cuda.synchronize()
    return dev_t


# ------------------------------------------------------------------------------------------------------------------
# config 3: prefill attention
# ------------------------------------------------------------------------------------------------------------------
class PrefillInputs:
    """q [S, HQ*D], k, v [S, HKV*D] per batch item from ``default_rng([seed, 1 + b])`` (drawn q, k, v), rounded to bf16."""

    B, S, HQ, HKV, D = 4, 4096, 32, 8, 128

    def __init__(self, seed: int = 1, B: int | None = None, S: int | None = None):
        self.seed = seed
        self.B, self.S = B or self.B, S or self.S

    def item(self, b: int) -> dict:
        rng = np.random.default_rng([self.seed, 1 + b])
        out = {}
        for name, heads in (("q", self.HQ), ("k", self.HKV), ("v", self.HKV)):
            out[name] = bf16_bits(rng.standard_normal((self.S, heads * self.D), dtype=np.float32))
        return out

    def flops(self) -> int:
        """Causal: unmasked entries only, QK^T and PV, 2 flops per multiply-add."""
        return 4 * self.B * self.HQ * self.D * (self.S * (self.S + 1) // 2)


def upload_prefill(inp: PrefillInputs, kv_heads=None) -> dict:
    """Device q [B, S, hq*D], k, v [B, S, hkv*D] (int16 views of bf16) holding only the listed KV heads and the query
    heads of their groups, in ascending head order: the pre-sharded slices of one rank (all heads when kv_heads is None)."""
    import torch

    kv_heads = list(range(inp.HKV)) if kv_heads is None else list(kv_heads)
    group = inp.HQ // inp.HKV
    q_heads = [h * group + j for h in kv_heads for j in range(group)]
    D_ = inp.D
    with ThreadPoolExecutor(min(inp.B, host_threads())) as pool:
        items = list(pool.map(inp.item, range(inp.B)))

    def take(a, heads):
        return np.ascontiguousarray(a.reshape(inp.S, -1, D_)[:, heads, :]).reshape(inp.S, len(heads) * D_)

    out = {}
    for name, heads in (("q", q_heads), ("k", kv_heads), ("v", kv_heads)):
        host = np.stack([take(it[name], heads) for it in items])
        out[name] = torch.from_numpy(host.view(np.int16)).cuda()
    out["q_heads"], out["kv_heads"] = q_heads, kv_heads
    return out
