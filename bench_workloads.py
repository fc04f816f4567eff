"""Secondary benchmark workloads (the other BASELINE configurations), used by bench.py.

    convert  config 2: dtype conversion sweep over 2^28 elements, six directions, GB/s; elements divided among the ranks
    chain    config 5: residual add + RMSNorm + gated residual (fused) and SwiGLU at 8B-class shapes, bf16, GB/s;
             token rows are divided among the ranks and the outputs all-gathered over NCCL when world > 1
    prefill  config 3: causal GQA prefill with fused RoPE, bf16, TFLOP/s; (batch item, KV head) units divided among the ranks

All of them run ONE seeded global problem (bench_inputs), so the N-GPU numbers are strong scaling.
"""
from __future__ import annotations

import os
import time

import numpy as np

import bench_inputs as BI


class ConvertWorkload:
    """Every 8/16-bit pattern tiled to N elements for widening; uniform random 32-bit patterns for narrowing."""

    dtype = "u16/u8<->f32 bit ops"
    scaling = "strong"
    N = 1 << 28

    @staticmethod
    def static_config(world):
        return {"workload": "dtype_convert_sweep", "elements": ConvertWorkload.N, "directions": "bf16,f16,e4m3,e5m2->f32; f32->bf16,f16",
                "parallelism": "elements over %d GPU(s); no collective" % world, "l2": "inputs larger than L2 (>= 128 MB per direction and rank)"}

    def __init__(self, dev, rank, world):
        import torch

        from puter_b200 import dtypes as D

        self.torch, self.dev, self.D, self.world = torch, dev, D, world
        n = self.n = self.N // world
        first = rank * n
        g = torch.Generator(device="cuda")
        g.manual_seed(20 + rank)
        # narrowing source: uniform random 32-bit patterns (device generator: 2^28 host draws would dominate the run)
        self.f32 = torch.randint(-2**31, 2**31 - 1, (n,), dtype=torch.int32, device="cuda", generator=g)
        self.b16 = ((torch.arange(n, dtype=torch.int64, device="cuda") + first) & 0xFFFF).to(torch.int16)
        self.b8 = ((torch.arange(n, dtype=torch.int64, device="cuda") + first) & 0xFF).to(torch.uint8)
        self.out32 = torch.empty(n, dtype=torch.int32, device="cuda")
        self.out16 = torch.empty(n, dtype=torch.int16, device="cuda")
        self.directions = [(D.BFloat16, D.Float32), (D.Float16, D.Float32), (D.Float8E4M3, D.Float32), (D.Float8E5M2, D.Float32),
                           (D.Float32, D.BFloat16), (D.Float32, D.Float16)]
        self.bytes_per_step = sum(n * (D.SIZE[s] + D.SIZE[d]) for s, d in self.directions)
        self.bytes_per_step_global = self.bytes_per_step * world
        self.traffic_ratio = 1.0  # ncu launch list of the sweep: every direction's DRAM bytes equal its algorithmic bytes
        # end to end = the convert package's own call shape: host slices in, host slices out (f32 -> bf16, 2^26 elements)
        self.e2e_n = (1 << 26) // world
        self.src_host = torch.empty(self.e2e_n, dtype=torch.float32).pin_memory()
        self.src_host.copy_(torch.from_numpy(np.random.default_rng([21, rank]).standard_normal(self.e2e_n, dtype=np.float32)))
        self.dst_host = torch.empty(self.e2e_n, dtype=torch.int16).pin_memory()
        self.h2d, self.d2h = self.e2e_n * 4, self.e2e_n * 2
        self.e2e_bytes = self.e2e_n * 6

    def _src(self, dt):
        D = self.D
        return self.f32 if dt == D.Float32 else (self.b16 if D.SIZE[dt] == 2 else self.b8)

    def step(self):
        D = self.D
        for s, d in self.directions:
            dst = self.out32 if d == D.Float32 else self.out16
            self.dev.Convert(dst, self._src(s), self.n, d, s)

    def step_e2e(self):
        D = self.D
        self.dev.ConvertHost(self.dst_host.numpy(), self.src_host.numpy(), D.BFloat16, D.Float32)

    def config(self):
        return self.static_config(self.world)

    def metric(self):
        return "convert_hbm_gbps", "GB/s"

    def value(self, sec, world):
        return self.bytes_per_step_global / sec / 1e9

    def e2e_value(self, sec, world):
        return self.e2e_bytes * world / sec / 1e9

    def extra(self, sec, world):
        return {}

    def cpu_baseline(self):
        import oracle as O

        O.build()
        threads = os.cpu_count() or 1
        O.set_threads(threads)
        n = 1 << 28
        src = np.random.default_rng(20).integers(0, 2**32, n, dtype=np.uint64).astype(np.uint32).view(np.float32)
        t0 = time.perf_counter()
        b = O.convert(src, O.F32, O.BF16)
        O.convert(b, O.BF16, O.F32)
        dt = time.perf_counter() - t0
        return {"value": n * 12 / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                "sample": f"f32->bf16 and bf16->f32 over 2^28 elements, {dt:.2f} s"}


class ChainWorkload:
    """Config 5.  h = x + r; n = RMSNorm(h); g = GatedResidual(h, branch, mod); s = SwiGLU(gate, up)."""

    dtype = "bf16"
    scaling = "strong"  # the token rows are divided among the ranks

    @staticmethod
    def tokens():
        return int(os.environ.get("PUTER_BENCH_CHAIN_TOKENS", BI.ChainInputs.T))

    @staticmethod
    def static_config(world, gather="fused"):
        c = BI.ChainInputs
        coll = "none"
        if world > 1:
            coll = ("all-gather of n,g,s fused into the kernels' stores (plain peer stores over NVLink into every rank's gathered "
                    "tensors) + a one-element all-reduce as the barrier" if gather == "fused" else
                    "nccl all_gather of n,g,s, in place, n and g overlapped with the SwiGLU kernel")
        return {"workload": "add_rmsnorm_gated_residual_swiglu", "tokens": ChainWorkload.tokens(), "hidden": c.C, "intermediate": c.I,
                "parallelism": "token rows over %d GPU(s)" % world, "collective": coll, "l2": "inputs larger than L2 (2.08 GB per step)"}

    def __init__(self, dev, rank, world, gather="fused"):
        import torch

        from puter_b200 import RMSNormConfig, dtypes as D, sharding

        self.torch, self.dev, self.D, self.world, self.rank = torch, dev, D, world, rank
        self.gather = gather if world > 1 else "none"
        inp = self.inp = BI.ChainInputs(T=self.tokens())
        self.T, self.C, self.I = inp.T, inp.C, inp.I
        r0, r1 = sharding.row_shard(self.T, world, rank)
        self.r0, self.rows = r0, r1 - r0
        first, nb, self.local_rpb = sharding.modulation_rows(r0, r1, inp.rows_per_batch)
        t = BI.upload_chain(inp, r0, r1)
        self.x, self.r, self.branch, self.gate, self.up, self.gamma = t["x"], t["r"], t["branch"], t["gate"], t["up"], t["gamma"]
        self.mod = t["mod"][first:first + nb].contiguous()
        i16 = torch.bfloat16  # raw 16-bit storage (NCCL has no int16 collectives)
        if world > 1 and self.gather == "fused":
            # the gathered tensors live in memory every rank of the box can address (CUDA IPC); the kernels write each finished
            # vector into all of them, so no collective moves data: a one-element all-reduce is the closing barrier
            import torch.distributed as dist

            self.shared, self.tables = {}, {}
            for name, cols in (("n", self.C), ("g", self.C), ("s", self.I)):
                mine = dev.alloc_shared(self.T * cols * 2)
                handles = [None] * world
                dist.all_gather_object(handles, mine.handle)
                peers = [mine if r == rank else dev.open_shared(handles[r], mine.nbytes) for r in range(world)]
                self.shared[name], self.tables[name] = mine, peers
            as_t = lambda b, cols: torch.as_tensor(b, device="cuda").view(i16).view(self.T, cols)
            self.n_all, self.g_all, self.s_all = as_t(self.shared["n"], self.C), as_t(self.shared["g"], self.C), as_t(self.shared["s"], self.I)
            self.n_out, self.g_out, self.s_out = (t_[r0:r1] for t_ in (self.n_all, self.g_all, self.s_all))
            self.token = torch.zeros(1, device="cuda")
            dist.barrier()
        elif world > 1:
            # the kernels write this rank's rows straight into their place in the gathered tensors, so the all-gathers run in
            # place (no local copy) and the first two overlap the SwiGLU kernel
            self.n_all = torch.empty(self.T, self.C, device="cuda", dtype=i16)
            self.g_all = torch.empty(self.T, self.C, device="cuda", dtype=i16)
            self.s_all = torch.empty(self.T, self.I, device="cuda", dtype=i16)
            self.n_out, self.g_out, self.s_out = (t_[r0:r1] for t_ in (self.n_all, self.g_all, self.s_all))
        else:
            self.n_out = torch.empty(self.rows, self.C, device="cuda", dtype=i16)
            self.g_out = torch.empty(self.rows, self.C, device="cuda", dtype=i16)
            self.s_out = torch.empty(self.rows, self.I, device="cuda", dtype=i16)
        self.cfg = RMSNormConfig(1e-6)
        self.bytes_per_step_global = inp.algorithmic_bytes()
        self.bytes_per_step = self.bytes_per_step_global // world
        # ncu captures of the two kernels: (402.7 + 225.0 + 939.6 + 435.9) MB measured for 671.1 + 1409.3 MB algorithmic (the
        # write counters lag the cache flush)
        self.traffic_ratio = (402.7 + 225.0 + 939.6 + 435.9) / (671.1 + 1409.3)
        self.x_host = self.x.cpu().pin_memory()
        self.n_host = torch.empty(self.rows, self.C, dtype=i16).pin_memory()
        self.h2d, self.d2h = self.x_host.numel() * 2, self.n_host.numel() * 2

    def step(self):
        D = self.D
        if self.gather == "fused":
            import torch.distributed as dist

            self.dev.AddRMSNormGatedResidualGather(self.cfg, self.x, self.r, self.gamma, self.branch, self.mod, self.tables["n"],
                                                   self.tables["g"], self.world, self.rank, self.rows, self.C, self.local_rpb, 3 * self.C, 0,
                                                   D.BFloat16)
            self.dev.SwiGLUTensorsGather(self.tables["s"], self.world, self.rank, self.gate, self.up, self.rows * self.I, D.BFloat16)
            dist.all_reduce(self.token)  # stream-ordered barrier: when it completes, every rank's rows are in place here
            return
        self.dev.AddRMSNormGatedResidual(self.cfg, self.x, self.r, self.gamma, self.branch, self.mod, None, self.n_out, self.g_out,
                                         self.rows, self.C, self.local_rpb, 3 * self.C, 0, D.BFloat16)
        works = []
        if self.world > 1:
            import torch.distributed as dist

            # in place (input = this rank's slice of the output); asynchronous, so they travel while SwiGLU computes
            works.append(dist.all_gather_into_tensor(self.n_all, self.n_out, async_op=True))
            works.append(dist.all_gather_into_tensor(self.g_all, self.g_out, async_op=True))
        self.dev.SwiGLUTensors(self.s_out, self.gate, self.up, self.rows * self.I, D.BFloat16)
        if self.world > 1:
            works.append(dist.all_gather_into_tensor(self.s_all, self.s_out, async_op=True))
            for w in works:
                w.wait()  # orders the current stream after the collective; no host block

    def verify(self):
        """Checks that the in-place, overlapped gathers delivered complete data: every rank publishes a checksum of its own
        rows of n, g and s, and every rank compares each slice of the gathered tensors with its owner's checksum."""
        if self.world == 1:
            return
        import torch.distributed as dist

        torch = self.torch
        self.step()
        torch.cuda.synchronize()
        mine = torch.stack([t.to(torch.int64).sum() for t in (self.n_out, self.g_out, self.s_out)])
        sums = torch.empty(self.world, 3, dtype=torch.int64, device="cuda")
        dist.all_gather_into_tensor(sums, mine)
        for j, full in enumerate((self.n_all, self.g_all, self.s_all)):
            for r in range(self.world):
                if int(full[r * self.rows:(r + 1) * self.rows].to(torch.int64).sum()) != int(sums[r, j]):
                    raise RuntimeError("chain workload: gathered rows of rank %d differ from what that rank computed" % r)

    def step_e2e(self):
        self.x.copy_(self.x_host, non_blocking=True)
        self.step()
        self.n_host.copy_(self.n_out, non_blocking=True)

    def config(self):
        return self.static_config(self.world, self.gather)

    def metric(self):
        return "norm_swiglu_chain_hbm_gbps", "GB/s"

    def value(self, sec, world):
        return self.bytes_per_step_global / sec / 1e9

    def extra(self, sec, world):
        return {"tokens_per_s": self.T / sec}

    def cpu_baseline(self):
        import oracle as O

        O.build()
        threads = os.cpu_count() or 1
        O.set_threads(threads)
        inp = BI.ChainInputs()
        rows = 2048  # a bounded sample: the first 2048 token rows (8 blocks), all four ops
        blocks = [inp.block(b) for b in range(rows // inp.BLOCK)]
        x, r, br, gate, up = (np.concatenate([b[k] for b in blocks]) for k in ("x", "r", "branch", "gate", "up"))
        t0 = time.perf_counter()
        h = O.binary(O.ADD, O.BF16, x, r)
        O.rmsnorm(O.BF16, h, inp.gamma, 1e-6)
        O.gated_residual(O.BF16, h, br, inp.mod[:1], rows, inp.C, rows, 3 * inp.C, 0)
        O.gated_tensors(O.SWIGLU, O.BF16, gate, up)
        dt = time.perf_counter() - t0
        nbytes = 2 * (5 * rows * inp.C) + 2 * (3 * rows * inp.I)
        return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                "sample": f"the first {rows} of 16384 token rows, the four unfused ops, {dt:.2f} s"}


class PrefillWorkload:
    """Config 3: causal GQA prefill, bf16, RoPE (theta 5e5, half mode) fused, B=4, S=4096, 32/8 heads, head_dim 128."""

    dtype = "bf16"
    scaling = "strong"  # the 32 (batch item, KV head) units are divided among the ranks
    S, HQ, HKV, D_ = 4096, 32, 8, 128

    @staticmethod
    def batch_items():
        return int(os.environ.get("PUTER_BENCH_PREFILL_BATCH", BI.PrefillInputs.B))  # profiler captures use a single batch item

    @staticmethod
    def static_config(world):
        c = PrefillWorkload
        return {"workload": "prefill_causal_gqa_rope", "batch": c.batch_items(), "seq_len": c.S, "query_heads": c.HQ, "kv_heads": c.HKV,
                "head_dim": c.D_, "rope": "theta 5e5, half mode, fused", "flops": "causal 4*B*Hq*D*S(S+1)/2",
                "parallelism": "(batch item, KV head) units over %d GPU(s), unit u on rank u mod N; no collective" % world,
                "l2": "inputs larger than L2 (q,k,v,out = 320 MB per step over all ranks)"}

    def __init__(self, dev, rank, world):
        import torch

        from puter_b200 import MultiHeadAttentionConfig, RoPEConfig, dtypes as D, sharding

        self.torch, self.dev, self.D, self.world = torch, dev, D, world
        self.B = self.batch_items()
        inp = self.inp = BI.PrefillInputs(B=self.B, S=self.S)
        units = sharding.prefill_units(self.B, self.HKV, world, rank)
        heads = sorted({h for _, h in units})
        # unit u = (u // HKV, u % HKV) on rank u % world: for world in {1,2,4,8} a rank owns the same KV heads of every batch item,
        # so its slice is a dense [B, S, heads] problem
        assert sorted(units) == [(b, h) for b in range(self.B) for h in heads], "units of a rank must form a batch x heads block"
        t = BI.upload_prefill(inp, heads)
        self.q, self.k, self.v = t["q"], t["k"], t["v"]
        self.o = torch.empty_like(self.q)
        self.hkv_local = len(heads)
        self.hq_local = len(t["q_heads"])
        self.rope = RoPEConfig(BaseFreq=500000.0, Mode=1)
        self.attn = MultiHeadAttentionConfig(NumHeads=self.hq_local, HeadDim=self.D_, Causal=True, KVHeadCount=self.hkv_local)
        self.flops_global = inp.flops()
        self.flops = self.flops_global * self.hq_local // self.HQ
        self.bytes_per_step = (2 * self.q.numel() + 2 * self.k.numel()) * 2
        self.q_host = self.q.cpu().pin_memory()
        self.k_host = self.k.cpu().pin_memory()
        self.v_host = self.v.cpu().pin_memory()
        self.o_host = torch.empty(self.o.shape, dtype=self.o.dtype).pin_memory()
        self.h2d = (self.q.numel() + 2 * self.k.numel()) * 2
        self.d2h = self.o.numel() * 2

    def step(self):
        self.dev.RoPEAttentionPrefill(self.rope, self.attn, self.q, self.k, self.v, self.o, self.B, self.S, self.D.BFloat16)

    def step_e2e(self):
        self.q.copy_(self.q_host, non_blocking=True)
        self.k.copy_(self.k_host, non_blocking=True)
        self.v.copy_(self.v_host, non_blocking=True)
        self.step()
        self.o_host.copy_(self.o, non_blocking=True)

    def config(self):
        return self.static_config(self.world)

    def cpu_baseline(self):
        """The CPU path on a bounded sample of config 3: RoPE of q and k of one batch item, then MultiHeadAttention on every 16th
        query row of every head (the causal FLOPs of those rows are what is counted)."""
        import oracle as O

        O.build()
        threads = os.cpu_count() or 1
        O.set_threads(threads)
        S, HQ, HKV, Dh = self.S, self.HQ, self.HKV, self.D_
        item = BI.PrefillInputs().item(0)
        q, k, v = item["q"], item["k"], item["v"]
        rows = np.repeat(np.arange(7, S, 16, dtype=np.int32), HQ)
        heads = np.tile(np.arange(HQ, dtype=np.int32), S // 16)
        flops = 4.0 * Dh * float((rows.astype(np.int64) + 1).sum())
        t0 = time.perf_counter()
        qr = O.rope(O.BF16, q, S, HQ, Dh, base=500000.0, mode=1)
        kr = O.rope(O.BF16, k, S, HKV, Dh, base=500000.0, mode=1)
        O.mha_rows(O.BF16, qr, kr, v, S, S, HQ, HKV, Dh, rows, heads, True)
        dt = time.perf_counter() - t0
        return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": f"one batch item: RoPE(q), RoPE(k), then every 16th query row of all {HQ} heads ({flops:.3g} causal FLOPs) in {dt:.2f} s"}

    def metric(self):
        return "prefill_attn_tflops", "TFLOP/s"

    def value(self, sec, world):
        return self.flops_global / sec / 1e12

    def extra(self, sec, world):
        return {"tokens_per_s": self.B * self.S / sec}

    def roofline(self, sec, peaks):
        ach = self.flops / sec / 1e12
        return {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"],
                # ncu capture of the batch-1 case: 52.5 MB read + 4.5 MB written per batch item (K/V re-reads hit in L2)
                "traffic": 57.0e6 * self.B * self.hq_local / self.HQ, "traffic_note": "bytes per step, scaled from the batch-1 ncu capture",
                "peak_source": peaks["source"],
                "note": "this rank's causal FLOPs / CUDA-event time of the step (K rotation pre-pass + attention kernel)"}


def make_workload(name, dev, rank, world, decode_cls):
    if name == "decode":
        return decode_cls(dev, rank, world, fp8=False)
    if name == "decode_fp8":
        return decode_cls(dev, rank, world, fp8=True)
    if name == "convert":
        return ConvertWorkload(dev, rank, world)
    if name == "chain":
        return ChainWorkload(dev, rank, world)
    if name == "chain_nccl":
        return ChainWorkload(dev, rank, world, gather="nccl")
    if name == "prefill":
        return PrefillWorkload(dev, rank, world)
    raise ValueError(name)


def row_ops_lines(dev, peaks, rows=16384, cols=4096, reps=20, warmup=3):
    """The sibling row operators beside config 5's chain (plain RMSNorm, the LayerNorm family with its fused residual form,
    row softmax / log-softmax) on the chain's row shape, bf16 and float32: CUDA-event time per call over `reps` calls after
    `warmup` untimed calls, inputs (134 / 268 MB per tensor) larger than L2.  One GPU; the operators are row-wise and shard by rows
    like the chain.  Algorithmic bytes: one read and one write of the rows (plus the residual rows for the fused entry)."""
    import torch

    import puter_b200
    from puter_b200 import dtypes as D

    def per_call(fn):
        for _ in range(warmup):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps / 1e3

    gen = torch.Generator(device="cuda").manual_seed(5)
    out = {"shape": [rows, cols], "unit": "GB/s", "peak": peaks["hbm_gbs"]}
    for tdt, name, es, fmt in ((torch.bfloat16, "bf16", 2, D.BFloat16), (torch.float32, "f32", 4, D.Float32)):
        x = torch.randn(rows, cols, device="cuda", generator=gen).to(tdt)
        res = torch.randn(rows, cols, device="cuda", generator=gen).to(tdt)
        scale = (torch.rand(cols, device="cuda", generator=gen) + 0.5).to(tdt)
        bias = torch.randn(cols, device="cuda", generator=gen).to(tdt)
        mod = (torch.randn(4, 3 * cols, device="cuda", generator=gen) * 0.1).to(tdt)
        o = torch.empty_like(x)
        rpb = rows // 4
        rms = puter_b200.RMSNormConfig(1e-6)
        ops = {
            "rmsnorm": (2, lambda: dev.RMSNorm(rms, x, scale, o, rows, cols, fmt)),
            "layernorm": (2, lambda: dev.LayerNorm(x, scale, bias, o, rows, cols, fmt)),
            "layernorm_residual": (3, lambda: dev.LayerNormResidual(x, scale, bias, res, o, rows, cols, fmt)),
            "adaptive_rmsnorm": (2, lambda: dev.AdaptiveRMSNorm(rms, x, mod, o, rows, cols, rpb, 3 * cols, fmt)),
            "modulated_layernorm": (2, lambda: dev.ModulatedLayerNorm(puter_b200.ModulatedLayerNormConfig(1e-6, 0), x, mod, o, rows, cols,
                                                                     rpb, 3 * cols, fmt)),
            "softmax": (2, lambda: dev.SoftmaxRows(o, x, rows, cols, fmt)),
            "log_softmax": (2, lambda: dev.SoftmaxRows(o, x, rows, cols, fmt, log=True)),
        }
        for op, (tensors, fn) in ops.items():
            sec = per_call(fn)
            gbs = tensors * rows * cols * es / sec / 1e9
            out[f"{op}_{name}"] = {"value": gbs, "ms": sec * 1e3, "roofline_frac": gbs / peaks["hbm_gbs"]}
        del x, res, o
        torch.cuda.empty_cache()
    # the other streaming operators of the path on shapes of the same 8B-class layer, bf16: element-wise add and the gated
    # residual on the chain's rows, a table-driven unary activation, standalone RoPE over [rows, 32 heads, 128], and the paged
    # KV write / gather of K rows ([8 x rows, 8 KV heads x 128], page 16, pages in a random permutation)
    tdt, fmt, es = torch.bfloat16, D.BFloat16, 2
    n = rows * cols
    a = torch.randn(rows, cols, device="cuda", generator=gen).to(tdt)
    b = torch.randn(rows, cols, device="cuda", generator=gen).to(tdt)
    o = torch.empty_like(a)
    mod = (torch.randn(4, 3 * cols, device="cuda", generator=gen) * 0.1).to(tdt)
    inner, page = 1024, 16
    prow = rows * 8  # 131072 token rows of K: 268 MB, larger than L2
    pages = prow // page
    vals = torch.randn(prow, inner, device="cuda", generator=gen).to(tdt)
    perm = torch.randperm(pages, device="cuda", generator=gen).to(torch.int32)
    ids = perm[torch.arange(prow, device="cuda") // page].contiguous()
    offs = (torch.arange(prow, device="cuda") % page).to(torch.int32).contiguous()
    storage = torch.zeros(pages * page, inner, device="cuda", dtype=tdt)
    gathered = torch.empty_like(vals)
    rope_cfg = puter_b200.RoPEConfig()
    stream = {
        "add_bf16": (3 * n * es, lambda: dev.Add(o, a, b, n, fmt)),
        "gated_residual_bf16": (3 * n * es, lambda: dev.GatedResidual(a, b, mod, o, rows, cols, rows // 4, 3 * cols, 0, fmt)),
        "silu_bf16": (2 * n * es, lambda: dev.Silu(o, a, n, fmt)),
        "rope_bf16": (2 * n * es, lambda: dev.RoPE(rope_cfg, a, o, rows, cols // 128, 128, fmt)),
        "kv_page_write_bf16": (2 * prow * inner * es, lambda: dev.KVPageWrite(storage, vals, ids, offs, storage, pages, page, inner, prow, 0, fmt)),
        "kv_page_gather_bf16": (2 * prow * inner * es, lambda: dev.KVPageGather(storage, perm, gathered, pages, page, inner, prow, 0, fmt)),
    }
    # the KV-cache producer on the same rows: RoPE(k) at per-row positions, then the paged write of K and V (2 in, 2 out)
    vvals = torch.randn(prow, inner, device="cuda", generator=gen).to(tdt)
    vstorage = torch.zeros(pages * page, inner, device="cuda", dtype=tdt)
    positions = (torch.arange(prow, device="cuda") % 32768).to(torch.int32).contiguous()
    stream["rope_kv_page_write_bf16"] = (4 * prow * inner * es, lambda: dev.RoPEKVPageWrite(
        rope_cfg, vals, vvals, positions, ids, offs, storage, vstorage, prow, inner // 128, 128, pages, page, 32768, fmt))
    # SwiGLU in the reference's packed form: rows of [gate | up], the 8B-class MLP width, a quarter of the chain's rows
    prows, phalf = rows // 4, 14336
    packed = torch.randn(prows, 2 * phalf, device="cuda", generator=gen).to(tdt)
    pout = torch.empty(prows, phalf, device="cuda", dtype=tdt)
    stream["swiglu_packed_bf16"] = (3 * prows * phalf * es, lambda: dev.SwiGLU(pout, packed, prows, phalf, fmt))
    for op, (nbytes, fn) in stream.items():
        sec = per_call(fn)
        gbs = nbytes / sec / 1e9
        out[op] = {"value": gbs, "ms": sec * 1e3, "roofline_frac": gbs / peaks["hbm_gbs"]}
    out["error_flag"] = int(dev.take_error())
    return out


def secondary_lines(dev, rank, world, timed, peaks, decode_cls, replica_cls, free=()):
    """Short measurements of the other configurations, reported beside the headline line.  For N > 1 every entry is the
    strong-scaling split of the one seeded problem; `weak_replicas` repeats the earlier every-rank-runs-everything decode
    measurement under its own label."""
    import torch

    for w in free:  # release the headline workload's device memory first
        for k in list(vars(w)):
            v = getattr(w, k)
            if isinstance(v, torch.Tensor) or isinstance(v, dict):
                setattr(w, k, None)
    torch.cuda.empty_cache()
    out = {}
    names = ["decode_fp8", "prefill", "chain", "convert"] + (["chain_nccl", "weak_replicas"] if world > 1 else [])
    for name in names:
        try:
            wl = replica_cls(dev, rank, world) if name == "weak_replicas" else make_workload(name, dev, rank, world, decode_cls)
            for _ in range(3):
                wl.step()
            if hasattr(wl, "verify"):
                wl.verify()
            steps = 10
            l0 = dev.launch_count()
            sec, _, per_rank = timed(wl.step, steps)
            per = sec / steps
            if name == "weak_replicas":
                val = wl.bytes_per_step * world / per / 1e9
                out[name] = {"metric": "decode_attn_hbm_gbps", "value": val, "unit": "GB/s", "ms_per_step": per * 1e3, "steps": steps,
                             "scaling": "weak", "note": "every rank runs its own full 64-sequence batch; value = N x bytes / time"}
            else:
                metric, unit = wl.metric()
                val = wl.value(per, world)
                entry = {"metric": metric, "value": val, "unit": unit, "ms_per_step": per * 1e3, "steps": steps, "scaling": wl.scaling,
                         "gpu_launches": int(dev.launch_count() - l0), "config": wl.config(),
                         "ms_per_step_per_rank": [t / steps * 1e3 for t in per_rank]}
                entry["roofline_frac"] = val / world / (peaks["hbm_gbs"] if unit == "GB/s" else peaks["bf16_tflops"])
                entry.update(wl.extra(per, world))
                out[name] = entry
            del wl
            torch.cuda.empty_cache()
        except Exception as e:  # a secondary workload must never take the headline number down with it
            out[name] = {"error": str(e)[:300]}
            torch.cuda.empty_cache()
    if world == 1:
        try:
            out["row_ops"] = row_ops_lines(dev, peaks)
        except Exception as e:
            out["row_ops"] = {"error": str(e)[:300]}
            torch.cuda.empty_cache()
    return out
