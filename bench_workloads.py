"""Secondary benchmark workloads (the other BASELINE configurations), used by bench.py.

    convert  config 2: dtype conversion sweep over 2^28 elements, six directions, GB/s
    chain    config 5: residual add + RMSNorm + gated residual (fused) and SwiGLU at 8B-class shapes, bf16, GB/s;
             rows are sharded across ranks and the outputs all-gathered over NCCL when world > 1
    prefill  config 3: causal GQA prefill with fused RoPE, bf16, TFLOP/s
"""
from __future__ import annotations

import os
import time

import numpy as np


class ConvertWorkload:
    """Every 8/16-bit pattern tiled to N elements for widening; uniform random 32-bit patterns for narrowing."""

    def __init__(self, dev, rank, n=1 << 28):
        import torch

        from puter_b200 import dtypes as D

        self.torch, self.dev, self.D, self.n = torch, dev, D, n
        self.name = "dtype_convert_sweep"
        self.dtype = "u16/u8<->f32 bit ops"
        g = torch.Generator(device="cuda")
        g.manual_seed(20 + rank)
        self.f32 = torch.randint(-2**31, 2**31 - 1, (n,), dtype=torch.int32, device="cuda", generator=g)
        self.b16 = (torch.arange(n, dtype=torch.int32, device="cuda") & 0xFFFF).to(torch.int16)
        self.b8 = (torch.arange(n, dtype=torch.int32, device="cuda") & 0xFF).to(torch.uint8)
        self.out32 = torch.empty(n, dtype=torch.int32, device="cuda")
        self.out16 = torch.empty(n, dtype=torch.int16, device="cuda")
        self.directions = [(D.BFloat16, D.Float32), (D.Float16, D.Float32), (D.Float8E4M3, D.Float32), (D.Float8E5M2, D.Float32),
                           (D.Float32, D.BFloat16), (D.Float32, D.Float16)]
        self.bytes_per_step = sum(n * (D.SIZE[s] + D.SIZE[d]) for s, d in self.directions)
        self.traffic_ratio = 1.0  # ncu launch list of the sweep: every direction's DRAM bytes equal its algorithmic bytes
        # end to end = the convert package's own call shape: host slices in, host slices out (f32 -> bf16, 2^26 elements)
        self.e2e_n = 1 << 26
        self.src_host = torch.empty(self.e2e_n, dtype=torch.float32).pin_memory()
        self.src_host.copy_(torch.randn(self.e2e_n))
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
        return {"workload": self.name, "elements": self.n, "directions": "bf16,f16,e4m3,e5m2->f32; f32->bf16,f16",
                "l2": "inputs larger than L2 (>= 256 MB per direction)"}

    def metric(self):
        return "convert_hbm_gbps", "GB/s"

    def value(self, sec, world):
        return self.bytes_per_step * world / sec / 1e9

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

    T, C, I, B = 16384, 4096, 14336, 4
    scaling = "strong"  # the 16384 token rows are divided among the ranks

    def __init__(self, dev, rank, world):
        import torch

        from puter_b200 import RMSNormConfig, dtypes as D

        self.torch, self.dev, self.D, self.world, self.rank = torch, dev, D, world, rank
        self.name = "add_rmsnorm_gated_residual_swiglu"
        self.dtype = "bf16"
        assert self.T % world == 0
        self.rows = self.T // world  # strong scaling: token rows are sharded
        self.rpb = self.T // self.B
        g = torch.Generator(device="cuda")
        g.manual_seed(3)
        bf = torch.bfloat16
        r0 = rank * self.rows
        self.x = torch.randn(self.rows, self.C, device="cuda", dtype=bf, generator=g)
        self.r = torch.randn(self.rows, self.C, device="cuda", dtype=bf, generator=g)
        self.branch = torch.randn(self.rows, self.C, device="cuda", dtype=bf, generator=g)
        self.gamma = torch.empty(self.C, device="cuda", dtype=torch.float32).uniform_(0.5, 1.5, generator=g).to(bf)
        # modulation rows for the batch items this rank's rows belong to (batch = global row / rowsPerBatch)
        mod_all = torch.empty(self.B, 3 * self.C, device="cuda", dtype=torch.float32).uniform_(0, 1, generator=g).to(bf)
        first_batch = r0 // self.rpb
        self.mod = mod_all[first_batch:].contiguous()
        self.row_in_batch_offset = r0 % self.rpb
        assert self.row_in_batch_offset == 0 or self.rows <= self.rpb - self.row_in_batch_offset
        self.gate = torch.randn(self.rows, self.I, device="cuda", dtype=bf, generator=g)
        self.up = torch.randn(self.rows, self.I, device="cuda", dtype=bf, generator=g)
        if world > 1:
            # the kernels write this rank's rows straight into their place in the gathered tensors, so the all-gathers run in
            # place (no local copy) and the first two overlap the SwiGLU kernel
            self.n_all = torch.empty(self.T, self.C, device="cuda", dtype=bf)
            self.g_all = torch.empty(self.T, self.C, device="cuda", dtype=bf)
            self.s_all = torch.empty(self.T, self.I, device="cuda", dtype=bf)
            self.n_out, self.g_out, self.s_out = (t[r0:r0 + self.rows] for t in (self.n_all, self.g_all, self.s_all))
        else:
            self.n_out = torch.empty(self.rows, self.C, device="cuda", dtype=bf)
            self.g_out = torch.empty(self.rows, self.C, device="cuda", dtype=bf)
            self.s_out = torch.empty(self.rows, self.I, device="cuda", dtype=bf)
        self.cfg = RMSNormConfig(1e-6)
        self.bytes_per_step_global = 2 * (3 * self.T * self.C + 2 * self.T * self.C) + 2 * (3 * self.T * self.I)
        self.bytes_per_step = self.bytes_per_step_global // world
        # ncu captures of the two kernels: (402.7 + 225.0 + 939.6 + 435.9) MB measured for 671.1 + 1409.3 MB algorithmic (the
        # write counters lag the cache flush)
        self.traffic_ratio = (402.7 + 225.0 + 939.6 + 435.9) / (671.1 + 1409.3)
        self.x_host = self.x.cpu().pin_memory()
        self.n_host = torch.empty(self.rows, self.C, dtype=bf).pin_memory()
        self.h2d, self.d2h = self.x_host.numel() * 2, self.n_host.numel() * 2

    def step(self):
        D = self.D
        # rowsPerBatch: with sharded rows every rank's rows fall inside whole batch items or a fraction of one
        rpb = min(self.rpb, self.rows) if self.rows < self.rpb else self.rpb
        self.dev.AddRMSNormGatedResidual(self.cfg, self.x, self.r, self.gamma, self.branch, self.mod, None, self.n_out, self.g_out,
                                         self.rows, self.C, rpb, 3 * self.C, 0, D.BFloat16)
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
        """Every rank draws the same seeded shard, so after the all-gathers each rank's slice of a gathered tensor must equal
        this rank's own: checks that the in-place, overlapped gathers delivered complete data."""
        if self.world == 1:
            return
        self.step()
        self.torch.cuda.synchronize()
        # (the gated residual depends on the modulation row of the batch item a rank's rows belong to, so only n and s compare)
        for full, mine in ((self.n_all, self.n_out), (self.s_all, self.s_out)):
            for r in range(self.world):
                if not self.torch.equal(full[r * self.rows:(r + 1) * self.rows], mine):
                    raise RuntimeError("chain workload: gathered rows of rank %d differ from the local result" % r)

    def step_e2e(self):
        self.x.copy_(self.x_host, non_blocking=True)
        self.step()
        self.n_host.copy_(self.n_out, non_blocking=True)

    def config(self):
        return {"workload": self.name, "tokens": self.T, "hidden": self.C, "intermediate": self.I, "rows_per_rank": self.rows,
                "collective": "nccl all_gather of n,g,s, in place, n and g overlapped with the SwiGLU kernel" if self.world > 1 else "none",
                "l2": "inputs larger than L2 (2.08 GB per step)"}

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
        rows = self.T
        rng = np.random.default_rng(3)
        mk = lambda *s: O.from_f32(rng.standard_normal(s, dtype=np.float32), O.BF16)
        x, r, br = mk(rows, self.C), mk(rows, self.C), mk(rows, self.C)
        gamma = O.from_f32(rng.uniform(0.5, 1.5, self.C).astype(np.float32), O.BF16)
        mod = O.from_f32(rng.uniform(0, 1, 3 * self.C).astype(np.float32), O.BF16)
        gate, up = mk(rows, self.I), mk(rows, self.I)
        t0 = time.perf_counter()
        h = O.binary(O.ADD, O.BF16, x, r)
        O.rmsnorm(O.BF16, h, gamma, 1e-6)
        O.gated_residual(O.BF16, h, br, mod, rows, self.C, rows, 3 * self.C, 0)
        O.gated_tensors(O.SWIGLU, O.BF16, gate, up)
        dt = time.perf_counter() - t0
        nbytes = 2 * (5 * rows * self.C) + 2 * (3 * rows * self.I)
        return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                "sample": f"all {rows} token rows, the four unfused ops, {dt:.2f} s"}


class PrefillWorkload:
    """Config 3: causal GQA prefill, bf16, RoPE (theta 5e5, half mode) fused, B=4, S=4096, 32/8 heads, head_dim 128."""

    B, S, HQ, HKV, D_ = 4, 4096, 32, 8, 128

    def __init__(self, dev, rank, world):
        self.B = int(os.environ.get("PUTER_BENCH_PREFILL_BATCH", self.B))  # profiler captures use a single batch item
        import torch

        from puter_b200 import MultiHeadAttentionConfig, RoPEConfig, dtypes as D

        self.torch, self.dev, self.D, self.world = torch, dev, D, world
        self.name = "prefill_causal_gqa_rope"
        self.dtype = "bf16"
        g = torch.Generator(device="cuda")
        g.manual_seed(1 + 1000 * rank)
        bf = torch.bfloat16
        self.q = torch.randn(self.B, self.S, self.HQ * self.D_, device="cuda", dtype=bf, generator=g)
        self.k = torch.randn(self.B, self.S, self.HKV * self.D_, device="cuda", dtype=bf, generator=g)
        self.v = torch.randn(self.B, self.S, self.HKV * self.D_, device="cuda", dtype=bf, generator=g)
        self.o = torch.empty_like(self.q)
        self.rope = RoPEConfig(BaseFreq=500000.0, Mode=1)
        self.attn = MultiHeadAttentionConfig(NumHeads=self.HQ, HeadDim=self.D_, Causal=True, KVHeadCount=self.HKV)
        self.flops = 4 * self.B * self.HQ * self.D_ * (self.S * (self.S + 1) // 2)
        self.bytes_per_step = (2 * self.q.numel() + 2 * self.k.numel()) * 2
        self.q_host = self.q.cpu().pin_memory()
        self.k_host = self.k.cpu().pin_memory()
        self.v_host = self.v.cpu().pin_memory()
        self.o_host = torch.empty(self.o.shape, dtype=bf).pin_memory()
        self.h2d = (self.q.numel() + 2 * self.k.numel()) * 2
        self.d2h = self.o.numel() * 2

    def step(self):
        self.dev.RoPEAttentionPrefill(self.rope, self.attn, self.q, self.k, self.v, self.o, self.B, self.S, self.D.BFloat16)

    def step_e2e(self):
        self.q.copy_(self.q_host, non_blocking=True)
        self.k.copy_(self.k_host, non_blocking=True)
        self.v.copy_(self.v_host, non_blocking=True)
        self.dev.RoPEAttentionPrefill(self.rope, self.attn, self.q, self.k, self.v, self.o, self.B, self.S, self.D.BFloat16)
        self.o_host.copy_(self.o, non_blocking=True)

    def config(self):
        return {"workload": self.name, "batch": self.B, "seq_len": self.S, "query_heads": self.HQ, "kv_heads": self.HKV,
                "head_dim": self.D_, "rope": "theta 5e5, half mode, fused", "flops": "causal 4*B*Hq*D*S(S+1)/2",
                "l2": "inputs larger than L2 (q,k,v,out = %d MB per step)" % ((2 * self.q.numel() + 2 * self.k.numel()) * 2 >> 20)}

    def cpu_baseline(self):
        """The CPU path on a bounded sample of config 3: RoPE of q and k of one batch item, then MultiHeadAttention on every 16th
        query row of every head (the causal FLOPs of those rows are what is counted)."""
        import oracle as O

        O.build()
        threads = os.cpu_count() or 1
        O.set_threads(threads)
        rng = np.random.default_rng(1)
        S, HQ, HKV, Dh = self.S, self.HQ, self.HKV, self.D_
        q = O.from_f32(rng.standard_normal((S, HQ * Dh), dtype=np.float32), O.BF16)
        k = O.from_f32(rng.standard_normal((S, HKV * Dh), dtype=np.float32), O.BF16)
        v = O.from_f32(rng.standard_normal((S, HKV * Dh), dtype=np.float32), O.BF16)
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
        return self.flops * world / sec / 1e12

    def extra(self, sec, world):
        return {"tokens_per_s": self.B * self.S * world / sec}

    def roofline(self, sec, peaks):
        ach = self.flops / sec / 1e12
        return {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"],
                # ncu capture of the batch-1 case: 52.5 MB read + 4.5 MB written per batch item (K/V re-reads hit in L2)
                "traffic": 57.0e6 * self.B, "traffic_note": "bytes per step, scaled from the batch-1 ncu capture",
                "peak_source": peaks["source"],
                "note": "causal FLOPs / CUDA-event time of the step (K rotation pre-pass + attention kernel)"}


def make_workload(name, dev, rank, decode_cls):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if name == "decode":
        return decode_cls(dev, rank, fp8=False)
    if name == "decode_fp8":
        return decode_cls(dev, rank, fp8=True)
    if name == "convert":
        return ConvertWorkload(dev, rank)
    if name == "chain":
        return ChainWorkload(dev, rank, world)
    if name == "prefill":
        return PrefillWorkload(dev, rank, world)
    raise ValueError(name)


def secondary_lines(dev, rank, world, timed, peaks, decode_cls, free=()):
    """Short measurements of the other configurations, reported beside the headline line (N = 1 only)."""
    import torch

    if world != 1:
        return None
    for w in free:  # release the headline workload's device memory first
        for k in list(vars(w)):
            if isinstance(getattr(w, k), torch.Tensor):
                setattr(w, k, None)
    torch.cuda.empty_cache()
    out = {}
    for name in ("decode_fp8", "prefill", "chain", "convert"):
        try:
            wl = make_workload(name, dev, rank, decode_cls)
            for _ in range(3):
                wl.step()
            steps = 10
            l0 = dev.launch_count()
            sec, _ = timed(wl.step, steps)
            per = sec / steps
            metric, unit = wl.metric()
            val = wl.value(per, world)
            entry = {"metric": metric, "value": val, "unit": unit, "ms_per_step": per * 1e3, "steps": steps,
                     "gpu_launches": int(dev.launch_count() - l0), "config": wl.config()}
            if unit == "GB/s":
                entry["roofline_frac"] = val / peaks["hbm_gbs"]
            else:
                entry["roofline_frac"] = val / peaks["bf16_tflops"]
            entry.update(wl.extra(per, world))
            out[name] = entry
            del wl
            torch.cuda.empty_cache()
        except Exception as e:  # a secondary workload must never take the headline number down with it
            out[name] = {"error": str(e)[:300]}
            torch.cuda.empty_cache()
    return out
