#!/usr/bin/env python
"""Benchmark of the hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|decode_fp8|prefill|convert|chain]
                    [--impl ours|reference]

Default workload = paged decode attention (batch 64, 32 query heads, 8 KV heads, head_dim 128, contexts
~U[512, 32768], page 16, bf16 KV, a random permutation of physical pages): the configuration the headline
metric "decode-attn HBM GB/s" is quoted on.  One step = one decode step over the whole batch.  Prints ONE
JSON line (rank 0).  For N > 1 launch with torchrun: every rank owns its own batch of sequences and page pool
(sequences are independent: no data-path collective; weak scaling).

`--impl reference` times the CPU restatement of the reference's device/cpu path (the Go reference cannot be
built here: no Go toolchain, and its `manifesto` dependency is absent) on a bounded sample of the same
workload with all host threads.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HQ, HKV, DIM, PAGE = 32, 8, 128, 16


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------------------
# clocks sampling (nvidia-smi in the background during the timed region)
# ------------------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20", "-i",
                                          str(self.gpu)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        rows = [r.strip().split(",") for r in open(self.file.name) if r.strip()]
        os.unlink(self.file.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------------------
CTX_RANGE = [512, 32768]  # --ctx-min / --ctx-max shrink the workload for profiler captures only


def decode_context_lengths(seed: int, batch: int = 64):
    rng = np.random.default_rng(seed)
    return rng.integers(CTX_RANGE[0], CTX_RANGE[1], batch, endpoint=True).astype(np.int32)


def decode_bytes(ctx, esize):
    """Algorithmic bytes of one decode step: K and V of every live token once, q and out rows, page-table entries."""
    pages = int(((ctx.astype(np.int64) + PAGE - 1) // PAGE).sum())
    kv = int(ctx.astype(np.int64).sum()) * HKV * DIM * 2 * esize
    qo = len(ctx) * HQ * DIM * (2 + 2)
    scales = 2 * HKV * 4 if esize == 1 else 0
    return kv + qo + 4 * pages + scales


class DecodeWorkload:
    """Config 4: paged decode attention, one new token per sequence."""

    def __init__(self, dev, rank: int, fp8: bool):
        import torch

        from puter_b200 import MultiHeadAttentionConfig, dtypes

        self.torch = torch
        self.dev = dev
        self.fp8 = fp8
        self.name = "paged_decode_fp8kv" if fp8 else "paged_decode_bf16kv"
        self.ctx = decode_context_lengths(2 + 1000 * rank)
        self.batch = len(self.ctx)
        rng = np.random.default_rng(2 + 1000 * rank)
        pages_per = (self.ctx.astype(np.int64) + PAGE - 1) // PAGE
        self.total_pages = int(pages_per.sum())
        self.max_pages = int(pages_per.max())
        perm = rng.permutation(self.total_pages).astype(np.int32)  # page table = a random permutation of the pool
        table = np.zeros((self.batch, self.max_pages), np.int32)
        at = 0
        for b, n in enumerate(pages_per):
            table[b, :n] = perm[at:at + n]
            at += n
        self.table_host = torch.from_numpy(table).pin_memory()
        self.ctx_host = torch.from_numpy(self.ctx.copy()).pin_memory()
        g = torch.Generator(device="cuda")
        g.manual_seed(2 + 1000 * rank)
        elems = self.total_pages * PAGE * HKV * DIM
        self.esize = 1 if fp8 else 2
        self.fmt = dtypes.BFloat16
        self.kvfmt = dtypes.Float8E4M3 if fp8 else dtypes.BFloat16
        if fp8:
            self.kscale = torch.empty(HKV, device="cuda").uniform_(0.01, 0.1, generator=g)
            self.vscale = torch.empty(HKV, device="cuda").uniform_(0.01, 0.1, generator=g)
            # stored byte = e4m3(x / s): generate in chunks to bound the float32 temporaries
            self.k = torch.empty(elems, dtype=torch.float8_e4m3fn, device="cuda")
            self.v = torch.empty(elems, dtype=torch.float8_e4m3fn, device="cuda")
            chunk = PAGE * HKV * DIM * 4096
            srep_k = (1.0 / self.kscale).repeat_interleave(DIM)
            srep_v = (1.0 / self.vscale).repeat_interleave(DIM)
            for dst, srep in ((self.k, srep_k), (self.v, srep_v)):
                for s in range(0, elems, chunk):
                    n = min(chunk, elems - s)
                    x = torch.randn(n, device="cuda", generator=g).view(-1, HKV * DIM) * srep
                    dst[s:s + n] = x.clamp_(-448, 448).to(torch.float8_e4m3fn).view(-1)
        else:
            self.kscale = self.vscale = None
            self.k = torch.randn(elems, device="cuda", dtype=torch.bfloat16, generator=g)
            self.v = torch.randn(elems, device="cuda", dtype=torch.bfloat16, generator=g)
        self.q_host = torch.randn(self.batch, HQ * DIM, dtype=torch.float32).to(torch.bfloat16).pin_memory()
        self.q = self.q_host.cuda()
        self.table = self.table_host.cuda()
        self.ctx_dev = self.ctx_host.cuda()
        self.out = torch.zeros(self.batch, HQ * DIM, dtype=torch.bfloat16, device="cuda")
        self.out_host = torch.zeros(self.batch, HQ * DIM, dtype=torch.bfloat16).pin_memory()
        self.cfg = MultiHeadAttentionConfig(NumHeads=HQ, HeadDim=DIM, Causal=True, KVHeadCount=HKV)
        self.bytes_per_step = decode_bytes(self.ctx, self.esize)
        # DRAM traffic (ncu dram__bytes_read + write) over algorithmic bytes, from the small-case captures summarised in
        # the profiles folder (bf16 and fp8 decode captures); traffic grows in proportion to the tokens read
        self.traffic_ratio = (317.9 + 4.6) / 316.8 if fp8 else (634.7 + 5.7) / 633.6
        self.units_per_step = self.batch  # tokens
        self.h2d = self.q_host.numel() * 2 + self.table_host.numel() * 4 + self.ctx_host.numel() * 4
        self.d2h = self.out_host.numel() * 2
        self.working_set = 2 * elems * self.esize

    def step(self):
        self.dev.PagedDecodeAttention(self.cfg, self.q, self.k, self.v, self.table, self.ctx_dev, self.out, self.batch, self.max_pages,
                                      self.total_pages, PAGE, self.fmt, kvFormat=self.kvfmt, kScale=self.kscale, vScale=self.vscale)

    def step_e2e(self):
        # a decode step as the caller sees it: this step's query rows, page tables and lengths arrive from the host,
        # the attention rows go back; the KV cache is device-resident state, as in the reference's paged-KV design
        self.q.copy_(self.q_host, non_blocking=True)
        self.table.copy_(self.table_host, non_blocking=True)
        self.ctx_dev.copy_(self.ctx_host, non_blocking=True)
        self.step()
        self.out_host.copy_(self.out, non_blocking=True)

    def config(self):
        return {"workload": self.name, "batch": self.batch, "query_heads": HQ, "kv_heads": HKV, "head_dim": DIM, "page_size": PAGE,
                "ctx_len": "U[%d,%d] seed 2" % tuple(CTX_RANGE), "kv_tokens": int(self.ctx.sum()), "kv_dtype": "e4m3+f32 scale" if self.fp8 else "bf16",
                "l2": "inputs larger than L2 (KV pool %.2f GB)" % (self.working_set / 1e9)}

    def metric(self):
        return "decode_attn_hbm_gbps", "GB/s"

    def value(self, seconds_per_step, world):
        return self.bytes_per_step * world / seconds_per_step / 1e9

    def extra(self, seconds_per_step, world):
        return {"tokens_per_s": self.units_per_step * world / seconds_per_step}


def cpu_decode_sample(fp8: bool, nseq: int = 4, threads: int | None = None, repeats: int = 1):
    """Times the CPU oracle (restatement of device/cpu: page_gather + MultiHeadAttention) on the first `nseq`
    sequences of the seeded batch, all host threads.  Returns (GB/s, tokens/s, threads, description)."""
    import oracle as O

    O.build()
    threads = threads or (os.cpu_count() or 1)
    O.set_threads(threads)
    ctx = decode_context_lengths(2)[:nseq]
    rng = np.random.default_rng(2)
    pages_per = (ctx.astype(np.int64) + PAGE - 1) // PAGE
    total = int(pages_per.sum())
    table = np.zeros((nseq, int(pages_per.max())), np.int32)
    perm = rng.permutation(total).astype(np.int32)
    at = 0
    for b, n in enumerate(pages_per):
        table[b, :n] = perm[at:at + n]
        at += n
    shape = (total, PAGE, HKV * DIM)
    kf = rng.standard_normal(shape, dtype=np.float32)
    vf = rng.standard_normal(shape, dtype=np.float32)
    q = O.from_f32(rng.standard_normal((nseq, HQ * DIM), dtype=np.float32), O.BF16)
    ks = vs = None
    if fp8:
        ks = rng.uniform(0.01, 0.1, HKV).astype(np.float32)
        vs = rng.uniform(0.01, 0.1, HKV).astype(np.float32)
        k = O.from_f32((kf.reshape(total, PAGE, HKV, DIM) / ks[None, None, :, None]).reshape(shape), O.E4M3)
        v = O.from_f32((vf.reshape(total, PAGE, HKV, DIM) / vs[None, None, :, None]).reshape(shape), O.E4M3)
        kvdt = O.E4M3
    else:
        k, v = O.from_f32(kf, O.BF16), O.from_f32(vf, O.BF16)
        kvdt = O.BF16
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.paged_decode(O.BF16, kvdt, q, k, v, table, ctx, PAGE, HQ, HKV, DIM, ks, vs)
        best = min(best, time.perf_counter() - t0)
    nbytes = decode_bytes(ctx, 1 if fp8 else 2)
    return (nbytes / best / 1e9, nseq / best, threads,
            f"first {nseq} of the 64 seeded sequences ({int(ctx.sum())} KV tokens), best of {repeats} x {best:.2f} s")


# ------------------------------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """The reference arm: the CPU path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    fp8 = args.workload == "decode_fp8"
    if args.workload not in ("decode", "decode_fp8"):
        # the other workloads time their own bounded CPU sample (the oracle's restatement of the same ops); the classes are
        # not constructed (their constructors allocate on the GPU), only their constants and cpu_baseline() are used
        import bench_workloads as W

        cls, name = {"convert": (W.ConvertWorkload, "dtype_convert_sweep"), "chain": (W.ChainWorkload, "add_rmsnorm_gated_residual_swiglu"),
                     "prefill": (W.PrefillWorkload, "prefill_causal_gqa_rope")}[args.workload]
        wl = object.__new__(cls)
        metric, unit = wl.metric()
        samples = []
        t0 = time.perf_counter()
        for _ in range(max(args.steps, 1)):
            samples.append(wl.cpu_baseline())
        wall = time.perf_counter() - t0
        value = float(np.mean([x["value"] for x in samples]))
        base = dict(samples[-1], value=value)
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": wall / max(args.steps, 1) * 1e3, "higher_is_better": True, "scaling": getattr(cls, "scaling", "weak"),
            "vs_baseline": None, "dtype": "bf16" if args.workload != "convert" else "u8/u16/f32 bit patterns", "data": "synthetic",
            "config": {"workload": name, "sample": base["sample"]}, "cpu_baseline": base,
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0,
            "note": "C++ restatement of puter device/cpu, not the Go binary: no Go toolchain here"}))
        return
    threads = os.cpu_count() or 1
    for _ in range(max(args.warmup, 0)):
        cpu_decode_sample(fp8, nseq=1, threads=threads)
    vals, toks, desc = [], [], ""
    t0 = time.perf_counter()
    for _ in range(args.steps):
        gbs, tps, threads, desc = cpu_decode_sample(fp8, nseq=args.ref_seqs, threads=threads)
        vals.append(gbs)
        toks.append(tps)
    wall = time.perf_counter() - t0
    value = float(np.mean(vals))
    ctx = decode_context_lengths(2)
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": wall / max(args.steps, 1) * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "paged_decode_fp8kv" if fp8 else "paged_decode_bf16kv", "batch": 64, "query_heads": HQ, "kv_heads": HKV,
                   "head_dim": DIM, "page_size": PAGE, "ctx_len": "U[512,32768] seed 2", "kv_tokens": int(ctx.sum()),
                   "kv_dtype": "e4m3+f32 scale" if fp8 else "bf16"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": desc,
                         "tokens_per_s": float(np.mean(toks))},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "C++ restatement of puter device/cpu (page_gather + MultiHeadAttention), not the Go binary: no Go toolchain here",
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="decode", choices=["decode", "decode_fp8", "prefill", "convert", "chain"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-seqs", type=int, default=16, help="sequences in the CPU sample")
    ap.add_argument("--ctx-min", type=int, default=512)
    ap.add_argument("--ctx-max", type=int, default=32768, help="smaller values give a profiler-sized case; not a bench number")
    ap.add_argument("--prefill-batch", type=int, default=4, help="1 gives a profiler-sized prefill case; not a bench number")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true")
    args = ap.parse_args()
    CTX_RANGE[0], CTX_RANGE[1] = args.ctx_min, args.ctx_max
    os.environ["PUTER_BENCH_PREFILL_BATCH"] = str(args.prefill_batch)
    profiling = (args.ctx_min, args.ctx_max) != (512, 32768) or args.prefill_batch != 4
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not profiling else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import puter_b200
    from bench_workloads import make_workload  # noqa: E402  (secondary workloads live beside this file)

    dev = puter_b200.Device(local_rank)
    wl = make_workload(args.workload, dev, rank, DecodeWorkload)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, sample_clocks=False):
        """Times `steps` calls of fn with CUDA events on the launching stream; returns (max-over-ranks seconds, clocks)."""
        sampler = ClockSampler(local_rank) if sample_clocks else None
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        if sampler:
            sampler.start()
            time.sleep(0.15)
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        barrier()
        clocks = sampler.stop() if sampler else None
        sec = start.elapsed_time(stop) / 1e3
        if world > 1:
            t = torch.tensor([sec], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        return sec, clocks

    for _ in range(args.warmup):
        wl.step()
    if hasattr(wl, "verify"):
        wl.verify()  # untimed self-check of the multi-GPU exchange
    launches0 = dev.launch_count()
    sec, clocks = timed(wl.step, args.steps, sample_clocks=True)
    launches = dev.launch_count() - launches0
    per_step = sec / args.steps

    for _ in range(2):
        wl.step_e2e()
    sec_e2e, _ = timed(wl.step_e2e, args.steps)
    per_step_e2e = sec_e2e / args.steps

    peaks = measured_peaks()
    metric, unit = wl.metric()
    value = wl.value(per_step, world)
    roof = wl.roofline(per_step, peaks) if hasattr(wl, "roofline") else None
    if roof is None:
        achieved = wl.bytes_per_step / per_step / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "traffic": (wl.bytes_per_step * wl.traffic_ratio) if getattr(wl, "traffic_ratio", None) else None,
                "traffic_note": "bytes per step: ncu dram read+write of a captured case scaled by algorithmic bytes (see profiles/)",
                "peak_source": peaks["source"],
                "note": "achieved = algorithmic bytes / CUDA-event time of the whole step (all launches of the step); rank-local"}

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": getattr(wl, "scaling", "weak"), "vs_baseline": None,
        "dtype": wl.dtype if hasattr(wl, "dtype") else "bf16", "data": "synthetic", "config": wl.config(), "clocks": clocks,
        "e2e": {"value": getattr(wl, "e2e_value", wl.value)(per_step_e2e, world), "unit": unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                "ms_per_step": per_step_e2e * 1e3},
        "gpu_launches": int(launches), "roofline": roof,
    }
    line.update(wl.extra(per_step, world))

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        if args.workload in ("decode", "decode_fp8"):
            gbs, tps, threads, desc = cpu_decode_sample(args.workload == "decode_fp8", nseq=args.ref_seqs, repeats=3)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": desc, "tokens_per_s": tps}
        elif hasattr(wl, "cpu_baseline"):
            line["cpu_baseline"] = wl.cpu_baseline()

    if not args.no_secondary and args.workload == "decode":
        from bench_workloads import secondary_lines

        sec_lines = secondary_lines(dev, rank, world, timed, peaks, DecodeWorkload, free=[wl])
        if sec_lines:
            line["secondary"] = sec_lines

    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
