#!/usr/bin/env python
"""Benchmark of the hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|decode_fp8|prefill|convert|chain]
                    [--impl ours|reference]

Default workload = paged decode attention (batch 64, 32 query heads, 8 KV heads, head_dim 128, contexts
~U[512, 32768], page 16, bf16 KV, a random permutation of physical pages): the configuration the headline
metric "decode-attn HBM GB/s" is quoted on.  One step = one decode step over the whole batch.  Prints ONE
JSON line (rank 0).

For N > 1 launch with torchrun.  The ONE seeded batch is divided among the ranks: whole sequences, assigned
longest first to the least loaded rank, then balanced by exchanges; each rank holds only the KV pages of its own sequences and there is no
data-path collective (strong scaling: value = bytes of the whole batch / slowest rank's time).

`--impl reference` times the CPU restatement of the reference's device/cpu path (the Go reference cannot be
built here: no Go toolchain, and its `manifesto` dependency is absent) on a bounded sample of the same
workload with all host threads.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench_inputs as BI  # noqa: E402

HQ, HKV, DIM, PAGE = BI.HQ, BI.HKV, BI.DIM, BI.PAGE
CTX_RANGE = [512, 32768]  # --ctx-min / --ctx-max shrink the workload for profiler captures only


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
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
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

    @staticmethod
    def _when(text: str):
        """nvidia-smi's timestamp (local time, milliseconds) as seconds since the epoch; None if it does not parse."""
        try:
            return datetime.datetime.strptime(text.strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self, window=None):
        """Median SM clock, maximum power and the throttle reasons seen.  `window` = (t0, t1) in time.time() seconds keeps
        only the samples taken while the measured loop was running (the sampler starts before it and stops after it)."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "power_w_max": None}
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
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            if window is not None:
                when = self._when(r[0])
                if when is not None and not (window[0] <= when <= window[1]):
                    continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                pw.append(float(r[3]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm),
                       power_w_max=float(max(pw)))
        return out


# ------------------------------------------------------------------------------------------------------------
# config 4: paged decode attention
# ------------------------------------------------------------------------------------------------------------
def decode_batch() -> BI.DecodeBatch:
    return BI.DecodeBatch(seed=2, batch=64, ctx_min=CTX_RANGE[0], ctx_max=CTX_RANGE[1])


def decode_config(batch: BI.DecodeBatch, fp8: bool, world: int) -> dict:
    """The config dict both arms print (identical for a given N)."""
    esize = 1 if fp8 else 2
    return {"workload": "paged_decode_fp8kv" if fp8 else "paged_decode_bf16kv", "batch": batch.batch, "query_heads": HQ, "kv_heads": HKV,
            "head_dim": DIM, "page_size": PAGE, "ctx_len": "U[%d,%d] seed 2" % tuple(CTX_RANGE), "kv_tokens": int(batch.ctx.sum()),
            "kv_dtype": "e4m3+f32 scale" if fp8 else "bf16",
            "parallelism": "whole sequences over %d GPU(s), longest first to the least loaded, then balanced by exchanges; no collective" % world,
            "l2": "inputs larger than L2 (KV pools %.2f GB)" % (2 * int(batch.pages_per.sum()) * PAGE * BI.INNER * esize / 1e9)}


class DecodeWorkload:
    """Config 4: paged decode attention, one new token per sequence; this rank's share of the seeded batch."""

    scaling = "strong"

    def __init__(self, dev, rank: int, world: int, fp8: bool):
        import torch

        from puter_b200 import MultiHeadAttentionConfig, dtypes, sharding

        self.torch, self.dev, self.fp8, self.world, self.rank = torch, dev, fp8, world, rank
        self.data = decode_batch()
        self.owned_all = sharding.lpt_assign(self.data.ctx, world)
        self.owned = self.owned_all[rank]
        self.esize = 1 if fp8 else 2
        st = BI.upload_decode(dev, self.data, self.owned, fp8)
        self.st = st
        self.batch = len(self.owned)
        self.fmt = dtypes.BFloat16
        self.kvfmt = dtypes.Float8E4M3 if fp8 else dtypes.BFloat16
        self.k, self.v = st["k"], st["v"]
        self.kscale, self.vscale = st.get("k_scale"), st.get("v_scale")
        self.total_pages, self.max_pages = st["total_pages"], st["max_pages"]
        # this step's host inputs (query rows, page tables, lengths) live in ONE pinned buffer and reach the device in one copy;
        # two device copies of it and of the output alternate, so that the copies of step i+1 / i-1 travel on their own
        # streams while step i computes
        qb, tb, cb = st["q_host"].numel() * 2, st["table_host"].numel() * 4, st["ctx_host"].numel() * 4
        off_t = (qb + 255) & ~255
        off_c = (off_t + tb + 255) & ~255
        total = off_c + max(cb, 4)
        self.stage_host = torch.zeros(total, dtype=torch.uint8).pin_memory()
        self.stage_host[:qb].copy_(st["q_host"].view(torch.uint8).view(-1))
        self.stage_host[off_t:off_t + tb].copy_(st["table_host"].view(torch.uint8).view(-1))
        self.stage_host[off_c:off_c + cb].copy_(st["ctx_host"].view(torch.uint8).view(-1))
        self.slots = []
        for _ in range(2):
            sd = torch.zeros(total, dtype=torch.uint8, device="cuda")
            sd.copy_(self.stage_host)
            self.slots.append(dict(
                stage=sd, q=sd[:qb].view(torch.int16).view(self.batch, HQ * DIM),
                table=sd[off_t:off_t + tb].view(torch.int32).view(self.batch, self.max_pages), ctx=sd[off_c:off_c + cb].view(torch.int32),
                out=torch.zeros(self.batch, HQ * DIM, dtype=torch.int16, device="cuda"),
                out_host=torch.zeros(self.batch, HQ * DIM, dtype=torch.int16).pin_memory(),
                ready=torch.cuda.Event(), consumed=torch.cuda.Event(), computed=torch.cuda.Event(), downloaded=torch.cuda.Event()))
        self.up_stream, self.down_stream = torch.cuda.Stream(), torch.cuda.Stream()
        self.e2e_i = 0
        s0 = self.slots[0]
        self.q, self.table, self.ctx_dev, self.out, self.out_host = s0["q"], s0["table"], s0["ctx"], s0["out"], s0["out_host"]
        self.cfg = MultiHeadAttentionConfig(NumHeads=HQ, HeadDim=DIM, Causal=True, KVHeadCount=HKV)
        self.bytes_per_step = self.data.algorithmic_bytes(self.owned, self.esize)       # this rank
        self.bytes_per_step_global = self.data.algorithmic_bytes(None, self.esize)      # the whole batch
        # DRAM traffic (ncu dram__bytes_read + write) over algorithmic bytes, from the small-case captures summarised in
        # the profiles folder (bf16 and fp8 decode captures); traffic grows in proportion to the tokens read
        self.traffic_ratio = (317.5 + 3.8) / 316.8 if fp8 else (634.3 + 4.2) / 633.6
        self.h2d = qb + tb + cb
        self.d2h = self.out_host.numel() * 2
        torch.cuda.synchronize()

    def step(self):
        self.dev.PagedDecodeAttention(self.cfg, self.q, self.k, self.v, self.table, self.ctx_dev, self.out, self.batch, self.max_pages,
                                      self.total_pages, PAGE, self.fmt, kvFormat=self.kvfmt, kScale=self.kscale, vScale=self.vscale)

    def step_e2e(self):
        # a decode step as the caller sees it: this step's query rows, page tables and lengths arrive from the host (one
        # copy), the attention rows go back; the KV cache is device-resident state, as in the reference's paged-KV design.
        # Upload, compute and download run on three streams chained by events, over two alternating buffer sets.
        torch = self.torch
        s = self.slots[self.e2e_i & 1]
        self.e2e_i += 1
        cur = torch.cuda.current_stream()
        with torch.cuda.stream(self.up_stream):
            self.up_stream.wait_event(s["consumed"])      # the step that last read this buffer set has run
            s["stage"].copy_(self.stage_host, non_blocking=True)
            s["ready"].record(self.up_stream)
        cur.wait_event(s["ready"])
        cur.wait_event(s["downloaded"])                    # its previous output rows have left the device
        self.dev.PagedDecodeAttention(self.cfg, s["q"], self.k, self.v, s["table"], s["ctx"], s["out"], self.batch, self.max_pages,
                                      self.total_pages, PAGE, self.fmt, kvFormat=self.kvfmt, kScale=self.kscale, vScale=self.vscale)
        s["consumed"].record(cur)
        with torch.cuda.stream(self.down_stream):
            self.down_stream.wait_event(s["consumed"])
            s["out_host"].copy_(s["out"], non_blocking=True)
            s["downloaded"].record(self.down_stream)

    def e2e_drain(self):
        # inside the timed region: the last steps' output rows must have reached the host before the clock stops
        cur = self.torch.cuda.current_stream()
        for s in self.slots:
            cur.wait_event(s["downloaded"])

    def config(self):
        return decode_config(self.data, self.fp8, self.world)

    def metric(self):
        return "decode_attn_hbm_gbps", "GB/s"

    def value(self, seconds_per_step, world):
        return self.bytes_per_step_global / seconds_per_step / 1e9

    def bytes_per_rank(self):
        return [self.data.algorithmic_bytes(o, self.esize) for o in self.owned_all]

    def extra(self, seconds_per_step, world):
        loads = [int(self.data.ctx[o].sum()) for o in self.owned_all]
        return {"tokens_per_s": self.data.batch / seconds_per_step,
                "partition": {"sequences_per_rank": [len(o) for o in self.owned_all], "kv_tokens_per_rank": loads,
                              "imbalance_max_over_mean": max(loads) / (sum(loads) / len(loads))}}


class ReplicaDecodeWorkload:
    """The earlier weak-scaling measurement, kept as a labelled secondary: every rank runs its own full-size batch
    (device-generated data; nothing is shared or divided)."""

    scaling = "weak"

    def __init__(self, dev, rank: int, world: int):
        import torch

        from puter_b200 import MultiHeadAttentionConfig, dtypes

        self.dev = dev
        data = BI.DecodeBatch(seed=2 + 1000 * rank)
        table, count = data.shard_tables(range(data.batch))
        g = torch.Generator(device="cuda")
        g.manual_seed(2 + 1000 * rank)
        elems = count * PAGE * BI.INNER
        self.k = torch.randn(elems, device="cuda", dtype=torch.bfloat16, generator=g)
        self.v = torch.randn(elems, device="cuda", dtype=torch.bfloat16, generator=g)
        self.q = torch.randn(data.batch, HQ * DIM, device="cuda", dtype=torch.bfloat16, generator=g)
        self.table = torch.from_numpy(table).cuda()
        self.ctx = torch.from_numpy(data.ctx.copy()).cuda()
        self.out = torch.zeros_like(self.q)
        self.cfg = MultiHeadAttentionConfig(NumHeads=HQ, HeadDim=DIM, Causal=True, KVHeadCount=HKV)
        self.args = (data.batch, table.shape[1], count, PAGE, dtypes.BFloat16)
        self.bytes_per_step = data.algorithmic_bytes(None, 2)

    def step(self):
        self.dev.PagedDecodeAttention(self.cfg, self.q, self.k, self.v, self.table, self.ctx, self.out, *self.args)


def cpu_decode_sample(fp8: bool, nseq: int = 16, threads: int | None = None, repeats: int = 1, prepared=None):
    """Times the CPU oracle (restatement of device/cpu: page_gather + MultiHeadAttention) on the first `nseq`
    sequences of the seeded batch.  Returns (GB/s, tokens/s, threads, description, prepared inputs)."""
    import oracle as O

    O.build()
    threads = threads or (os.cpu_count() or 1)
    O.set_threads(threads)
    data = decode_batch()
    if prepared is None:
        seqs = list(range(nseq))
        qs, ks, vs = [], [], []
        for i in seqs:
            q, k, v = data.sequence(i)
            if fp8:
                k, v = data.scaled_for_fp8(k, v)
            qs.append(O.from_f32(q, O.BF16))
            ks.append(O.from_f32(k, O.E4M3 if fp8 else O.BF16))
            vs.append(O.from_f32(v, O.E4M3 if fp8 else O.BF16))
        table, count = data.shard_tables(seqs)
        kp = np.zeros((count, PAGE, BI.INNER), ks[0].dtype)
        vp = np.zeros((count, PAGE, BI.INNER), ks[0].dtype)
        for row, i in enumerate(seqs):
            n = int(data.pages_per[i])
            kp[table[row, :n]] = ks[row].reshape(n, PAGE, BI.INNER)
            vp[table[row, :n]] = vs[row].reshape(n, PAGE, BI.INNER)
        prepared = (np.stack(qs), kp, vp, table, data.ctx[seqs].copy(), seqs)
    q, kp, vp, table, ctx, seqs = prepared
    kvdt = O.E4M3 if fp8 else O.BF16
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.paged_decode(O.BF16, kvdt, q, kp, vp, table, ctx, PAGE, HQ, HKV, DIM, data.k_scale if fp8 else None, data.v_scale if fp8 else None)
        best = min(best, time.perf_counter() - t0)
    nbytes = data.algorithmic_bytes(seqs, 1 if fp8 else 2)
    return (nbytes / best / 1e9, len(seqs) / best, threads,
            f"first {len(seqs)} of the 64 seeded sequences ({int(ctx.sum())} KV tokens), best of {repeats} x {best:.2f} s", prepared)


def cpu_decode_baseline(fp8: bool, nseq: int):
    """All host threads on `nseq` sequences, and one thread (the reference ops are single-goroutine loops) on two of them."""
    gbs, tps, threads, desc, _ = cpu_decode_sample(fp8, nseq=nseq, repeats=3)
    gbs1, tps1, _, desc1, _ = cpu_decode_sample(fp8, nseq=min(2, nseq), threads=1, repeats=1)
    return {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": desc, "tokens_per_s": tps,
            "value_1thread": gbs1, "tokens_per_s_1thread": tps1, "sample_1thread": desc1}


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

        cls = {"convert": W.ConvertWorkload, "chain": W.ChainWorkload, "chain_nccl": W.ChainWorkload, "prefill": W.PrefillWorkload}[args.workload]
        wl = object.__new__(cls)
        wl.world = args.gpus
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
            "ms_per_step": wall / max(args.steps, 1) * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": cls.dtype, "data": "synthetic",
            "config": cls.static_config(args.gpus, "nccl") if args.workload == "chain_nccl" else cls.static_config(args.gpus), "cpu_baseline": base,
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0,
            "note": "C++ restatement of puter device/cpu, not the Go binary: no Go toolchain here"}))
        return
    threads = os.cpu_count() or 1
    prepared = None
    vals, toks, desc = [], [], ""
    for _ in range(max(args.warmup, 0)):
        *_, prepared = cpu_decode_sample(fp8, nseq=args.ref_seqs, threads=threads, prepared=prepared)
    if prepared is None:
        *_, prepared = cpu_decode_sample(fp8, nseq=args.ref_seqs, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        gbs, tps, threads, desc, prepared = cpu_decode_sample(fp8, nseq=args.ref_seqs, threads=threads, prepared=prepared)
        vals.append(gbs)
        toks.append(tps)
    wall = time.perf_counter() - t0
    value = float(np.mean(vals))
    gbs1, tps1, _, desc1, _ = cpu_decode_sample(fp8, nseq=min(2, args.ref_seqs), threads=1)
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": wall / max(args.steps, 1) * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": decode_config(decode_batch(), fp8, args.gpus),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": desc,
                         "tokens_per_s": float(np.mean(toks)), "value_1thread": gbs1, "tokens_per_s_1thread": tps1, "sample_1thread": desc1},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "C++ restatement of puter device/cpu (page_gather + MultiHeadAttention), not the Go binary: no Go toolchain here; "
                "a step is one pass over the sample named in cpu_baseline.sample (a rate, so comparable with the whole batch)",
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="decode", choices=["decode", "decode_fp8", "prefill", "convert", "chain", "chain_nccl", "row_ops"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-seqs", type=int, default=16, help="sequences in the CPU sample")
    ap.add_argument("--ctx-min", type=int, default=512)
    ap.add_argument("--ctx-max", type=int, default=32768, help="smaller values give a profiler-sized case; not a bench number")
    ap.add_argument("--prefill-batch", type=int, default=4, help="1 gives a profiler-sized prefill case; not a bench number")
    ap.add_argument("--chain-tokens", type=int, default=16384, help="fewer token rows give a profiler-sized chain case; not a bench number")
    ap.add_argument("--sustained-seconds", type=float, default=2.0, help="length of the sustained loop of the headline step (0 = skip)")
    ap.add_argument("--clock-window", type=float, default=0.3,
                    help="seconds of the same loop run untimed directly before the timed steps while nvidia-smi samples the clocks")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true")
    args = ap.parse_args()
    CTX_RANGE[0], CTX_RANGE[1] = args.ctx_min, args.ctx_max
    os.environ["PUTER_BENCH_PREFILL_BATCH"] = str(args.prefill_batch)
    os.environ["PUTER_BENCH_CHAIN_TOKENS"] = str(args.chain_tokens)
    profiling = (args.ctx_min, args.ctx_max) != (512, 32768) or args.prefill_batch != 4 or args.chain_tokens != 16384
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
    if args.workload == "row_ops":
        # the sibling row operators on the chain's row shape, one line of per-operator rates (also the `row_ops` entry of the
        # default run's `secondary`); --steps = timed calls per operator, --warmup = untimed calls before them
        from bench_workloads import row_ops_lines

        if rank == 0:
            ops = row_ops_lines(dev, measured_peaks(), reps=max(1, args.steps), warmup=args.warmup)
            print(json.dumps({"metric": "row_ops_hbm_gbps", "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                              "higher_is_better": True, "data": "synthetic", "config": {"workload": "row_ops", "rows": ops["shape"][0],
                                                                                       "cols": ops["shape"][1]},
                              "row_ops": ops}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    wl = make_workload(args.workload, dev, rank, world, DecodeWorkload)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, sample_clocks=False, drain=None):
        """Times `steps` calls of fn with CUDA events on the launching stream; returns (max-over-ranks seconds, clocks,
        per-rank seconds).  `drain` runs after the last call, inside the timed region (work of side streams joins there).
        With sample_clocks the same call is looped for --clock-window seconds (0.3) directly before the timed steps (untimed, the same count on
        every rank): nvidia-smi samples every 20 ms and the timed steps alone can be shorter than that, so the clocks are
        those of the load window that ends with the timed steps."""
        sampler = ClockSampler(local_rank) if sample_clocks else None
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        preroll = 0
        if sampler:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            a.record()
            for _ in range(3):
                fn()
            b.record()
            torch.cuda.synchronize()
            est = torch.tensor([a.elapsed_time(b) / 3e3], device="cuda", dtype=torch.float64)
            if world > 1:
                dist.all_reduce(est, op=dist.ReduceOp.MAX)
            preroll = 0 if profiling else min(20000, int(args.clock_window / max(float(est.item()), 1e-6)) + 1)
        barrier()
        window0 = None
        if sampler:
            sampler.start()
            time.sleep(0.15)
            window0 = time.time() + 0.04  # the first samples after the load starts still see the idle clocks
            for i in range(preroll):
                fn()
                if i % 64 == 63:
                    torch.cuda.synchronize()  # keeps the launch queue short
        launches0 = dev.launch_count()
        start.record()
        for _ in range(steps):
            fn()
        if drain:
            drain()
        stop.record()
        timed.launches = dev.launch_count() - launches0  # kernels of this library launched between the two events
        torch.cuda.synchronize()
        window1 = time.time()
        barrier()
        clocks = sampler.stop((window0, window1)) if sampler else None
        if clocks is not None:
            clocks["window"] = "%d untimed steps of the same loop + the timed steps" % preroll
        sec = start.elapsed_time(stop) / 1e3
        per_rank = [sec]
        if world > 1:
            t = torch.tensor([sec], device="cuda", dtype=torch.float64)
            allt = torch.empty(world, device="cuda", dtype=torch.float64)
            dist.all_gather_into_tensor(allt, t)
            per_rank = [float(x) for x in allt.tolist()]
            sec = max(per_rank)
        return sec, clocks, per_rank

    for _ in range(args.warmup):
        wl.step()
    if hasattr(wl, "verify"):
        wl.verify()  # untimed self-check of the multi-GPU exchange
    sec, clocks, per_rank = timed(wl.step, args.steps, sample_clocks=True)
    launches = timed.launches
    per_step = sec / args.steps

    for _ in range(2):
        wl.step_e2e()
    sec_e2e, _, _ = timed(wl.step_e2e, args.steps, drain=getattr(wl, "e2e_drain", None))
    per_step_e2e = sec_e2e / args.steps

    peaks = measured_peaks()
    metric, unit = wl.metric()
    value = wl.value(per_step, world)
    roof = wl.roofline(per_step, peaks) if hasattr(wl, "roofline") else None
    if roof is None:
        # rank-local: this rank's algorithmic bytes over this rank's own time
        mine = per_rank[rank] / args.steps
        achieved = wl.bytes_per_step / mine / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "traffic": (wl.bytes_per_step * wl.traffic_ratio) if getattr(wl, "traffic_ratio", None) else None,
                "traffic_note": "bytes per step: ncu dram read+write of a captured case scaled by algorithmic bytes",
                "peak_source": peaks["source"],
                "note": "achieved = this rank's algorithmic bytes / CUDA-event time of its whole step (all launches of the step)"}
        if world > 1 and hasattr(wl, "bytes_per_rank"):
            roof["per_rank_frac"] = [b / (t / args.steps) / 1e9 / peaks["hbm_gbs"] for b, t in zip(wl.bytes_per_rank(), per_rank)]

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": getattr(wl, "scaling", "strong"), "vs_baseline": None,
        "dtype": wl.dtype if hasattr(wl, "dtype") else "bf16", "data": "synthetic", "config": wl.config(), "clocks": clocks,
        "e2e": {"value": getattr(wl, "e2e_value", wl.value)(per_step_e2e, world), "unit": unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                "ms_per_step": per_step_e2e * 1e3},
        "gpu_launches": int(launches), "roofline": roof, "ms_per_step_per_rank": [t / args.steps * 1e3 for t in per_rank],
    }
    line.update(wl.extra(per_step, world))

    if args.sustained_seconds > 0 and not profiling:
        # the same step looped for seconds of device time, clocks sampled: what a serving loop sees once the part is warm
        n = max(args.steps, int(args.sustained_seconds / per_step) + 1)
        sec_s, clocks_s, _ = timed(wl.step, n, sample_clocks=True)
        line["sustained"] = {"value": wl.value(sec_s / n, world), "unit": unit, "ms_per_step": sec_s / n * 1e3, "steps": n,
                             "seconds": sec_s, "sm_mhz_median": clocks_s["sm_mhz"], "power_w_max": clocks_s["power_w_max"],
                             "reasons": clocks_s["reasons"], "ms_x_mhz": (sec_s / n * 1e3 * clocks_s["sm_mhz"]) if clocks_s["sm_mhz"] else None}

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        if args.workload in ("decode", "decode_fp8"):
            line["cpu_baseline"] = cpu_decode_baseline(args.workload == "decode_fp8", args.ref_seqs)
        elif hasattr(wl, "cpu_baseline"):
            line["cpu_baseline"] = wl.cpu_baseline()

    if not args.no_secondary and args.workload == "decode" and not profiling:
        from bench_workloads import secondary_lines

        sec_lines = secondary_lines(dev, rank, world, timed, peaks, DecodeWorkload, ReplicaDecodeWorkload, free=[wl])
        if sec_lines:
            line["secondary"] = sec_lines

    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
