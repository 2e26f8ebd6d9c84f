"""Benchmark of the paged KV-cache hot path: KV append + paged decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload at N GPUs: the Qwen3-8B decode shape (32 query / 8 KV heads, head_dim 128,
page 256 tokens, context lengths uniform in [512, 8192], one appended token per sequence),
batch 64*N, KV heads sharded N ways (rank r owns 8/N KV heads and their query heads of
every sequence; page ids, slots and lengths are replicated).  Per-GPU KV bytes are the same
at every N (weak scaling); at N=1 it is exactly the 64-sequence configuration.  A step is
one append (one new row per sequence) followed by one paged decode attention pass.

One JSON line is printed by rank 0:
  value      whole-job KV GB/s: algorithmic KV bytes of all ranks / step time.  The K steps are
             captured as ONE CUDA graph, which is replayed R >= 50 times inside the clock-sampling
             window with an event pair around every replay; the step time is the median over
             replays (max over ranks), minimum and maximum are reported next to it.
             value_launched_one_by_one is the same K steps launched kernel by kernel;
  e2e        same metric with the step's host inputs coming from pinned host memory and the attention
             output going back to it inside the timed region, the stream synchronised every step; three
             ways of moving the same bytes are timed (copies both ways; output written to host memory by the
             kernel; q read from and output written to host memory by the kernel), the fastest is reported;
  roofline   the decode kernel against the measured HBM copy peak: algorithmic KV bytes / the kernel's average launch
             duration inside the replayed graph (the step is one launch of it); the figure from events around every
             eager call is kept beside it;
  append     bulk-append throughput (32768 rows, the chunked-prefill append) in tok/s;
  prefill    (N = 1) the paged chunked-prefill configuration: TFLOP/s against the measured bf16 peak;
  fp8_kv     the same pool as e4m3 bytes: decode GB/s on e4m3 bytes, decode-shape and bulk append;
  fused_append   q/k RMSNorm + rotary embedding + append in one pass, 32768 tokens;
  strong     strong scaling: the long-context configuration (batch 256, 64q/8kv heads) and the
             Qwen3-8B decode shape at batch 64, the 8 KV heads sharded N ways, with the single-GPU
             step they scale from measured in the same process;
  engine     (N = 1) the path inside the engine loop: scheduler, step metadata, one synthetic-weight attention
             layer, decode through per-bucket CUDA graphs; prefill tok/s and decode ms per step, host work included;
  validated  the timed step's outputs (all-gathered over NCCL when N > 1) checked against the CPU oracle on three
             sequences, and the rows it appended compared bit for bit with the inputs;
  reference_gpu  (N = 1) the library call the reference makes for decode (flash_attn's
             flash_attn_with_kvcache), timed on the same tensors;
  cpu_baseline  the torch-CPU restatement of the reference path, timed on a sample.

``--impl reference`` times that CPU restatement alone (the reference has no CPU or
buildable GPU implementation of this path; the oracle port stands in for it).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "paged decode-attn KV GB/s"
UNIT = "GB/s"
BASE_BATCH = 64
# DRAM traffic figures from the ncu captures summarised under profiles/ (dram__bytes_read.sum +
# dram__bytes_write.sum of one launch of a small case; each tile is read once, so traffic grows with the
# units processed): decode_tma_kernel 253.5 MB for 249.9 MB of KV; prefill_tc_kernel 520.0 MB for the 16 sequences
# of the benchmark itself (119.0 MB for a 4-sequence case).
DECODE_TRAFFIC_PER_KV_BYTE = 253.5 / 249.9
PREFILL_TRAFFIC_PER_SEQUENCE = 520.0e6 / 16
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1400.0


def measured_peak():
    try:
        with open(ROOT / "MEASURED_PEAKS.json") as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tflops():
    try:
        with open(ROOT / "MEASURED_PEAKS.json") as f:
            return float(json.load(f)["bf16_tflops_sustained"]), "of measured (sustained)"
    except Exception:
        return FALLBACK_TFLOPS, "of fallback"


def measured_tflops_burst():
    try:
        with open(ROOT / "MEASURED_PEAKS.json") as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return None


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def build_workload(world: int, rank: int, device, base_batch: int = BASE_BATCH, kind: str = "decode"):
    """decode: the headline weak-scaling workload (batch 64 * world); long / decode64: the two
    strong-scaling workloads (fixed batch, the 8 KV heads sharded world ways, page ids replicated)."""
    from infer_b200 import workloads
    if kind == "long":
        return workloads.config4(device=device, seed=1004, n_kv_heads=8 // world, n_q_heads=64 // world,
                                 tensor_seed=1004 + rank)
    batch = base_batch if kind == "decode64" else base_batch * world
    return workloads.config1(device=device, seed=1001, batch=batch, n_kv_heads=8 // world,
                             n_q_heads=32 // world, tensor_seed=1001 + rank)


# ------------------------------------------------------------------------------- CPU leg
def cpu_sample(w, n_seqs: int, repeats: int):
    """Times append + decode of the torch-CPU restatement on the first ``n_seqs`` sequences.
    Returns (seconds per pass, KV bytes per pass, threads)."""
    from oracle import paged_kv_oracle as oracle
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    pages = sorted({p for t in w.block_tables[:n_seqs] for p in t})
    remap = {p: i for i, p in enumerate(pages)}
    idx = torch.tensor(pages, device=w.k_cache.device)
    kc, vc = w.k_cache[idx].cpu(), w.v_cache[idx].cpu()
    tables = [[remap[p] for p in t] for t in w.block_tables[:n_seqs]]
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32)
    lens = w.context_lens[:n_seqs]
    cl = torch.tensor(lens, dtype=torch.int32)
    slots = torch.tensor([t[(n - 1) // 256] * 256 + (n - 1) % 256 for t, n in zip(tables, lens)], dtype=torch.int32)
    q, k, v = w.q[:n_seqs].cpu(), w.k[:n_seqs].cpu(), w.v[:n_seqs].cpu()
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.store_kvcache(k, v, kc, vc, slots)
        oracle.paged_decode_bf16_sdpa(q, kc, vc, cl, bt, w.scale)
        best = min(best, time.perf_counter() - t0)
    kv_bytes = sum(lens) * w.n_kv_heads * 128 * 2 * 2
    return best, kv_bytes, threads


def run_reference(args, rank, world):
    """The reference arm: the CPU restatement on the host cores, rank 0 only."""
    if rank != 0:
        return
    from infer_b200 import workloads
    w = workloads.config1(device="cpu", seed=1001, batch=8, tensor_seed=1001)   # sample: first 8 sequences' lengths
    n_seqs = 8
    for _ in range(args.warmup):
        cpu_sample(w, n_seqs, 1)
    times = []
    for _ in range(args.steps):
        t, kv_bytes, threads = cpu_sample(w, n_seqs, 1)
        times.append(t)
    t = statistics.mean(times)
    value = kv_bytes / t / 1e9
    sample = f"append + decode of {n_seqs} sequences ({kv_bytes / 1e6:.0f} MB of KV) of the same length distribution"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "qwen3-8b decode shape, sample of 8 sequences on host cores", "block_size": 256},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------- timing helpers
def _timed(fn, reps, warm, stream):
    """Mean milliseconds of ``fn`` over ``reps`` back-to-back calls (CUDA events on the launching stream)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record(stream)
    for _ in range(reps):
        fn()
    a1.record(stream)
    torch.cuda.synchronize()
    return a0.elapsed_time(a1) / reps


def time_decode_steps(ops, w, cl, bt, slots, out, steps, warmup, barrier, window_s=0.5, min_replays=50, graph=True):
    """Times ``steps`` steps (append + decode, in one launch: ``paged_attn_decode_append``) of one workload three ways:
      * captured once as ONE CUDA graph of ``steps`` steps and replayed R >= min_replays times (at least
        ``window_s`` seconds), an event pair around every replay: median / min / max ms per step;
      * launched kernel by kernel, one event pair around the whole run: ms per step;
      * launched kernel by kernel with events around every decode call: the decode kernel's own time."""
    stream = torch.cuda.current_stream()

    def step_two():                                           # the reference's two calls (infer/ops/attention.py:109, :117-121)
        ops.store_kvcache(w.k, w.v, w.k_cache, w.v_cache, slots)
        ops.paged_attn_decode(w.q, w.k_cache, w.v_cache, cl, bt, w.scale, out=out)

    def step():                                               # the same step in one launch
        ops.paged_attn_decode_append(w.q, w.k, w.v, w.k_cache, w.v_cache, cl, bt, w.scale, out=out)

    for _ in range(warmup):
        step_two()
        step()
    barrier()
    res = {"graph": None, "graph_two_launches": None, "launches_per_step": 1}

    def capture(fn):
        try:
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg):
                for _ in range(steps):
                    fn()
            cg.replay()                                       # untimed: the first replay uploads the graph
            torch.cuda.synchronize()
            return cg
        except Exception as exc:                              # pragma: no cover - reported as absent
            print(f"[bench] CUDA-graph capture of the device-resident steps failed ({exc})", file=sys.stderr)
            return None

    g = capture(step) if graph else None
    g2 = capture(step_two) if graph else None
    t_begin = time.time()
    if g is not None:
        # how many replays fill the window: one timed probe
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record(stream)
        g.replay()
        p1.record(stream)
        torch.cuda.synchronize()
        replays = max(min_replays, int(math.ceil(window_s * 1e3 / max(p0.elapsed_time(p1), 1e-3))))
        replays = min(replays, 2000)
        mk = lambda: [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(replays)]
        evs, evs2 = mk(), mk() if g2 is not None else []
        barrier()
        # the one-launch step and the two-launch step take turns, replay by replay, so that both see the same clocks
        for i, (e0, e1) in enumerate(evs):
            e0.record(stream)
            g.replay()
            e1.record(stream)
            if g2 is not None:
                f0, f1 = evs2[i]
                f0.record(stream)
                g2.replay()
                f1.record(stream)
        barrier()
        per_step = sorted(e0.elapsed_time(e1) / steps for e0, e1 in evs)
        res["graph"] = {"median": statistics.median(per_step), "min": per_step[0], "max": per_step[-1],
                        "replays": replays, "timed_s": sum(per_step) * steps / 1e3}
        if g2 is not None:
            res["graph_two_launches"] = statistics.median(f0.elapsed_time(f1) / steps for f0, f1 in evs2)
    # launched one by one, no events in between (events between kernels would break their overlap)
    reps = max(1, int(math.ceil(0.1 / max(1e-6, steps * 2e-4)))) if window_s > 0 else 1      # about 0.1 s of steps
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    s0.record(stream)
    for _ in range(reps * steps):
        step()
    s1.record(stream)
    barrier()
    res["eager_ms"] = s0.elapsed_time(s1) / (reps * steps)
    # per-call events: the decode kernel and the decode-shape append on their own
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    for i in range(steps):
        ev[i][0].record(stream)
        ops.store_kvcache(w.k, w.v, w.k_cache, w.v_cache, slots)
        ev[i][1].record(stream)
        ops.paged_attn_decode(w.q, w.k_cache, w.v_cache, cl, bt, w.scale, out=out)
        ev[i][2].record(stream)
    barrier()
    decode_all = [e[1].elapsed_time(e[2]) for e in ev]
    res["decode_ms"] = statistics.mean(decode_all)
    res["decode_ms_median"] = statistics.median(decode_all)
    res["decode_ms_min"] = min(decode_all)
    res["append_ms"] = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    res["region_s"] = time.time() - t_begin
    return res


def reduce_max(values, device, world):
    import torch.distributed as dist
    t = torch.tensor(values, device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def reduce_sum(value, device, world):
    import torch.distributed as dist
    t = torch.tensor([float(value)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.item()


# ------------------------------------------------------------------------------- validation over NCCL
def validate_gathered(w, out, world, rank, n_check=3):
    """north-star use of NCCL: all-gather the attention outputs (and, for the checked sequences, the
    pages and queries of every shard) and compare with the CPU oracle of the unsharded problem on rank 0."""
    import numpy as np
    import torch.distributed as dist
    from oracle import paged_kv_oracle as oracle
    if world > 1:
        from infer_b200.sharding import gather_heads
    else:
        gather_heads = lambda t: t                     # one GPU holds every head: nothing to gather
    full_out = gather_heads(out)
    full_q = gather_heads(w.q)
    order = np.argsort(w.context_lens)
    picks = sorted({int(order[0]), int(order[len(order) // 2]), int(order[-1])})[:n_check]
    max_err, ok = 0.0, True
    for b in picks:
        pages = torch.tensor(w.block_tables[b], device=out.device)
        kc = gather_heads(w.k_cache[pages].reshape(-1, w.n_kv_heads, 128)).reshape(len(pages), 256, -1, 128)
        vc = gather_heads(w.v_cache[pages].reshape(-1, w.n_kv_heads, 128)).reshape(len(pages), 256, -1, 128)
        if rank == 0:
            local = torch.arange(len(pages), dtype=torch.int32)[None]
            want = oracle.paged_decode(full_q[b:b + 1].cpu(), kc.cpu(), vc.cpu(),
                                       torch.tensor([w.context_lens[b]], dtype=torch.int32), local, w.scale).float()
            err = (full_out[b:b + 1].float().cpu() - want).abs()
            max_err = max(max_err, float(err.max()))
            ok = ok and bool((err <= 2e-2 + 1e-2 * want.abs()).all())
    # the rows the step appended: bit-exact in the pools, every sequence
    flat_k, flat_v = w.k_cache.view(-1, w.n_kv_heads, 128), w.v_cache.view(-1, w.n_kv_heads, 128)
    at = w.slot_mapping.to(out.device).long()
    rows_ok = bool(torch.equal(flat_k[at], w.k)) and bool(torch.equal(flat_v[at], w.v))
    if world > 1:
        flag = torch.tensor([int(rows_ok)], device=out.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        rows_ok = bool(flag.item())
        dist.barrier()
    return {"nranks": world, "sequences": len(picks), "max_err": max_err, "ok": ok and rows_ok, "appended_rows_bit_exact": rows_ok,
            "tolerance": "2e-2 abs + 1e-2 rel against the CPU oracle",
            "gather": "nccl all_gather" if world > 1 else "none (one GPU holds every head)"}


# ------------------------------------------------------------------------------- sub-benchmarks
def bench_prefill(ops, device, n_seqs, steps, warmup, dense=True, sample_clocks=True):
    """Chunked prefill over cached prefixes: append the chunk, then causal attention over
    prefix + chunk.  FLOPs = 4 * 128 * Hq * sum(chunk * prefix + chunk * (chunk + 1) / 2)."""
    from infer_b200 import workloads
    w = workloads.config2(device=device, n_seqs=n_seqs)
    cu_q, cu_k = (t.to(device) for t in w.cu_seqlens())
    bt = w.block_tables_tensor().to(device)
    slots = w.slot_mapping.to(device)
    out = torch.empty_like(w.q)
    mq, mk = max(w.new_lens), max(w.context_lens)
    flops = 4 * 128 * w.n_q_heads * sum(c * (n - c) + c * (c + 1) // 2 for c, n in zip(w.new_lens, w.context_lens))
    stream = torch.cuda.current_stream()

    def step():
        ops.store_kvcache(w.k, w.v, w.k_cache, w.v_cache, slots)
        ops.paged_attn_prefill(w.q, w.k_cache, w.v_cache, cu_q, cu_k, mq, mk, w.scale, bt, out=out)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    # a burst on a GPU that has idled for two seconds (the way MEASURED_PEAKS.json's bf16_tflops was taken), before the
    # sustained measurement below: under the 1000 W cap the chip clocks lower once the cap binds
    burst_tflops = None
    if sample_clocks:
        time.sleep(2.0)
        burst_ms = _timed(lambda: ops.paged_attn_prefill(w.q, w.k_cache, w.v_cache, cu_q, cu_k, mq, mk, w.scale, bt, out=out),
                          10, 0, stream)
        burst_tflops = flops / (burst_ms * 1e-3) / 1e12
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    with ClockSampler(device.index) as clocks:
        t_end = time.time() + (0.5 if sample_clocks else 0.0)
        rounds = 0
        while True:
            for i in range(steps):
                ev[i][0].record(stream)
                ops.store_kvcache(w.k, w.v, w.k_cache, w.v_cache, slots)
                ev[i][1].record(stream)
                ops.paged_attn_prefill(w.q, w.k_cache, w.v_cache, cu_q, cu_k, mq, mk, w.scale, bt, out=out)
                ev[i][2].record(stream)
            torch.cuda.synchronize()
            rounds += 1
            if time.time() >= t_end:
                break
    attn_all = [e[1].elapsed_time(e[2]) for e in ev]           # the last round's steps
    attn_ms = statistics.median(attn_all)
    append_ms = statistics.median(e[0].elapsed_time(e[1]) for e in ev)
    step_ms = statistics.median(e[0].elapsed_time(e[2]) for e in ev)
    peak, kind = measured_tflops()
    achieved = flops / (attn_ms * 1e-3) / 1e12
    n_tok = sum(w.new_lens)
    res = {
        "workload": f"paged chunked prefill: {n_seqs} sequences, prefix U[0,4096], chunk 2048, 16q/8kv heads, page 256; "
                    "append of the chunk + causal attention over prefix + chunk",
        "flops_per_step": flops, "tflops_step": flops / (step_ms * 1e-3) / 1e12, "ms_per_step": step_ms,
        "attn_ms": attn_ms, "attn_ms_min": min(attn_all), "attn_ms_max": max(attn_all),
        "tflops": achieved, "peak": peak, "frac": achieved / peak, "peak_kind": kind, "bound": "tensor",
        "tflops_burst": burst_tflops, "burst_note": "10 calls after two idle seconds; compare with bf16_tflops (burst) of "
                                                    "MEASURED_PEAKS.json, `tflops` with bf16_tflops_sustained",
        "frac_burst": (burst_tflops / measured_tflops_burst()) if burst_tflops and measured_tflops_burst() else None,
        "timed_steps": steps * rounds,
        "traffic": PREFILL_TRAFFIC_PER_SEQUENCE * n_seqs,
        "append": {"rows": n_tok, "ms": append_ms, "tok_s": n_tok / (append_ms * 1e-3),
                   "gbs": n_tok * w.n_kv_heads * 128 * 2 * 4 / (append_ms * 1e-3) / 1e9},
        "clocks": clocks.summary(),
    }
    # the library call the reference makes for this step (infer/ops/attention.py:113-116), on the same tensors
    try:
        import flash_attn
        from flash_attn import flash_attn_varlen_func
        fa = lambda: flash_attn_varlen_func(w.q, w.k_cache, w.v_cache, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, max_seqlen_q=mq,
                                            max_seqlen_k=mk, softmax_scale=w.scale, causal=True, block_table=bt)
        ref = fa()
        torch.cuda.synchronize()
        fa_ms = _timed(fa, 5, 2, stream)
        res["reference_gpu"] = {"kind": f"flash_attn {getattr(flash_attn, '__version__', '?')} flash_attn_varlen_func with block_table",
                                "attn_ms": fa_ms, "tflops": flops / (fa_ms * 1e-3) / 1e12,
                                "max_abs_diff_vs_this_library": float((ref.float() - out.float()).abs().max())}
    except Exception as exc:
        res["reference_gpu"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:120]}"}
    del w
    if dense:
        gen = torch.Generator(device=device).manual_seed(7)
        B, H, Hkv, S = 4, 16, 8, 4096
        dq = torch.randn(B, H, S, 128, generator=gen, device=device).bfloat16()
        dk = torch.randn(B, Hkv, S, 128, generator=gen, device=device).bfloat16()
        dv = torch.randn(B, Hkv, S, 128, generator=gen, device=device).bfloat16()
        do = torch.empty_like(dq)
        dms = _timed(lambda: ops.flash_attn_prefill(dq, dk, dv, do), 10, 3, stream)
        dflops = 4 * 128 * B * H * S * (S + 1) // 2
        res["dense_op"] = {"shape": [B, H, S, 128], "kv_heads": Hkv, "ms": dms, "tflops": dflops / (dms * 1e-3) / 1e12,
                           "frac": dflops / (dms * 1e-3) / 1e12 / peak}
    return res


def bench_fp8(ops, w, cl, bt, slots, out, decode_ms_bf16, peak, profile):
    """The same pool as e4m3 bytes with one fp32 scale per (page, kv head)."""
    device, hkv, nb = w.q.device, w.n_kv_heads, w.num_blocks
    stream = torch.cuda.current_stream()
    k8 = torch.zeros(nb, 256, hkv, 128, dtype=torch.uint8, device=device)
    v8 = torch.zeros_like(k8)
    ks8 = torch.zeros(nb, hkv, device=device)
    vs8 = torch.zeros(nb, hkv, device=device)
    for lo in range(0, nb, 64):                           # quantise the bf16 pool page group by page group
        hi = min(nb, lo + 64)
        sl = torch.arange(lo * 256, hi * 256, dtype=torch.int32, device=device)
        ops.store_kvcache(w.k_cache[lo:hi].reshape(-1, hkv, 128), w.v_cache[lo:hi].reshape(-1, hkv, 128), k8, v8, sl, ks8, vs8)
    torch.cuda.synchronize()
    reps, warm = (3, 0) if profile else (20, 3)
    dec8_ms = _timed(lambda: ops.paged_attn_decode(w.q, k8, v8, cl, bt, w.scale, out=out, k_scale=ks8, v_scale=vs8),
                     reps, warm, stream)
    app8_ms = _timed(lambda: ops.store_kvcache(w.k, w.v, k8, v8, slots, ks8, vs8), reps, warm, stream)
    # the whole e4m3 step (append + decode, two calls) as a graph of 20 steps, like the bf16 headline
    step8_us = None
    if not profile:
        def step8():
            ops.store_kvcache(w.k, w.v, k8, v8, slots, ks8, vs8)
            ops.paged_attn_decode(w.q, k8, v8, cl, bt, w.scale, out=out, k_scale=ks8, v_scale=vs8)
        try:
            step8()
            torch.cuda.synchronize()
            g8 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g8):
                for _ in range(20):
                    step8()
            g8.replay()
            torch.cuda.synchronize()
            step8_us = statistics.median(_timed(g8.replay, 5, 0, stream) for _ in range(5)) / 20 * 1e3
        except Exception as exc:                              # pragma: no cover - reported as absent
            print(f"[bench] CUDA-graph capture of the e4m3 steps failed ({exc})", file=sys.stderr)
    n_rows = min(32768, nb * 256)
    sl = torch.arange(0, n_rows, dtype=torch.int32, device=device)
    rk = w.k_cache.view(-1, hkv, 128)[:n_rows]
    rv = w.v_cache.view(-1, hkv, 128)[:n_rows]
    bulk8_ms = _timed(lambda: ops.store_kvcache(rk, rv, k8, v8, sl, ks8, vs8), reps, warm, stream)
    kv8 = w.kv_bytes(elem_bytes=1) + 2 * 4 * hkv * sum(-(-n // 256) for n in w.context_lens)
    dec_gbs = kv8 / (dec8_ms * 1e-3) / 1e9
    bulk_gbs = n_rows * hkv * 128 * 2 * (2 + 1) / (bulk8_ms * 1e-3) / 1e9
    return {"decode_us": dec8_ms * 1e3, "kv_bytes_e4m3": kv8, "decode_gbs": dec_gbs, "decode_frac": dec_gbs / peak,
            "tokens_per_us_vs_bf16": decode_ms_bf16 / dec8_ms, "append_decode_shape_us": app8_ms * 1e3,
            "step_us": step8_us, "step_gbs": (kv8 / (step8_us * 1e-6) / 1e9) if step8_us else None,
            "step_note": "append + decode of the e4m3 pool (two calls) as a graph of 20 steps, replayed; median",
            "bulk_rows": n_rows, "bulk_us": bulk8_ms * 1e3, "bulk_tok_s": n_rows / (bulk8_ms * 1e-3),
            "bulk_gbs": bulk_gbs, "bulk_frac": bulk_gbs / peak,
            "bulk_bytes_note": "per row and head: 256 B of bf16 read for K and V each, 128 B of e4m3 written each"}


def bench_fused_append(ops, w, peak, profile):
    """q/k RMSNorm + rotary embedding + KV append in one pass over the fused qkv rows (32768 tokens)."""
    device, hq, hkv, t = w.q.device, w.n_q_heads, w.n_kv_heads, 32768
    stream = torch.cuda.current_stream()
    gen = torch.Generator(device=device).manual_seed(9)
    qkv = torch.randn(t, (hq + 2 * hkv) * 128, generator=gen, device=device).bfloat16()
    q = qkv[:, :hq * 128].view(t, hq, 128)
    k = qkv[:, hq * 128:(hq + hkv) * 128].view(t, hkv, 128)
    v = qkv[:, (hq + hkv) * 128:].view(t, hkv, 128)
    qw = torch.randn(128, generator=gen, device=device).bfloat16()
    kw = torch.randn(128, generator=gen, device=device).bfloat16()
    cache = torch.randn(8192, 128, generator=gen, device=device).bfloat16()
    pos = torch.randint(0, 8192, (t,), generator=gen, device=device)
    slots = torch.randperm(w.num_blocks * 256, generator=gen, device=device)[:t].to(torch.int32)
    qo = torch.empty(t, hq, 128, device=device, dtype=torch.bfloat16)
    reps, warm = (3, 0) if profile else (20, 3)
    ms = _timed(lambda: ops.qk_norm_rope_append(q, k, v, qw, kw, 1e-6, pos, cache, w.k_cache, w.v_cache, slots, q_out=qo),
                reps, warm, stream)
    nbytes = t * (hq + 2 * hkv) * 256 + t * hq * 256 + t * 2 * hkv * 256
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"tokens": t, "heads": f"{hq}q/{hkv}kv", "us": ms * 1e3, "min_traffic_bytes": nbytes, "gbs": gbs,
            "frac": gbs / peak, "tok_s": t / (ms * 1e-3)}


def bench_flash_attn(w, cl, bt, slots, out, steps):
    """The library call the reference makes for decode (infer/ops/attention.py:117-121), on the same
    tensors.  The append stands in for the reference's Triton store kernel (whose source is not
    shipped with this repository) as torch's index_copy_."""
    try:
        import flash_attn
        from flash_attn import flash_attn_with_kvcache
    except Exception as exc:
        return {"unavailable": f"flash_attn does not import ({type(exc).__name__})"}
    stream = torch.cuda.current_stream()
    kflat = w.k_cache.view(-1, w.n_kv_heads, 128)
    vflat = w.v_cache.view(-1, w.n_kv_heads, 128)
    idx = slots.long()
    q4 = w.q.unsqueeze(1)

    def step():
        kflat.index_copy_(0, idx, w.k)
        vflat.index_copy_(0, idx, w.v)
        return flash_attn_with_kvcache(q4, w.k_cache, w.v_cache, cache_seqlens=cl, block_table=bt,
                                       softmax_scale=w.scale, causal=True)
    try:
        o = step()
        torch.cuda.synchronize()
        err = float((o.squeeze(1).float() - out.float()).abs().max())
        ms = _timed(step, steps, 3, stream)
    except Exception as exc:
        return {"unavailable": f"flash_attn_with_kvcache failed here ({type(exc).__name__}: {str(exc)[:120]})"}
    kv = w.kv_bytes()
    return {"kind": f"flash_attn {getattr(flash_attn, '__version__', '?')} flash_attn_with_kvcache + torch index_copy_ append, "
                    "launched one by one", "ms_per_step": ms, "value": kv / (ms * 1e-3) / 1e9, "unit": UNIT,
            "max_abs_diff_vs_this_library": err}


def bench_engine(device, n_requests=64, max_tokens=48, device_metadata=False):
    """The path inside the engine loop (scheduler -> step metadata -> model -> postprocess, the reference's
    LLMEngine.step, infer/engine/llm_engine.py:46-82) with ONE synthetic-weight attention layer as the model:
    prompts U[512, 2048] prefilled, then decode steps through per-bucket CUDA graphs.  Host scheduling and the
    per-step metadata upload are inside the timed regions (wall clock around synchronised steps)."""
    import numpy as np
    from infer_b200.context import reset_context
    from infer_b200.engine import AttentionLayerModel, Engine, LayerRunner, Scheduler
    rng = np.random.default_rng(77)
    hidden, hq, hkv, vocab, block = 2048, 32, 8, 4096, 256
    prompts = [rng.integers(0, vocab, size=int(n)).tolist() for n in rng.integers(512, 2049, size=n_requests)]
    pages = sum(-(-(len(pr) + max_tokens) // block) for pr in prompts) + 8
    model = AttentionLayerModel(hidden, hq, hkv, vocab, 4096, device, seed=3)
    runner = LayerRunner(model, pages, block, n_requests, 4096, device, device_metadata=device_metadata)
    engine = Engine(runner, Scheduler(pages, block, max_num_seqs=n_requests, max_num_batched_tokens=1 << 20))
    for pr in prompts:
        engine.add_request(pr, max_tokens)
    t = {True: 0.0, False: 0.0}
    n = {True: 0, False: 0}
    toks = {True: 0, False: 0}
    while not engine.scheduler.is_finished():
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        seqs, is_prefill, _ = engine.step()
        torch.cuda.synchronize()
        t[is_prefill] += time.perf_counter() - t0
        n[is_prefill] += 1
        toks[is_prefill] += sum(len(s) - 1 for s in seqs) if is_prefill else len(seqs)
        reset_context()
    res = {"model": f"one attention layer, hidden {hidden}, {hq}q/{hkv}kv heads, synthetic weights (the real checkpoints are "
                    "not in the image); qkv / output projections and norm + rotary in PyTorch, append + attention through "
                    "this library",
           "requests": n_requests, "prompt_tokens": toks[True], "prefill_steps": n[True],
           "prefill_tok_s": toks[True] / max(t[True], 1e-9),
           "decode_steps": n[False], "decode_ms_per_step": 1e3 * t[False] / max(n[False], 1),
           "decode_tok_s": toks[False] / max(t[False], 1e-9),
           "decode_launch": "one CUDA graph per batch-size bucket, replayed; host scheduling and metadata upload inside the time"}
    del engine, runner, model
    torch.cuda.empty_cache()
    return res


def bench_strong(ops, kind, world, rank, device, steps, warmup, barrier, peak):
    """One strong-scaling workload at ``world`` GPUs and, in the same process, the single-GPU problem it
    scales from (all 8 KV heads on this GPU)."""
    res = {}
    for label, wd, rk in (("sharded", world, rank), ("single_gpu", 1, 0)):
        if label == "single_gpu" and world == 1:
            res[label] = res["sharded"]
            break
        w = build_workload(wd, rk, device, BASE_BATCH, kind)
        cl, bt, slots = w.context_lens_tensor().to(device), w.block_tables_tensor().to(device), w.slot_mapping.to(device)
        out = torch.empty_like(w.q)
        r = time_decode_steps(ops, w, cl, bt, slots, out, steps, warmup, barrier if label == "sharded" else torch.cuda.synchronize,
                              window_s=0.2, min_replays=20)
        kv = w.kv_bytes()
        g = r["graph"]
        step_ms = g["median"] if g else r["eager_ms"]
        vals = [step_ms, r["eager_ms"], r["decode_ms"]]
        if label == "sharded":
            vals = reduce_max(vals, device, world)
            job = reduce_sum(kv, device, world)
        else:
            job = kv
        res[label] = {"n_gpus": wd, "batch": len(w.context_lens), "kv_bytes_per_gpu": kv, "job_kv_bytes": job,
                      "step_us": vals[0] * 1e3, "step_us_launched_one_by_one": vals[1] * 1e3,
                      "decode_us": vals[2] * 1e3, "aggregate_gbs": job / (vals[0] * 1e-3) / 1e9,
                      "per_gpu_decode_gbs": kv / (vals[2] * 1e-3) / 1e9, "per_gpu_decode_frac": kv / (vals[2] * 1e-3) / 1e9 / peak}
        if label == "sharded" and world > 1 and kind == "long":
            ops.store_kvcache(w.k, w.v, w.k_cache, w.v_cache, slots)
            ops.paged_attn_decode(w.q, w.k_cache, w.v_cache, cl, bt, w.scale, out=out)
            res["validated"] = validate_gathered(w, out, world, rank)
        del w, out
        torch.cuda.empty_cache()
    s, one = res["sharded"], res["single_gpu"]
    res["speedup_vs_single_gpu"] = one["step_us"] / s["step_us"]
    res["step_efficiency"] = one["step_us"] / (world * s["step_us"])
    res["step_efficiency_launched_one_by_one"] = one["step_us_launched_one_by_one"] / (world * s["step_us_launched_one_by_one"])
    return res


# ------------------------------------------------------------------------------- GPU leg
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="short run for profiler captures: the headline steps launched one by one and 3 bulk appends, "
                         "no graph, no end-to-end leg, no sub-benchmarks, no CPU baseline")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "long"],
                    help="decode = the full line; prefill = only the paged chunked-prefill configuration (single GPU, "
                         "used for profiler captures); long = only the long-context configuration as the headline")
    ap.add_argument("--only", default="", help="comma-separated sub-benchmarks to run (prefill,fp8,fused,strong,flash,engine); "
                                               "default: all, or none with --profile")
    ap.add_argument("--fp8", action="store_true", help="same as adding fp8 to --only")
    ap.add_argument("--batch", type=int, default=BASE_BATCH,
                    help="sequences per GPU share (default 64 = the benchmark configuration; smaller values "
                         "give the small case used for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if 8 % world:
        raise SystemExit("KV-head sharding needs a GPU count that divides 8")

    import torch.distributed as dist
    from infer_b200 import ops

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if args.workload == "prefill":
        if world != 1:
            raise SystemExit("--workload prefill runs on one GPU")
        n_seqs = 16 if args.batch == BASE_BATCH else args.batch
        res = bench_prefill(ops, device, n_seqs, args.steps, args.warmup, dense=not args.profile,
                            sample_clocks=not args.profile)
        print(json.dumps({"metric": "paged chunked-prefill attention TFLOP/s", "value": res["tflops_step"], "unit": "TFLOP/s",
                          "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"],
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                          "data": "synthetic", "config": {"workload": res["workload"]}, "gpu_launches": 2 * res["timed_steps"],
                          "roofline": {"bound": "tensor", "kernel": "prefill_tc_kernel", "achieved": res["tflops"],
                                       "peak": res["peak"], "unit": "TFLOP/s", "frac": res["frac"],
                                       "peak_kind": res["peak_kind"], "traffic": res["traffic"]},
                          "prefill": res, "clocks": res["clocks"]}))
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    want = set(filter(None, args.only.split(",")))
    if not want and not args.profile:
        want = {"prefill", "fp8", "fused", "strong", "flash", "engine"}
    if args.fp8:
        want.add("fp8")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    peak, peak_kind = measured_peak()
    w = build_workload(world, rank, device, args.batch, "long" if args.workload == "long" else "decode")
    cl = w.context_lens_tensor().to(device)
    bt = w.block_tables_tensor().to(device)
    slots = w.slot_mapping.to(device)
    out = torch.empty_like(w.q)
    kv_bytes = w.kv_bytes()                      # this rank's algorithmic KV bytes per step
    stream = torch.cuda.current_stream()

    # ---- device-resident timing, inside the clock-sampling window
    with ClockSampler(local_rank) as clocks:
        r = time_decode_steps(ops, w, cl, bt, slots, out, args.steps, args.warmup, barrier,
                              window_s=0.0 if args.profile else 0.5, min_replays=50, graph=not args.profile)
    g = r["graph"]

    # ---- end to end: host inputs in pinned memory, output read back, every step
    from infer_b200.staging import StepStaging
    src = {"q": w.q, "k": w.k, "v": w.v, "slots": slots, "cl": cl, "bt": bt}
    stage = StepStaging({k: (tuple(v.shape), v.dtype) for k, v in src.items()}, device)
    for k, v in src.items():
        stage.host[k].copy_(v)                                # the step's inputs as the host produced them
    dev = stage.dev
    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in src.values())
    d2h = out_host.numel() * out_host.element_size()

    # Three ways a caller can feed one step from host memory; all move the same bytes over PCIe every step:
    #   staged     one H2D copy of the arena (q, k, v, metadata), kernels, one D2H copy of the output
    #   out_host   same upload; the attention kernel writes its output rows straight into pinned host memory
    #              (the pointer of a pinned tensor is valid on the device), so the read-back overlaps the kernel
    #   q_out_host additionally the kernel reads q from pinned host memory; only k, v and the metadata are copied
    #   all_host   the one-launch step (append + attention) reads q, k and v from pinned host memory and writes its
    #              output there; only lengths and block tables are copied
    small = {k: v for k, v in src.items() if k != "q"}
    stage_small = StepStaging({k: (tuple(v.shape), v.dtype) for k, v in small.items()}, device)
    for k, v in small.items():
        stage_small.host[k].copy_(v)
    q_host = stage.host["q"]

    def body_staged():
        stage.upload()                                        # one copy for q, k, v and the step metadata
        ops.store_kvcache(dev["k"], dev["v"], w.k_cache, w.v_cache, dev["slots"])
        ops.paged_attn_decode(dev["q"], w.k_cache, w.v_cache, dev["cl"], dev["bt"], w.scale, out=out)
        out_host.copy_(out, non_blocking=True)

    def body_out_host():
        stage.upload()
        ops.store_kvcache(dev["k"], dev["v"], w.k_cache, w.v_cache, dev["slots"])
        ops.paged_attn_decode(dev["q"], w.k_cache, w.v_cache, dev["cl"], dev["bt"], w.scale, out=out_host)

    def body_q_out_host():
        ds = stage_small.dev
        stage_small.upload()
        ops.store_kvcache(ds["k"], ds["v"], w.k_cache, w.v_cache, ds["slots"])
        ops.paged_attn_decode(q_host, w.k_cache, w.v_cache, ds["cl"], ds["bt"], w.scale, out=out_host)

    kv_host = {"k": stage.host["k"], "v": stage.host["v"]}
    meta = {k: v for k, v in src.items() if k in ("cl", "bt")}
    stage_meta = StepStaging({k: (tuple(v.shape), v.dtype) for k, v in meta.items()}, device)
    for k, v in meta.items():
        stage_meta.host[k].copy_(v)

    def body_all_host():
        dm = stage_meta.dev
        stage_meta.upload()                                   # lengths and block tables: 9 KB
        ops.paged_attn_decode_append(q_host, kv_host["k"], kv_host["v"], w.k_cache, w.v_cache, dm["cl"], dm["bt"], w.scale,
                                     out=out_host)

    def body_all_host_resident():
        # lengths and block tables stay on the device between steps (metadata.DecodeState keeps them there and
        # advances them with one small kernel; this workload's lengths do not change from step to step)
        ops.paged_attn_decode_append(q_host, kv_host["k"], kv_host["v"], w.k_cache, w.v_cache, cl, bt, w.scale, out=out_host)

    def time_e2e(body):
        """ms per step: the step captured once in a CUDA graph (the way the reference replays its decode graphs,
        infer/engine/model_runner.py:135-152) and replayed, the stream synchronised after every step."""
        graph = None
        try:
            body()
            torch.cuda.synchronize()
            eg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(eg):
                body()
            graph = eg
        except Exception as exc:                              # pragma: no cover - falls back to eager launches
            print(f"[bench] CUDA-graph capture of the end-to-end step failed ({exc}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()

        def one():
            if graph is not None:
                graph.replay()
            else:
                body()
            torch.cuda.current_stream().synchronize()       # the caller reads the result every step

        for _ in range(args.warmup):
            one()
        steps = max(args.steps, 1000)                        # about a quarter of a second
        e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e_start.record(stream)
        for _ in range(steps):
            one()
        e_stop.record(stream)
        barrier()
        return max(e_start.elapsed_time(e_stop), 1e-6) / steps, steps, graph is not None

    nbytes = lambda *names: sum(src[n].numel() * src[n].element_size() for n in names)
    h2d_by_mode = {"staged": h2d, "out_host": h2d, "q_out_host": h2d, "all_host": nbytes("q", "k", "v", "cl", "bt"),
                   "all_host_resident_metadata": nbytes("q", "k", "v")}      # bytes that cross PCIe towards the GPU per step
    e2e_ms, e2e_steps, e2e_graphed, e2e_mode, e2e_all = 1e-6, 0, False, "none", {}
    if not args.profile:
        for mode, body in (("staged", body_staged), ("out_host", body_out_host), ("q_out_host", body_q_out_host),
                           ("all_host", body_all_host), ("all_host_resident_metadata", body_all_host_resident)):
            ms, e2e_steps, graphed = time_e2e(body)
            e2e_all[mode] = ms
            # every rank must pick the same mode: decide on the maximum over ranks
            ms_all = reduce_max([ms], device, world)[0]
            if e2e_mode == "none" or ms_all < e2e_ms:
                e2e_ms, e2e_mode, e2e_graphed = ms_all, mode, graphed
        # the result really is in host memory: compare the last step's rows with the device copy
        torch.cuda.synchronize()
        body_staged()
        torch.cuda.synchronize()
        ref_rows = out_host.clone()
        for body in (body_q_out_host, body_all_host, body_all_host_resident):
            out_host.zero_()
            body()
            torch.cuda.synchronize()
            if not torch.equal(ref_rows, out_host):
                raise SystemExit("bench: the output written straight to host memory differs from the copied one")

    # ---- bulk append (the chunked-prefill append: 32768 rows)
    n_bulk = 32768
    hkv = w.n_kv_heads
    gen = torch.Generator(device=device).manual_seed(5)
    bk = torch.randn(n_bulk, hkv, 128, generator=gen, device=device).bfloat16()
    bv = torch.randn(n_bulk, hkv, 128, generator=gen, device=device).bfloat16()
    bslots = torch.randperm(w.num_blocks * 256, generator=gen, device=device)[:n_bulk].to(torch.int32)
    bulk_ms = _timed(lambda: ops.store_kvcache(bk, bv, w.k_cache, w.v_cache, bslots), 3 if args.profile else 20,
                     0 if args.profile else 3, stream)
    bulk_bytes = n_bulk * hkv * 128 * 2 * (2 + 2)
    del bk, bv, bslots

    # ---- a second bulk point: 262144 rows (every row of 1024 pages), when the pool has them
    n_bulk2, bulk2_ms = 262144, 0.0
    if not args.profile and w.num_blocks * 256 >= n_bulk2:
        bk = torch.randn(n_bulk2, hkv, 128, generator=gen, device=device).bfloat16()
        bv = torch.randn(n_bulk2, hkv, 128, generator=gen, device=device).bfloat16()
        bslots = torch.randperm(w.num_blocks * 256, generator=gen, device=device)[:n_bulk2].to(torch.int32)
        bulk2_ms = _timed(lambda: ops.store_kvcache(bk, bv, w.k_cache, w.v_cache, bslots), 5, 2, stream)
        del bk, bv, bslots
    bulk2_bytes = n_bulk2 * hkv * 128 * 2 * (2 + 2)

    # ---- sub-benchmarks on the same pool (rank 0's figures are reported)
    fp8 = bench_fp8(ops, w, cl, bt, slots, out, r["decode_ms"], peak, args.profile) if "fp8" in want else None
    fused = bench_fused_append(ops, w, peak, args.profile) if "fused" in want else None
    flash = None
    if "flash" in want and world == 1:
        ops.store_kvcache(w.k, w.v, w.k_cache, w.v_cache, slots)
        ops.paged_attn_decode(w.q, w.k_cache, w.v_cache, cl, bt, w.scale, out=out)
        flash = bench_flash_attn(w, cl, bt, slots, out, args.steps)
    validated = None
    if world > 1 or not args.profile:
        # the step as it was timed (one launch), on pools whose new rows are cleared first
        flat = w.slot_mapping.to(device).long()
        w.k_cache.view(-1, w.n_kv_heads, 128)[flat] = 0
        w.v_cache.view(-1, w.n_kv_heads, 128)[flat] = 0
        ops.paged_attn_decode_append(w.q, w.k, w.v, w.k_cache, w.v_cache, cl, bt, w.scale, out=out)
        validated = validate_gathered(w, out, world, rank)

    # ---- max over ranks
    step_ms_rank = g["median"] if g else r["eager_ms"]
    vals = reduce_max([step_ms_rank, g["min"] if g else 0.0, g["max"] if g else 0.0, r["eager_ms"], r["decode_ms"],
                       r["append_ms"], e2e_ms, bulk_ms, bulk2_ms], device, world)
    step_ms, step_min, step_max, eager_ms, decode_ms, append_ms, e2e_ms, bulk_ms, bulk2_ms = vals
    job_bytes = reduce_sum(kv_bytes, device, world)
    cpu = None
    if rank == 0 and not args.no_cpu_baseline and not args.profile and world == 1:
        secs, cpu_bytes, threads = cpu_sample(w, 8, 2)
        cpu = {"value": cpu_bytes / secs / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"append + decode of the first 8 sequences ({cpu_bytes / 1e6:.0f} MB of KV), best of 2"}
    n_seq = len(w.context_lens)
    kv_logical = w.kv_bytes(unique=False)
    del w, out, stage
    torch.cuda.empty_cache()

    strong = None
    if "strong" in want and args.workload == "decode":
        strong = {"long": bench_strong(ops, "long", world, rank, device, 20, 3, barrier, peak),
                  "decode64": bench_strong(ops, "decode64", world, rank, device, 20, 3, barrier, peak)}
    prefill = None
    if "prefill" in want and world == 1:
        prefill = bench_prefill(ops, device, 16, 10, 3)
    engine = None
    if "engine" in want and world == 1:
        try:
            engine = bench_engine(device)
            on_device = bench_engine(device, device_metadata=True)
            engine["decode_ms_per_step_device_metadata"] = on_device["decode_ms_per_step"]
            engine["decode_tok_s_device_metadata"] = on_device["decode_tok_s"]
            engine["device_metadata"] = ("the same loop with the decode step's lengths, slots and positions advanced on the "
                                         "GPU by one small kernel instead of rebuilt and uploaded by the host every step")
        except Exception as exc:                                  # pragma: no cover - reported, the line still prints
            engine = {"failed": f"{type(exc).__name__}: {str(exc)[:200]}"}

    if rank == 0:
        value = job_bytes / (step_ms * 1e-3) / 1e9
        # The step is ONE launch of the decode kernel, so inside the replayed graph the kernel's average launch duration
        # over the timed region is the step time itself (this rank's median replay / K).  Events around every eager
        # call also time the gap between launches; that figure is kept beside it.
        launch_ms = step_ms_rank if g else decode_ms
        achieved = kv_bytes / (launch_ms * 1e-3) / 1e9
        achieved_per_call = kv_bytes / (decode_ms * 1e-3) / 1e9
        if args.workload == "long":
            desc = (f"qwen3-32b long-context decode: batch {n_seq}, ctx lognormal(median 4096, sigma 0.8) capped at 32768, "
                    f"half the batch sharing the pages of a 2048-token prefix, 64q/8kv heads sharded {world}-way by KV "
                    "head, page 256, 1 appended token per sequence; KV bytes count a shared page once")
        else:
            desc = (f"qwen3-8b decode shape: batch {n_seq}, ctx U[512,8192], 32q/8kv heads "
                    f"sharded {world}-way by KV head, page 256, 1 appended token per sequence")
        n_replays = g["replays"] if g else 0
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "strong" if args.workload == "long" else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": desc,
                       "global_batch": n_seq, "kv_bytes_per_gpu": kv_bytes,
                       "kv_bytes_per_gpu_logical": kv_logical,
                       "l2": f"KV per step ({kv_bytes / 1e9:.1f} GB per GPU) exceeds L2 (126 MB); no flush needed",
                       "parallelism": f"kv-head-shard{world}"},
            "timing": {"method": f"one CUDA graph of {args.steps} steps replayed {n_replays} times, an event pair per replay; "
                                 "value from the median replay (max over ranks); the two-launch form of the step is replayed in turn with it" if g else "kernels launched one by one",
                       "replays": n_replays, "ms_per_step_min": step_min, "ms_per_step_max": step_max,
                       "timed_region_s": g["timed_s"] if g else eager_ms * args.steps / 1e3},
            "e2e": {"value": job_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": h2d_by_mode.get(e2e_mode, h2d), "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "launch": "cuda graph replay" if e2e_graphed else "eager", "mode": e2e_mode,
                    "ms_per_step_by_mode": e2e_all,
                    "modes": "staged = one H2D copy of all inputs + one D2H copy of the output; out_host = the kernel "
                             "writes the output into pinned host memory; q_out_host = it also reads q from pinned host memory; "
                             "all_host = the one-launch step reads q, k, v from pinned host memory, only lengths and block "
                             "tables are copied; all_host_resident_metadata = the same with lengths and block tables kept on "
                             "the device between steps"},
            "gpu_launches": args.steps * max(n_replays, 1),
            "step": "append + paged decode attention in ONE launch (paged_attn_decode_append); the same step as the "
                    "reference's two calls (store_kvcache, then attention) is timed beside it",
            "ms_per_step_two_launches": r["graph_two_launches"],
            "launch": "cuda graph replay of the K steps" if g else "one launch per kernel",
            "value_launched_one_by_one": job_bytes / (eager_ms * 1e-3) / 1e9, "ms_per_step_launched_one_by_one": eager_ms,
            "roofline": {"bound": "hbm", "kernel": "decode_tma_kernel", "achieved": achieved,
                         "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                         "frac_of_8000": achieved / 8000.0, "launch_ms": launch_ms,
                         "timing": ("average duration of the kernel's launches inside the replayed graph of K one-launch "
                                    "steps (CUDA events around every replay, median replay / K)") if g else
                                   "CUDA events around every eager decode call",
                         "events_around_every_eager_call": {"achieved": achieved_per_call, "frac": achieved_per_call / peak,
                                                            "note": "decode after a separate append; includes the gap between launches"},
                         "decode_ms": decode_ms,
                         "decode_ms_median": r["decode_ms_median"], "decode_ms_min": r["decode_ms_min"],
                         "traffic": kv_bytes * DECODE_TRAFFIC_PER_KV_BYTE,
                         "traffic_note": "DRAM bytes per decode launch: ncu capture of a batch-16 case (253.5 MB read + "
                                         "written for 249.9 MB of KV), scaled by KV bytes"},
            "append": {"decode_shape_us": append_ms * 1e3, "decode_shape_tok_s": n_seq / (append_ms * 1e-3),
                       "bulk_rows": n_bulk, "bulk_tok_s": n_bulk / (bulk_ms * 1e-3),
                       "bulk_gbs": bulk_bytes / (bulk_ms * 1e-3) / 1e9, "bulk_frac": bulk_bytes / (bulk_ms * 1e-3) / 1e9 / peak,
                       "bulk2_rows": n_bulk2 if bulk2_ms else 0,
                       "bulk2_tok_s": n_bulk2 / (bulk2_ms * 1e-3) if bulk2_ms else None,
                       "bulk2_gbs": bulk2_bytes / (bulk2_ms * 1e-3) / 1e9 if bulk2_ms else None},
            "clocks": clocks.summary(),
        }
        for key, obj in (("fp8_kv", fp8), ("fused_append", fused), ("prefill", prefill), ("strong", strong), ("engine", engine),
                         ("validated", validated), ("reference_gpu", flash), ("cpu_baseline", cpu)):
            if obj is not None:
                line[key] = obj
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
