#!/usr/bin/env python
"""Benchmark of the W4 decode matmul (BASELINE.json config 2) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: int4 block-quantized weights W [K=4096 -> N=14336], group 32, fp32
activations [M,4096]; the headline is M=1 (decode), M=4 and M=16 are reported
beside it. One "step" is one matmul over each of COPIES distinct weight
matrices (COPIES x 36.7 MB > the 126 MB L2, so every launch streams its
weights from HBM). The metric is algorithmic HBM GB/s: the bytes one call has
to move (packed nibbles + scales + activations + outputs) divided by time.

Arms
  default            the CUDA library through its C ABI (device-resident timing
                     for `value`, host activations/outputs for `e2e`)
  --impl reference   the reference's CPU path (AVX-512 restatement under
                     oracle/, the reference being Rust and not buildable here),
                     all host threads, same workload and metric
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

K, N, GROUP = 4096, 14336, 32
COPIES = 16
M_HEADLINE = 1
M_EXTRA = (4, 16)


def algorithmic_bytes(m: int) -> int:
    """Bytes one call must move: nibbles + scales + activations + outputs."""
    return N * K // 2 + N * (K // GROUP) * 4 + m * K * 4 + m * N * 4


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.rows.append([time.perf_counter()] + parts)

    def stop(self, t0=None, t1=None):
        """Summary of the samples that arrived inside [t0, t1] (host clock)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [r[1:] for r in self.rows if t0 is None or t0 <= r[0] <= t1]
        window = "timed region"
        if not rows:
            rows, window = [r[1:] for r in self.rows], "whole run (no sample landed in the timed region)"
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(rows), "window": window}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ----------------------------------------------------------------------------------
# reference arm: the reference's CPU path, all host threads
# ----------------------------------------------------------------------------------

def cpu_workload(oracle, seed=1):
    """One packed weight (seeded normal, std 0.02) replicated COPIES times in host
    memory, plus an activation row per M."""
    from yscv_b200 import synth
    w = synth.normal(seed, 0, 1024 * K, 0.02)
    packed_1k, scales_1k = oracle.pack_int4(w, 1024, K, GROUP)
    reps = N // 1024
    packed = np.tile(packed_1k, reps)
    scales = np.tile(scales_1k, reps)
    copies = [(packed.copy(), scales.copy()) for _ in range(COPIES)]
    return copies


def time_cpu(oracle, copies, m, threads, steps, warmup, max_copies=None):
    from yscv_b200 import synth
    act = synth.normal(1, 1, m * K, 1.0)
    use = copies if max_copies is None else copies[:max_copies]
    for _ in range(warmup):
        for p, s in use:
            oracle.exec_matmul_int4(p, s, act, m, N, K, GROUP, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        for p, s in use:
            oracle.exec_matmul_int4(p, s, act, m, N, K, GROUP, threads=threads)
    dt = time.perf_counter() - t0
    calls = steps * len(use)
    return algorithmic_bytes(m) * calls / dt / 1e9, dt / steps * 1e3, calls


def cpu_int8_baselines(oracle, threads):
    """The reference's int8 GEMM (AVX-512-VNNI restatement, prepacked B) on the host cores:
    BASELINE configs[0] in full and a bounded row sample of configs[2]; one thread (what the
    reference kernel does) and rows split over `threads` threads."""
    import numpy as np
    out = {}
    rng = np.random.default_rng(2)
    for name, (m, k, n), sample_m in (("matmul_integer_64x1024x1024", (64, 1024, 1024), 64),
                                      ("qlinear_matmul_2048x4096x4096", (2048, 4096, 4096), 256)):
        a = rng.integers(-128, 128, size=(sample_m, k), dtype=np.int8)
        b = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
        bt = oracle.transpose_b_i8(b, k, n)
        ops = 2.0 * sample_m * k * n
        res = {"sample": f"{sample_m} of {m} rows of A, prepacked B, i32 accumulate (the requant pass is not timed)"}
        for label, t, rows, reps in (("threads", threads, sample_m, 3), ("one_thread", 1, min(sample_m, 64), 2)):
            aa = np.ascontiguousarray(a[:rows])
            oracle.int8_matmul_prepacked(aa, bt, rows, k, n, simd=True, threads=t)
            t0 = time.perf_counter()
            for _ in range(reps):
                oracle.int8_matmul_prepacked(aa, bt, rows, k, n, simd=True, threads=t)
            dt = (time.perf_counter() - t0) / reps
            res[f"tops_{label}"] = 2.0 * rows * k * n / dt / 1e12
        res["cores"] = threads
        out[name] = res
    return out


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle_lib
    oracle = oracle_lib.load()
    threads = os.cpu_count() or 1
    copies = cpu_workload(oracle)
    steps = max(1, min(args.steps, 40))  # bounded sample: a step is ~30 ms of CPU work
    gbs, ms, calls = time_cpu(oracle, copies, M_HEADLINE, threads, steps, max(1, min(args.warmup, 2)))
    line = {
        "impl": "reference",
        "metric": "w4_decode_gemv_hbm_gbs", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "isa": oracle.isa(),
                         "sample": f"{calls} calls of the M=1 GEMV over {COPIES} weight copies, "
                                   f"weight rows split across {threads} threads "
                                   "(the reference kernel itself is single-threaded)"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config():
    return {"workload": f"BASELINE configs[1]: W4A32 block-quantized matmul, K={K} N={N} group={GROUP}, "
                        f"M=1 headline (M=4,16 in by_m), seeded synthetic N(0,0.02) weights / N(0,1) activations",
            "k": K, "n": N, "group_size": GROUP, "m": M_HEADLINE, "weight_copies_per_step": COPIES,
            "l2_policy": f"inputs larger than L2: each step streams {COPIES} distinct weight matrices "
                         f"({COPIES * (N * K // 2 + N * (K // GROUP) * 4) / 1e6:.0f} MB)"}


# ----------------------------------------------------------------------------------
# CUDA arm
# ----------------------------------------------------------------------------------

def run_cuda(args):
    import torch
    import yscv_b200

    rank, world, local = dist_env()
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    stream = torch.cuda.Stream(device=dev)
    ctx = yscv_b200.Context(local, stream=stream.cuda_stream)

    # ---- synthetic weights, packed on the GPU by the library's own packer ----
    weights = []
    with torch.cuda.stream(stream):
        gen = torch.Generator(device=dev)
        for c in range(COPIES):
            gen.manual_seed(1000 * (rank + 1) + c)
            w = torch.randn(N, K, device=dev, generator=gen) * 0.02
            packed = torch.empty(N * K // 2, dtype=torch.uint8, device=dev)
            scales = torch.empty(N * (K // GROUP), dtype=torch.float32, device=dev)
            ctx.pack_int4_dev(w.data_ptr(), N, K, GROUP, packed.data_ptr(), scales.data_ptr())
            weights.append((packed, scales, ctx.int4_weight_wrap(packed.data_ptr(), scales.data_ptr(), N, K, GROUP)))
            if c == 0:
                w0 = w
            del w
        gen.manual_seed(7)
        acts = {m: torch.randn(m, K, device=dev, generator=gen) for m in (M_HEADLINE, *M_EXTRA)}
        outs = {m: torch.empty(m, N, device=dev) for m in acts}
    stream.synchronize()

    # ---- sanity: the timed kernel really computes the matmul (fp32 torch dequant check) ----
    with torch.cuda.stream(stream):
        p0, s0, h0 = weights[0]
        lo = (p0 & 15).to(torch.int8)
        hi = (p0 >> 4).to(torch.int8)
        lo = torch.where(lo > 7, lo - 16, lo)
        hi = torch.where(hi > 7, hi - 16, hi)
        q = torch.stack([lo, hi], dim=1).reshape(N, K).float()
        deq = q * s0.reshape(N, K // GROUP).repeat_interleave(GROUP, dim=1)
        want = acts[16] @ deq.T
        ctx.int4_matmul_dev(h0, acts[16].data_ptr(), outs[16].data_ptr(), 16)
        check = float((outs[16] - want).abs().max() / want.abs().max())
        del lo, hi, q, deq, want, w0
    stream.synchronize()
    if not check < 1e-3:
        raise SystemExit(f"bench sanity check failed: rel err {check}")
    torch.cuda.empty_cache()

    def one_step(m):
        a, o = acts[m].data_ptr(), outs[m].data_ptr()
        for _, _, h in weights:
            ctx.int4_matmul_dev(h, a, o, m)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()

    def timed(m, steps, warmup, sample_clocks=False):
        with torch.cuda.stream(stream):
            sampler = ClockSampler(local) if sample_clocks else None
            if sampler:
                sampler.start()
                t_up = time.perf_counter()   # nvidia-smi takes a moment to print its first line
                while not sampler.rows and time.perf_counter() - t_up < 3.0:
                    one_step(m)
                    stream.synchronize()
            for _ in range(warmup):
                one_step(m)
            stream.synchronize()
            barrier()
            torch.cuda.synchronize()
            l0 = ctx.launch_count()
            t_begin = time.perf_counter()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                one_step(m)
            e1.record(stream)
            torch.cuda.synchronize()
            barrier()
            ms = e0.elapsed_time(e1)
            t_end = time.perf_counter()
            launches = ctx.launch_count() - l0
            if sampler and not any(t_begin <= r[0] <= t_end for r in sampler.rows):
                # the timed region was shorter than the sampling period: keep the same load
                # running (untimed) until a few samples have landed and report those
                t_begin = time.perf_counter()
                while time.perf_counter() - t_begin < 0.25:
                    one_step(m)
                stream.synchronize()
                t_end = time.perf_counter()
                clocks = sampler.stop(t_begin, t_end)
                clocks["window"] = "the same load continued right after the timed region (the region itself is shorter than the 20 ms sampling period)"
            else:
                clocks = sampler.stop(t_begin, t_end) if sampler else None
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, launches, clocks

    steps, warmup = max(1, args.steps), max(3, args.warmup)
    ms, launches, clocks = timed(M_HEADLINE, steps, warmup, sample_clocks=True)
    calls = steps * COPIES
    value = algorithmic_bytes(M_HEADLINE) * calls * world / (ms * 1e-3) / 1e9

    by_m = {}
    for m in M_EXTRA:
        ms_m, _, _ = timed(m, max(5, steps // 4), max(3, warmup // 4))
        c_m = max(5, steps // 4) * COPIES
        by_m[str(m)] = {"gbs": algorithmic_bytes(m) * c_m * world / (ms_m * 1e-3) / 1e9,
                        "us_per_call": ms_m * 1e3 / c_m}

    # ---- roofline of the dominant kernel: CUDA events around it, on its stream ----
    peak, peak_kind = load_peaks()
    ctx.profile_enable(True)
    with torch.cuda.stream(stream):
        for _ in range(max(5, min(steps // 4, 100))):
            one_step(M_HEADLINE)
    n_prof, prof_ms = ctx.profile_read()
    ctx.profile_enable(False)
    iso_us = prof_ms * 1e3 / max(n_prof, 1)
    # The timed region launches nothing but the dominant kernel (kernels_per_call == 1), so its
    # average launch duration over that region is region time / launches. Consecutive launches
    # overlap their start-up with the predecessor's tail (programmatic dependent launch); the
    # same kernel bracketed by its own pair of events, which serialises it, is reported beside it.
    kern_us = ms * 1e3 / max(launches, 1)
    achieved = algorithmic_bytes(M_HEADLINE) / (kern_us * 1e-6) / 1e9
    roofline = {"bound": "hbm", "kernel": ctx.last_kernel(), "achieved": achieved, "peak": peak,
                "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                "frac_of_nominal_8000": achieved / 8000.0,
                "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "algorithmic_bytes": algorithmic_bytes(M_HEADLINE),
                "us_per_launch": kern_us, "launches_timed": launches,
                "us_per_launch_isolated": iso_us, "achieved_isolated": algorithmic_bytes(M_HEADLINE) / (iso_us * 1e-6) / 1e9,
                "launches_isolated": n_prof}

    # ---- e2e: the operator call a runner makes (resident weights, host activations) ----
    e2e_steps = max(3, min(steps // 4, 100))
    host_act = torch.randn(M_HEADLINE, K).pin_memory()
    host_out = torch.empty(M_HEADLINE, N).pin_memory()
    a_np, o_np = host_act.numpy(), host_out.numpy()
    for _ in range(3):
        for _, _, h in weights:
            ctx.int4_matmul(h, a_np, M_HEADLINE, out=o_np)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        for _, _, h in weights:
            ctx.int4_matmul(h, a_np, M_HEADLINE, out=o_np)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([dt], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    e2e_calls = e2e_steps * COPIES
    # the same calls from pageable host memory (what a caller that never pinned its buffers gets)
    a_pg, o_pg = np.array(a_np), np.empty_like(o_np)
    for _, _, h in weights:
        ctx.int4_matmul(h, a_pg, M_HEADLINE, out=o_pg)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        for _, _, h in weights:
            ctx.int4_matmul(h, a_pg, M_HEADLINE, out=o_pg)
    torch.cuda.synchronize()
    dt_pg = time.perf_counter() - t0
    e2e_ok = bool(np.array_equal(o_pg, o_np))
    e2e = {"value": algorithmic_bytes(M_HEADLINE) * e2e_calls * world / dt / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": COPIES * M_HEADLINE * K * 4, "d2h_bytes_per_step": COPIES * M_HEADLINE * N * 4,
           "us_per_call": dt * 1e6 / e2e_calls,
           "us_per_call_pageable_buffers": dt_pg * 1e6 / e2e_calls,
           "pinned_equals_pageable_result": e2e_ok,
           "api": "yscv_cuda_int4_matmul (weights uploaded once at load time, pinned host activation "
                  "copied in, output written by the kernel into the caller's pinned buffer, synchronised per call; "
                  "pageable buffers go through a staging copy each way)"}

    # ---- CPU baseline beside it (rank 0, N=1 only): bounded sample ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sys.path.insert(0, str(ROOT / "oracle"))
        import oracle_lib
        oracle = oracle_lib.load()
        threads = os.cpu_count() or 1
        copies = cpu_workload(oracle)
        g1, _, c1 = time_cpu(oracle, copies, M_HEADLINE, 1, 2, 1, max_copies=8)
        gt, _, ct = time_cpu(oracle, copies, M_HEADLINE, threads, 6, 1)
        cpu = {"value": gt, "unit": "GB/s", "cores": threads, "kind": "port", "isa": oracle.isa(),
               "single_thread_value": g1,
               "sample": f"M=1 GEMV, AVX-512 restatement of the reference kernel: {ct} calls with weight rows "
                         f"split across {threads} threads; single_thread_value from {c1} calls on 1 thread "
                         "(the reference kernel is single-threaded)"}

    # ---- the other two quantities of BASELINE's metric, measured beside the headline ----
    other = None
    if not args.no_extras:
        # release the headline's 590 MB of weights first: the 70B-shape decoder wants the room
        weights.clear()
        acts.clear()
        outs.clear()
        del p0, s0, h0
        torch.cuda.empty_cache()
        other = extra_metrics(ctx, stream, dev) if world == 1 else {}
        if other is not None and cpu is not None:
            for name, res in cpu_int8_baselines(oracle, threads).items():
                other[name]["cpu_baseline"] = res
        sharded = sharded_metrics(world)      # every rank takes part
        if rank == 0:
            other.update(sharded)
            if world == 1:  # the same run under the name earlier result files carry
                other["int4_decoder_llama70b_b1"] = other["int4_decoder_llama70b_tp"]

    if rank == 0:
        line = {
            "metric": "w4_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(),
            "us_per_call": ms * 1e3 / calls,
            "by_m": by_m,
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": launches,
            "kernels_per_call": launches / calls,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "other_metrics": other,
            "sanity_rel_err_vs_torch_fp32": check,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def extra_metrics(ctx, stream, dev):
    """int8 GEMM TOPS on BASELINE configs[2] (QLinearMatMul 2048x4096x4096, uint8 in/out) and
    configs[0] (MatMulInteger 64x1024x1024), and decode tokens/s of the TinyLlama-1.1B-shape
    int4 decoder (configs[3], batch 1 / 8 / 32, 128-token prompt, 128 greedy steps)."""
    import torch
    from yscv_b200.llm_bench import run as llm_run
    out = {}
    with torch.cuda.stream(stream):
        for name, (m, k, n), reps in (("qlinear_matmul_2048x4096x4096", (2048, 4096, 4096), 50),
                                      ("matmul_integer_64x1024x1024", (64, 1024, 1024), 200)):
            a = torch.randint(0, 256, (m, k), dtype=torch.uint8, device=dev)
            b = torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev)
            pk = ctx.pack_i8_b_dev(b.data_ptr(), k, n)
            o8 = torch.empty(m, n, dtype=torch.uint8, device=dev)
            o32 = torch.empty(m, n, dtype=torch.int32, device=dev)
            rq = ctx.requant(1e-4, 128.0, 0, 255, a_unsigned=True, a_zp=128)
            if name.startswith("qlinear"):
                f = lambda: ctx.qlinear_matmul_dev(a.data_ptr(), pk, m, rq, o8.data_ptr())
            else:
                f = lambda: ctx.matmul_integer_dev(a.data_ptr(), True, 128, pk, m, o32.data_ptr())
            for _ in range(5):
                f()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                f()
            e1.record(stream)
            stream.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            out[name] = {"us_per_call": us, "tops": 2.0 * m * k * n / us / 1e6, "kernel": ctx.last_kernel(),
                         "frac_of_nominal_4500_tops": 2.0 * m * k * n / us / 1e6 / 4500.0}
            pk.free()
    stream.synchronize()
    for batch in (1, 8, 32):   # configs[3]: batch 1 / 8 / 32
        d = llm_run("tinyllama", batch=batch, prompt_len=128, max_tokens=128, warmup=1)
        out[f"int4_decoder_tinyllama_b{batch}"] = {k: d[k] for k in LLM_KEYS}
        torch.cuda.empty_cache()
    return out


LLM_KEYS = ("decode_tokens_per_sec", "ms_per_step", "prefill_ms", "weight_stream_gbs_per_gpu", "decode_step",
            "kv_cache", "device_status")


def sharded_metrics(world):
    """The workloads BASELINE shards across the GPUs of the job, run at tensor-parallel degree
    = number of ranks (also 1): the Llama-3-70B-shape int4 decoder (configs[4]: batch 1, prompt
    2048, 32 greedy steps; column-parallel qkv / gate / up, row-parallel output / down, the
    partial sums exchanged inside the decode-step kernel) with its gate "greedy tokens equal the
    one-GPU decoder's for 32 steps" on a 2-layer truncation, and QLinearMatMul configs[2]
    sharded over output channels (bit-exact gate inside). Every rank calls this; rank 0 gets the
    numbers."""
    import torch
    from yscv_b200 import int8_shard_bench
    from yscv_b200.llm_bench import run as llm_run, tokens_match_single_gpu
    out = {}
    try:
        gate = tokens_match_single_gpu("llama70b", layers=2, prompt_len=64, steps=32)
        torch.cuda.empty_cache()
        d = llm_run("llama70b", batch=1, prompt_len=2048, max_tokens=32, warmup=0)
        res = {k: d[k] for k in LLM_KEYS}
        res.update({"tensor_parallel": world, "tokens_equal_one_gpu_32_steps_2_layers": gate,
                    "workload": "BASELINE configs[4]: batch 1, prompt 2048, 32 greedy steps, 80 layers"})
        out["int4_decoder_llama70b_tp"] = res
    except Exception as e:  # e.g. not enough free memory on a shared GPU: report, do not fail the bench
        out["int4_decoder_llama70b_tp"] = {"error": f"{type(e).__name__}: {e}"[:300], "tensor_parallel": world}
    torch.cuda.empty_cache()
    try:
        out["qlinear_matmul_nshard"] = int8_shard_bench.run(2048, 4096, 4096, iters=30)
    except Exception as e:
        out["qlinear_matmul_nshard"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    return out


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel,
# from the ncu capture summarised under profiles/ (None until captured).
NCU_DRAM_BYTES_PER_LAUNCH = 36_762_880  # 36.763 MB read + 0 written: dram__bytes of one launch (profiles/int4_gemv_fast_m1_k4096_n14336.md)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the int8 GEMM and decoder side measurements")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
