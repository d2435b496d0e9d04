"""Kernel microbenchmark, the counterpart of apps/llm-bench/src/bin/kernel_bench.rs:
the same three sections (int8 GEMM, int4 GEMV, int4 GEMM), LLM-linear shape tables of the
same kind plus the BASELINE configurations, a parity gate before every timing, and the
same derived figures (weight bandwidth N*K/2 / t for the GEMV, kernel_bench.rs:317-324;
2*M*N*K / t for the GEMMs, :389-396), median and min over the timed iterations (:54-69).

    python -m yscv_b200.kernel_bench [--section int8|conv1x1|int4_gemv|int4_gemm|attention|lm_head] [--only SUBSTR]
                                     [--iters N] [--copies C]

The parity gate recomputes a random sample of outputs on the GPU in float64 from the raw
operands (torch, exact for the integer kernels) - independent of the kernels under test.
`--only` selects shapes by label (used to profile one shape under ncu).
"""
from __future__ import annotations

import argparse
import statistics

import torch

from . import Context

INT8_SHAPES = [
    ("BASELINE cfg1 MatMulInteger 64x1024x1024", 64, 1024, 1024),
    ("BASELINE cfg3 QLinearMatMul 2048x4096x4096", 2048, 4096, 4096),
    ("TLlama  Q/K/V    64x2048x2048", 64, 2048, 2048),
    ("TLlama  gate/up  64x2048x5632", 64, 2048, 5632),
    ("TLlama  down     64x5632x2048", 64, 5632, 2048),
    ("TLlama  vocab    64x2048x32000", 64, 2048, 32000),
    ("Llama-7B Q/K/V   64x4096x4096", 64, 4096, 4096),
    ("Llama-7B gate/up 64x4096x11008", 64, 4096, 11008),
    ("Llama-7B down    64x11008x4096", 64, 11008, 4096),
    ("M-sweep 256x2048x2048", 256, 2048, 2048),
    ("square 4096x4096x4096", 4096, 4096, 4096),
    ("square 8192x8192x8192", 8192, 8192, 8192),
]

# pointwise (1x1) QLinearConv as a GEMM over NHWC pixels: (label, pixels, c_in, c_out)
CONV1X1_SHAPES = [
    ("56x56  64->256", 3136, 64, 256),
    ("28x28 128->512", 784, 128, 512),
    ("14x14 256->1024", 196, 256, 1024),
    ("7x7  512->2048", 49, 512, 2048),
    ("8 x 56x56 64->256", 25088, 64, 256),
    ("8 x 14x14 1024->256", 1568, 1024, 256),
]

INT4_GEMV_SHAPES = [  # (label, N, K); timed at M = 1, 4, 16
    ("BASELINE cfg2 14336x4096", 14336, 4096),
    ("TLlama Q/K/V/out 2048x2048", 2048, 2048),
    ("TLlama gate/up   5632x2048", 5632, 2048),
    ("TLlama down      2048x5632", 2048, 5632),
    ("L3.2-1B gate/up  8192x2048", 8192, 2048),
    ("L3-70B qkv      10240x8192", 10240, 8192),
    ("L3-70B gate+up  57344x8192", 57344, 8192),
    ("L3-70B down      8192x28672", 8192, 28672),
]

INT4_GEMM_SHAPES = [  # (label, M, N, K)
    ("TLlama prefill M=32  2048x2048", 32, 2048, 2048),
    ("TLlama prefill M=128 2048x2048", 128, 2048, 2048),
    ("TLlama prefill M=128 5632x2048", 128, 5632, 2048),
    ("TLlama prefill M=128 2048x5632", 128, 2048, 5632),
    ("L3-70B decode batch M=64 10240x8192", 64, 10240, 8192),
    ("L3-70B decode batch M=64 57344x8192", 64, 57344, 8192),
    ("L3-70B decode batch M=64 8192x28672", 64, 8192, 28672),
    ("cfg2 weights M=2048 14336x4096", 2048, 14336, 4096),
    ("L3-70B prefill M=2048 8192x8192", 2048, 8192, 8192),
    ("L3-70B prefill M=2048 8192x28672", 2048, 8192, 28672),
]


def time_us(stream, fn, iters, warmup=5):
    """Median and min device time of fn() in microseconds (CUDA events on the stream)."""
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            fn()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for a, b in evs:
            a.record(stream)
            fn()
            b.record(stream)
    stream.synchronize()
    ts = [a.elapsed_time(b) * 1e3 for a, b in evs]
    return statistics.median(ts), min(ts)


def time_b2b_us(stream, fn, iters, warmup=5, rounds=3):
    """Device time per call of `iters` calls enqueued back to back between two CUDA events (best of
    `rounds`): no event record between the launches, so no bubble around each kernel."""
    best = float("inf")
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            fn()
        for _ in range(rounds):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(iters):
                fn()
            b.record(stream)
            stream.synchronize()
            best = min(best, a.elapsed_time(b) * 1e3 / iters)
    return best


def sample_idx(rows, cols, count, dev):
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    r = torch.randint(0, rows, (count,), device=dev, generator=g)
    c = torch.randint(0, cols, (count,), device=dev, generator=g)
    return r, c


def bench_int8(ctx, stream, dev, iters, only, calibrate=False):
    print("\n== INT8 GEMM (tcgen05, i32 accumulate; QLinearMatMul = + requant to u8) ==")
    for label, m, k, n in INT8_SHAPES:
        if only and only not in label:
            continue
        with torch.cuda.stream(stream):
            g = torch.Generator(device=dev)
            g.manual_seed(0xAA)
            a = torch.randint(0, 256, (m, k), dtype=torch.uint8, device=dev, generator=g)
            b = torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev, generator=g)
            pk = ctx.pack_i8_b_dev(b.data_ptr(), k, n)
            o32 = torch.empty(m, n, dtype=torch.int32, device=dev)
            o8 = torch.empty(m, n, dtype=torch.uint8, device=dev)
            ctx.matmul_integer_dev(a.data_ptr(), True, 128, pk, m, o32.data_ptr())
            r, c = sample_idx(m, n, 4096, dev)
            want = ((a[r].double() - 128.0) * b[:, c].t().double()).sum(dim=1)
            bad = int((o32[r, c].double() != want).sum())
        stream.synchronize()
        assert bad == 0, f"{label}: {bad} of 4096 sampled outputs differ"
        rq = ctx.requant(1e-4, 128.0, 0, 255, a_unsigned=True, a_zp=128)
        med, mn = time_us(stream, lambda: ctx.matmul_integer_dev(a.data_ptr(), True, 128, pk, m, o32.data_ptr()), iters)
        medq, mnq = time_us(stream, lambda: ctx.qlinear_matmul_dev(a.data_ptr(), pk, m, rq, o8.data_ptr()), iters)
        ops = 2.0 * m * k * n
        bb = time_b2b_us(stream, lambda: ctx.matmul_integer_dev(a.data_ptr(), True, 128, pk, m, o32.data_ptr()), iters)
        bbq = time_b2b_us(stream, lambda: ctx.qlinear_matmul_dev(a.data_ptr(), pk, m, rq, o8.data_ptr()), iters)
        print(f"  {label:46s} i32: med {med:9.2f} us min {mn:9.2f} us {ops / mn / 1e6:8.1f} TOPS | "
              f"requant-u8: min {mnq:9.2f} us {ops / mnq / 1e6:8.1f} TOPS  [{ctx.last_kernel()}]  parity: bit-exact")
        print(f"  {'':46s} back to back (no event between launches): i32 {bb:9.2f} us {ops / bb / 1e6:8.1f} TOPS | "
              f"requant-u8 {bbq:9.2f} us {ops / bbq / 1e6:8.1f} TOPS")
        if calibrate and m % 8 == 0 and k % 8 == 0 and n % 8 == 0 and m > 16:
            # CALIBRATION ONLY: what the vendor's own int8 GEMM (cuBLASLt through torch._int_mm)
            # reaches on this shape and this GPU, the practical ceiling of the int8 tensor pipe.
            # Never part of the library's code path.
            with torch.cuda.stream(stream):
                a8 = (a.to(torch.int16) - 128).to(torch.int8)
                lib = torch._int_mm(a8, b)
                same = bool(torch.equal(lib, o32))
            lmed, lmn = time_us(stream, lambda: torch._int_mm(a8, b), iters)
            lbb = time_b2b_us(stream, lambda: torch._int_mm(a8, b), iters)
            print(f"  {'':46s} calibration, library int8 GEMM (cuBLASLt, i32 out): min {lmn:9.2f} us "
                  f"{ops / lmn / 1e6:8.1f} TOPS, back to back {lbb:9.2f} us {ops / lbb / 1e6:8.1f} TOPS  "
                  f"same result: {same}")
        pk.free()


def bench_conv1x1(ctx, stream, dev, iters, only):
    print("\n== INT8 pointwise QLinearConv (GEMM + per-channel i8 requant in the epilogue) ==")
    for label, m, k, n in CONV1X1_SHAPES:
        if only and only not in label:
            continue
        with torch.cuda.stream(stream):
            g = torch.Generator(device=dev)
            g.manual_seed(0xC0)
            a = torch.randint(-128, 128, (m, k), dtype=torch.int8, device=dev, generator=g)
            b = torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev, generator=g)
            corr = torch.randint(-4000, 4000, (n,), dtype=torch.int32, device=dev, generator=g)
            comp = (0.0005 + 0.0001 * (torch.arange(n, device=dev) % 7)).float()
            pk = ctx.pack_i8_b_dev(b.data_ptr(), k, n)
            out = torch.empty(m, n, dtype=torch.int8, device=dev)
            ctx.int8_matmul_requant_per_channel_dev(a.data_ptr(), pk, m, corr.data_ptr(), comp.data_ptr(), -2.0,
                                                    out.data_ptr())
            # gate: exact accumulator (float64 is exact here), then the requant contract in fp32
            acc = (a.double() @ b.double()).to(torch.int32) + corr
            want = torch.clamp(torch.round(acc.float() * comp + (-2.0)), -128, 127).to(torch.int8)
            bad = int((out != want).sum())
        stream.synchronize()
        assert bad == 0, f"{label}: {bad} outputs differ"
        med, mn = time_us(stream, lambda: ctx.int8_matmul_requant_per_channel_dev(
            a.data_ptr(), pk, m, corr.data_ptr(), comp.data_ptr(), -2.0, out.data_ptr()), iters)
        ops = 2.0 * m * k * n
        byts = m * k + k * n + m * n
        print(f"  {label:22s} [{m}x{k}x{n}]: med {med:8.2f} us min {mn:8.2f} us {ops / mn / 1e6:8.1f} TOPS "
              f"{byts / mn / 1e3:7.1f} GB/s  [{ctx.last_kernel()}]  parity: bit-exact")
        pk.free()


def make_int4(ctx, dev, n, k, seed):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    w = torch.randn(n, k, device=dev, generator=g) * 0.02
    packed = torch.empty(n, k // 2, dtype=torch.uint8, device=dev)
    scales = torch.empty(n, k // 32, dtype=torch.float32, device=dev)
    ctx.pack_int4_dev(w.data_ptr(), n, k, 32, packed.data_ptr(), scales.data_ptr())
    return packed, scales, ctx.int4_weight_wrap(packed.data_ptr(), scales.data_ptr(), n, k, 32)


def int4_reference_rows(packed, scales, act, rows):
    """float64 dequantised reference of output columns `rows` (weight rows) for all of act."""
    p = packed[rows].to(torch.int16)
    lo, hi = p & 15, p >> 4
    lo = torch.where(lo > 7, lo - 16, lo)
    hi = torch.where(hi > 7, hi - 16, hi)
    q = torch.stack([lo, hi], dim=2).reshape(len(rows), -1).double()
    w = q * scales[rows].double().repeat_interleave(32, dim=1)
    return act.double() @ w.t()


def bench_int4_gemv(ctx, stream, dev, iters, only, copies):
    print("\n== INT4 packed GEMV / small-M matmul (decode) ==")
    for label, n, k in INT4_GEMV_SHAPES:
        if only and only not in label:
            continue
        with torch.cuda.stream(stream):
            # rotate over several copies so that every timed call streams from HBM, not L2
            c = max(1, min(copies, int(1.5e9 // (n * k * 0.625))))
            ws = [make_int4(ctx, dev, n, k, 7 + i) for i in range(c)]
        for m in (1, 4, 16):
            with torch.cuda.stream(stream):
                g = torch.Generator(device=dev)
                g.manual_seed(0xBB + m)
                act = torch.randn(m, k, device=dev, generator=g)
                out = torch.empty(m, n, device=dev)
                ctx.int4_matmul_dev(ws[0][2], act.data_ptr(), out.data_ptr(), m)
                rows = torch.arange(0, n, max(1, n // 512), device=dev)
                want = int4_reference_rows(ws[0][0], ws[0][1], act, rows)
                err = float((out[:, rows].double() - want).abs().max() / want.abs().max())
            stream.synchronize()
            assert err <= 1e-4, f"{label} M={m}: rel err {err}"
            state = {"i": 0}

            def call():
                ctx.int4_matmul_dev(ws[state["i"] % c][2], act.data_ptr(), out.data_ptr(), m)
                state["i"] += 1
            med, mn = time_us(stream, call, iters, warmup=max(5, c))
            wb = n * k / 2
            allb = wb + n * (k // 32) * 4 + m * k * 4 + m * n * 4
            print(f"  {label:30s} M={m:2d}: med {med:8.2f} us min {mn:8.2f} us  weight BW {wb / med / 1e3:7.1f} GB/s  "
                  f"all bytes {allb / med / 1e3:7.1f} GB/s  rel err {err:.1e}  [{ctx.last_kernel()}]")


def bench_int4_gemm(ctx, stream, dev, iters, only):
    print("\n== INT4 packed GEMM (prefill, bf16 tcgen05) ==")
    for label, m, n, k in INT4_GEMM_SHAPES:
        if only and only not in label:
            continue
        with torch.cuda.stream(stream):
            packed, scales, h = make_int4(ctx, dev, n, k, 3)
            g = torch.Generator(device=dev)
            g.manual_seed(0xCC)
            act = torch.randn(m, k, device=dev, generator=g)
            out = torch.empty(m, n, device=dev)
            ctx.int4_matmul_dev(h, act.data_ptr(), out.data_ptr(), m)
            rows = torch.arange(0, n, max(1, n // 256), device=dev)
            want = int4_reference_rows(packed, scales, act, rows)
            err = float(torch.linalg.norm(out[:, rows].double() - want) / torch.linalg.norm(want))
        stream.synchronize()
        assert err <= 2e-2, f"{label}: relative Frobenius error {err}"
        med, mn = time_us(stream, lambda: ctx.int4_matmul_dev(h, act.data_ptr(), out.data_ptr(), m), iters)
        print(f"  {label:36s}: med {med:9.2f} us min {mn:9.2f} us  {2.0 * m * n * k / mn / 1e6:8.1f} TFLOP/s  "
              f"fro err {err:.1e}  [{ctx.last_kernel()}]")


def bench_attention(ctx, stream, dev, iters, only):
    """Decode attention (one query position per sequence) over int8 KV caches at the Llama-3-70B and
    TinyLlama head shapes: the fp16 tensor-core kernel and the fp32 loop on the same caches."""
    print("\n== decode attention over an int8 KV cache (one query position, 2101 cached positions) ==")
    shapes = [("L3-70B heads 64/8 x 128, 16 sequences", 16, 64, 8, 128),
              ("L3-70B heads 64/8 x 128, 64 sequences", 64, 64, 8, 128),
              ("TLlama heads 32/4 x 64, 32 sequences", 32, 32, 4, 64)]
    S, pos_v = 2178, 2100
    for label, B, nq, nkv, d in shapes:
        if only and only not in label:
            continue
        with torch.cuda.stream(stream):
            kc = torch.randint(-127, 128, (B, S, nkv * d), dtype=torch.int8, device=dev)
            vc = torch.randint(-127, 128, (B, S, nkv * d), dtype=torch.int8, device=dev)
            ks = torch.rand(B, S, device=dev) * 0.02 + 0.001
            vs = torch.rand(B, S, device=dev) * 0.02 + 0.001
            qkv_w = (nq + 2 * nkv) * d
            qkv = torch.randn(B, qkv_w, device=dev)
            out = torch.empty(B, nq * d, device=dev)
            pos = torch.full((1,), pos_v, dtype=torch.int32, device=dev)
        call = lambda: ctx.gqa_attention_i8_dev(qkv.data_ptr(), qkv_w, B, 1, nq, nkv, d, kc.data_ptr(), ks.data_ptr(),
                                                vc.data_ptr(), vs.data_ptr(), S, pos.data_ptr(), True, out.data_ptr())
        res = {}
        for tc in (True, False):
            ctx.set_attention_tensor_cores(tc)
            med, mn = time_us(stream, call, iters)
            res[tc] = (mn, out.clone(), ctx.last_kernel())
        ctx.set_attention_tensor_cores(True)
        err = float((res[True][1] - res[False][1]).abs().max() / res[False][1].abs().max())
        mb = 2 * B * (pos_v + 1) * nkv * d / 1e6
        print(f"  {label:42s}: mma {res[True][0]:8.2f} us ({mb / res[True][0] * 1e3:6.0f} GB/s of cache)  "
              f"fp32 loop {res[False][0]:8.2f} us  max diff {err:.1e}  [{res[True][2]}]")
        del kc, vc


def bench_lm_head(ctx, stream, dev, iters, only):
    """The decoder's fp32 LM head for a wide batch (yscv_cuda_f32_matmul_dev, more than 8 rows): the
    3xTF32 tensor-core kernel and the tiled fp32 FMA kernel, both against float64 on sampled outputs."""
    print("\n== fp32 LM head, wide batch (out[m][n] = sum_k x[m][k] w[n][k]) ==")
    shapes = [("TLlama vocab 32000x2048, 32 rows", 32, 32000, 2048),
              ("TLlama vocab 32000x2048, 128 rows", 128, 32000, 2048),
              ("L3-70B vocab 128256x8192, 64 rows", 64, 128256, 8192)]
    for label, m, n, k in shapes:
        if only and only not in label:
            continue
        with torch.cuda.stream(stream):
            g = torch.Generator(device=dev)
            g.manual_seed(0xF3)
            w = torch.randn(n, k, device=dev, generator=g) * 0.02
            x = torch.randn(m, k, device=dev, generator=g)
            out = torch.empty(m, n, device=dev)
            r, c = sample_idx(m, n, 4096, dev)
            want = (x[r].double() * w[c].double()).sum(dim=1)
        call = lambda: ctx.f32_matmul_dev(w.data_ptr(), x.data_ptr(), m, n, k, out.data_ptr())
        res = {}
        for tc in (True, False):
            ctx.set_f32_tensor_cores(tc)
            med, mn = time_us(stream, call, max(3, iters // 3))
            err = float((out[r, c].double() - want).abs().max() / want.abs().max())
            res[tc] = (mn, err, ctx.last_kernel())
        ctx.set_f32_tensor_cores(True)
        print(f"  {label:38s}: 3xTF32 {res[True][0]:9.2f} us ({n * k * 4 / res[True][0] / 1e6:5.2f} TB/s of weights, "
              f"rel err {res[True][1]:.1e})  fp32 FMA {res[False][0]:9.2f} us (rel err {res[False][1]:.1e})  [{res[True][2]}]")
        del w, x, out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--section", choices=["int8", "conv1x1", "int4_gemv", "int4_gemm", "attention", "lm_head"], default=None)
    ap.add_argument("--only", default=None, help="substring of the shape label")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--copies", type=int, default=16)
    ap.add_argument("--calibrate-int8", action="store_true",
                    help="also time the vendor library's int8 GEMM on every int8 shape (calibration of the "
                         "tensor-pipe ceiling only)")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream()
    ctx = Context(0, stream=stream.cuda_stream)
    if a.section in (None, "int8"):
        bench_int8(ctx, stream, dev, a.iters, a.only, a.calibrate_int8)
    if a.section in (None, "conv1x1"):
        bench_conv1x1(ctx, stream, dev, a.iters, a.only)
    if a.section in (None, "int4_gemv"):
        bench_int4_gemv(ctx, stream, dev, a.iters, a.only, a.copies)
    if a.section in (None, "int4_gemm"):
        bench_int4_gemm(ctx, stream, dev, a.iters, a.only)
    if a.section in (None, "attention"):
        bench_attention(ctx, stream, dev, a.iters, a.only)
    if a.section in (None, "lm_head"):
        bench_lm_head(ctx, stream, dev, a.iters, a.only)
    assert ctx.device_status() == 0


if __name__ == "__main__":
    main()
