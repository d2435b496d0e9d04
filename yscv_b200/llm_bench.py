"""Decode benchmark of the random-init int4 decoder, the counterpart of
apps/llm-bench (apps/llm-bench/src/main.rs:491-586): warm-up passes, one timed prefill,
N timed single-token greedy steps with the KV cache, one JSON summary line with the
same keys (prompt_tokens, decode_tokens, prefill_ms, decode_total_ms,
decode_tokens_per_sec).

    python -m yscv_b200.llm_bench --model tinyllama --batch 1 --prompt-len 128 --max-tokens 256
    torchrun --nproc-per-node 8 -m yscv_b200.llm_bench --model llama70b --prompt-len 2048 --max-tokens 128

Under torchrun the linears are tensor-parallel across the ranks: the prompt pass and
batches above 1 sum the row-parallel partials with an NCCL all-reduce, the batch-1 decode
step is one kernel launch per rank whose CTAs exchange the partials through peer memory.
Prompts are uniform token ids from the seeded generator.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import Context, synth
from .decoder import LLAMA3_70B, TINYLLAMA_1B, Int4Decoder

MODELS = {"tinyllama": (TINYLLAMA_1B, 3), "llama70b": (LLAMA3_70B, 4)}


def weight_bytes_per_token(cfg, layers, tp, lm_head_sharded=False):
    d = cfg.head_dim
    per_layer = (cfg.n_q + 2 * cfg.n_kv) * d * cfg.hidden + cfg.hidden * cfg.n_q * d + 3 * cfg.mlp * cfg.hidden
    int4 = per_layer * layers * (0.5 + 4.0 / cfg.group_size) / tp
    return int4 + cfg.vocab * cfg.hidden * 4 / (tp if lm_head_sharded else 1)  # + fp32 LM head


def run(model="tinyllama", batch=1, prompt_len=128, max_tokens=256, warmup=1, layers=None, use_graph=True,
        exact_prefill=False, kv_int8=False, fused_step=True, return_tokens=False, synthetic_cache=False):
    """synthetic_cache: skip the prompt pass and fill the KV cache of the first prompt_len
    positions with seeded random rows instead (decode throughput does not depend on what the
    cache holds; used where the prompt pass of a wide batch would take minutes)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    pg = None
    if world > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        pg = dist.group.WORLD
    torch.cuda.set_device(local)
    cfg, seed = MODELS[model]
    stream = torch.cuda.Stream()
    ctx = Context(local, stream=stream.cuda_stream)
    ctx.set_int4_prefill_exact(exact_prefill)
    n_layers = layers or cfg.layers
    dec = Int4Decoder(ctx, cfg, batch, prompt_len + max_tokens + 2, stream, seed=seed, tp_rank=rank, tp_size=world,
                      process_group=pg, layers=n_layers, kv_int8=kv_int8, fused_step=fused_step)
    import numpy as np
    prompt = np.stack([synth.uniform_int(seed + b, 9, prompt_len, 0, cfg.vocab - 1) for b in range(batch)])
    d_prompt = torch.from_numpy(prompt.astype(np.int32)).cuda()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    if synthetic_cache:
        with torch.cuda.stream(stream):
            gen = torch.Generator(device=dec.dev)
            gen.manual_seed(seed + 77)
            for l in range(n_layers):
                for cache, scale in ((dec.kcache[l], dec.kscale[l] if kv_int8 else None),
                                     (dec.vcache[l], dec.vscale[l] if kv_int8 else None)):
                    if kv_int8:
                        cache[:, :prompt_len].copy_(torch.randint(-127, 128, cache[:, :prompt_len].shape, device=dec.dev,
                                                                  generator=gen, dtype=torch.int8))
                        scale[:, :prompt_len].fill_(1.0 / 127.0)
                    else:
                        cache[:, :prompt_len].normal_(0.0, 1.0, generator=gen)
            dec.pos.fill_(prompt_len)
            dec.next_tokens.copy_(d_prompt[:, -1])
        stream.synchronize()
    else:
        for _ in range(warmup):  # stateless warm-up with the full prompt, cache restored afterwards
            dec.reset()
            dec.prefill(d_prompt)
        stream.synchronize()
        dec.reset()
        with torch.cuda.stream(stream):
            e0.record(stream)
            dec.prefill(d_prompt)
            e1.record(stream)
        stream.synchronize()
    if use_graph:
        dec.capture_decode_step()
    l0 = ctx.launch_count()
    with torch.cuda.stream(stream):
        e1.record(stream)
    toks = dec.decode(max_tokens, use_graph=use_graph)
    with torch.cuda.stream(stream):
        e2.record(stream)
    stream.synchronize()
    prefill_ms, decode_ms = e0.elapsed_time(e1) if False else None, e1.elapsed_time(e2)
    # the prefill was timed before e1 was re-recorded: measure it again from a fresh pair
    prefill_ms = None
    if not synthetic_cache:
        dec.reset()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            p0.record(stream)
            dec.prefill(d_prompt)
            p1.record(stream)
        stream.synchronize()
        prefill_ms = p0.elapsed_time(p1)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([prefill_ms or 0.0, decode_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        prefill_ms, decode_ms = (float(t[0]) if prefill_ms is not None else None), float(t[1])
    tps = batch * max_tokens * 1000.0 / decode_ms
    wb = weight_bytes_per_token(cfg, n_layers, world, lm_head_sharded=dec.plan is not None and world > 1)
    if dec.plan is not None:
        dec.plan.check()
    summary = {
        "model": f"{model} (random-init int4, group {cfg.group_size}, {n_layers} layers)",
        "gpus": world, "batch": batch, "prompt_tokens": prompt_len, "decode_tokens": max_tokens,
        "prefill_ms": prefill_ms, "decode_total_ms": decode_ms, "decode_tokens_per_sec": tps,
        "ms_per_step": decode_ms / max_tokens,
        "weight_bytes_per_step_per_gpu": wb,
        "weight_stream_gbs_per_gpu": wb / (decode_ms / max_tokens * 1e-3) / 1e9,
        "cuda_graph": bool(use_graph), "prefill": "fp32-exact" if exact_prefill else "bf16 tensor-core",
        "decode_step": ("one persistent kernel per token" + (" per GPU, partial sums exchanged through peer memory "
                                                              "inside it" if world > 1 else ""))
        if dec.plan is not None else ("operator chain" + (" + NCCL all-reduce" if world > 1 else "")),
        "kv_cache": ("int8 rows + f32 scale per token" if kv_int8 else "f32") +
                    (", first prompt_len positions filled with random rows instead of a prompt pass" if synthetic_cache else ""),
        "first_tokens": toks[:8, 0].cpu().tolist(),
        "device_status": ctx.device_status(),
    }
    if return_tokens:
        summary["tokens"] = toks.cpu().numpy().copy()
    dec.close()
    ctx.close()
    return summary


def tokens_match_single_gpu(model="llama70b", layers=2, prompt_len=64, steps=32):
    """The tensor-parallel decoder of this job against the same decoder on one GPU, on a
    truncation of `layers` layers with the prompt pass in the fp32-exact mode: identical greedy
    tokens for `steps` steps (rank 0 runs the one-GPU decoder; returns None on other ranks)."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    tp = run(model, 1, prompt_len, steps, warmup=0, layers=layers, exact_prefill=True, return_tokens=True)
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    saved = {k: os.environ.get(k) for k in ("RANK", "WORLD_SIZE")}
    os.environ["RANK"], os.environ["WORLD_SIZE"] = "0", "1"
    try:
        # one GPU: the one-launch step against the operator chain; several GPUs: their
        # one-launch steps against the one-launch step of a single GPU
        one = run(model, 1, prompt_len, steps, warmup=0, layers=layers, exact_prefill=True, return_tokens=True,
                  fused_step=world > 1)
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    torch.cuda.empty_cache()
    import numpy as np
    return bool(np.array_equal(tp["tokens"], one["tokens"])) and tp["device_status"] == 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tinyllama", choices=sorted(MODELS))
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--layers", type=int, default=None, help="truncate the stack (default: the model's depth)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--kv-int8", action="store_true", help="KV cache as int8 rows with one f32 scale per token")
    ap.add_argument("--synthetic-cache", action="store_true",
                    help="no prompt pass: random cache contents for the first prompt-len positions")
    ap.add_argument("--exact-prefill", action="store_true",
                    help="prompt pass on the fp32-exact int4 kernel (token-for-token comparable across TP degrees)")
    a = ap.parse_args()
    s = run(a.model, a.batch, a.prompt_len, a.max_tokens, a.warmup, a.layers, not a.no_graph, a.exact_prefill,
            kv_int8=a.kv_int8, synthetic_cache=a.synthetic_cache)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(s), flush=True)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
