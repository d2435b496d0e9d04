"""Tensor-parallel decoder across 2 GPUs against the single-GPU decoder: same logits
(relative Frobenius) and the same greedy tokens, for the operator chain (NCCL all-reduce,
batch 2) and for the one-launch decode step whose kernels exchange their partial sums
through peer memory (batch 1). Needs two B200s; skipped on a one-GPU box. Each rank is a
child process; rank 0 also runs the TP=1 decoder."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = r'''
import json, os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["YSCV_ROOT"])
import yscv_b200
from yscv_b200 import synth
from yscv_b200.decoder import DecoderConfig, Int4Decoder
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
torch.cuda.set_device(local)
cfg = DecoderConfig(layers=3, hidden=1024, mlp=2048, n_q=16, n_kv=4, head_dim=64, vocab=2000)
B, P, steps = 2, 24, 12
prompt = torch.from_numpy(np.stack([synth.uniform_int(7 + b, 9, P, 0, cfg.vocab - 1) for b in range(B)]).astype(np.int32)).cuda()
stream = torch.cuda.Stream()
ctx = yscv_b200.Context(local, stream=stream.cuda_stream)
ctx.set_int4_prefill_exact(True)   # strict comparison: the bf16 prompt pass rounds differently per K split
tp = Int4Decoder(ctx, cfg, B, P + steps + 2, stream, seed=5, tp_rank=rank, tp_size=world, process_group=dist.group.WORLD)
lg = tp.prefill(prompt); stream.synchronize()
tp.capture_decode_step()
toks = tp.decode(steps); stream.synchronize()
out = {"status": ctx.device_status()}
if rank == 0:
    one = Int4Decoder(ctx, cfg, B, P + steps + 2, stream, seed=5)
    lg1 = one.prefill(prompt); stream.synchronize()
    one.capture_decode_step()
    toks1 = one.decode(steps); stream.synchronize()
    out["rel"] = float(torch.linalg.norm(lg - lg1) / torch.linalg.norm(lg1))
    out["tokens_equal"] = bool(torch.equal(toks, toks1))
    print("RESULT " + json.dumps(out), flush=True)
    one.close()
tp.close()
dist.barrier()

# ---- batch 1: the one-launch step on both ranks, partial sums exchanged inside the kernel ----
P1, steps1 = 40, 16
prompt1 = prompt[:1, :].contiguous()
prompt1 = torch.cat([prompt1, prompt1], dim=1)[:, :P1].contiguous()
ftp = Int4Decoder(ctx, cfg, 1, P1 + steps1 + 2, stream, seed=5, tp_rank=rank, tp_size=world, process_group=dist.group.WORLD)
assert ftp.plan is not None, "the tensor-parallel decode plan was not built"
ftp.prefill(prompt1); stream.synchronize()
with torch.cuda.stream(stream):
    first = ftp.forward(ftp.next_tokens, 1).clone()     # one eager step: this rank's slice of the logits
stream.synchronize()
ftp.capture_decode_step()
ftoks = ftp.decode(steps1); stream.synchronize()
ftp.plan.check()
parts = [torch.empty_like(first) for _ in range(world)]
dist.all_gather(parts, first)
V = cfg.vocab // world
full_logits = torch.cat([parts[r][0, r * V:(r + 1) * V] for r in range(world)])
allt = [torch.empty_like(ftoks) for _ in range(world)]
dist.all_gather(allt, ftoks.contiguous())
out2 = {"status": ctx.device_status(), "ranks_agree": bool(all(torch.equal(allt[0], t) for t in allt)),
        "kernel": ctx.last_kernel()}
if rank == 0:
    one = Int4Decoder(ctx, cfg, 1, P1 + steps1 + 2, stream, seed=5)
    assert one.plan is not None
    one.prefill(prompt1); stream.synchronize()
    with torch.cuda.stream(stream):
        lg1 = one.forward(one.next_tokens, 1).clone()
    stream.synchronize()
    one.capture_decode_step()
    toks1 = one.decode(steps1); stream.synchronize()
    out2["rel"] = float(torch.linalg.norm(full_logits - lg1[0]) / torch.linalg.norm(lg1[0]))
    out2["tokens_equal"] = bool(torch.equal(ftoks, toks1))
    print("RESULT2 " + json.dumps(out2), flush=True)
    one.close()
ftp.close()
dist.barrier()
dist.destroy_process_group()
'''


def test_tp2_matches_tp1(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, YSCV_ROOT=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    import json
    line = [l for l in proc.stdout.splitlines() if l.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    assert res["status"] == 0
    assert res["rel"] < 1e-5, res       # fp32 partial sums in a different order
    assert res["tokens_equal"], res
    line = [l for l in proc.stdout.splitlines() if l.startswith("RESULT2 ")][-1]
    res = json.loads(line[len("RESULT2 "):])
    assert res["status"] == 0 and res["ranks_agree"], res
    assert "decode_step" in res["kernel"], res
    assert res["rel"] < 1e-5, res
    assert res["tokens_equal"], res


def test_int8_n_shard_matches_unsharded():
    """QLinearMatMul with the output channels split over 2 GPUs: the all-gathered bytes equal
    the single-GPU result bit for bit."""
    import json
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29613", "-m", "yscv_b200.int8_shard_bench",
           "--rows", "512", "--inner", "1024", "--cols", "1536", "--iters", "5"]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    res = json.loads([l for l in proc.stdout.splitlines() if l.startswith("{")][-1])
    assert res["bit_exact_vs_unsharded"] and res["device_status"] == 0 and res["gpus"] == 2
