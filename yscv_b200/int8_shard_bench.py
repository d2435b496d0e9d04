"""QLinearMatMul with the output channels sharded over the ranks of a torchrun job
(BASELINE config 3 by default: A u8 [2048,4096] zero point 128, B i8 [4096,4096], u8 out).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
        --master-port P -m yscv_b200.int8_shard_bench [--rows M --inner K --cols N --iters I]

Rank r packs the columns [r*n/G, (r+1)*n/G) of B once, every rank holds A; a call runs the
rank's GEMM + requant and all-gathers the byte outputs (NCCL). Parity gate: the assembled
output equals the unsharded GPU result bit for bit (rank 0 computes both). Reports the
slowest rank's time per call with and without the gather (CUDA events, max over ranks).
Also runs as a single process (G = 1).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

from . import Context, sharding


def run(m=2048, k=4096, n=4096, iters=50):
    """One measurement inside an initialised job (or a single process). Returns the summary on
    rank 0, None elsewhere; raises if the gathered output differs from the unsharded one."""
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
    stream = torch.cuda.Stream()
    ctx = Context(local, stream=stream.cuda_stream)
    with torch.cuda.stream(stream):
        g = torch.Generator(device=dev)
        g.manual_seed(2)  # the same operands on every rank
        A = torch.randint(0, 256, (m, k), dtype=torch.uint8, device=dev, generator=g)
        B = torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev, generator=g)
        mine = sharding.shard_i8_b_cols(B, rank, world).contiguous()
        pk = ctx.pack_i8_b_dev(mine.data_ptr(), k, n // world)
        rq = ctx.requant(1e-4, 128.0, 0, 255, a_unsigned=True, a_zp=128)
        part = torch.empty(m, n // world, dtype=torch.uint8, device=dev)
        gathered = torch.empty(world, m, n // world, dtype=torch.uint8, device=dev)

        def compute():
            ctx.qlinear_matmul_dev(A.data_ptr(), pk, m, rq, part.data_ptr())

        def gather():
            if world > 1:
                dist.all_gather_into_tensor(gathered, part)
            else:
                gathered[0].copy_(part)

        compute()
        gather()
        full = sharding.assemble_cols(gathered).contiguous()
    stream.synchronize()
    exact = True
    if rank == 0:
        with torch.cuda.stream(stream):
            pk_all = ctx.pack_i8_b_dev(B.data_ptr(), k, n)
            ref = torch.empty(m, n, dtype=torch.uint8, device=dev)
            ctx.qlinear_matmul_dev(A.data_ptr(), pk_all, m, rq, ref.data_ptr())
        stream.synchronize()
        exact = bool(torch.equal(ref, full))
        pk_all.free()

    def timed(fn):
        ts = []
        with torch.cuda.stream(stream):
            for _ in range(5):
                fn()
            for _ in range(iters):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                fn()
                e1.record(stream)
                ts.append((e0, e1))
        stream.synchronize()
        t = torch.tensor([statistics.median(x.elapsed_time(y) for x, y in ts)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e3

    t_compute = timed(compute)
    t_both = timed(lambda: (compute(), gather()))
    out = None
    if rank == 0:
        ops = 2.0 * m * k * n
        out = {"workload": f"QLinearMatMul {m}x{k}x{n} u8 out, N-sharded", "gpus": world,
               "bit_exact_vs_unsharded": exact, "us_compute": t_compute, "us_with_all_gather": t_both,
               "tops_compute": ops / t_compute / 1e6, "tops_with_all_gather": ops / t_both / 1e6,
               "kernel": ctx.last_kernel(), "device_status": ctx.device_status()}
    pk.free()
    ctx.close()
    assert exact
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=2048, help="M")
    ap.add_argument("--inner", type=int, default=4096, help="K")
    ap.add_argument("--cols", type=int, default=4096, help="N")
    ap.add_argument("--iters", type=int, default=50)
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", 1))
    out = run(a.rows, a.inner, a.cols, a.iters)
    if out is not None:
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
