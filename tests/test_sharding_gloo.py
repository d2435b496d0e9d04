"""The multi-rank path on CPU: two gloo ranks shard a packed int4 weight column- and
row-parallel, compute their part with the CPU oracle, and exchange results exactly as
the GPU ranks do over NCCL (all_gather / all_reduce)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, q):
    sys.path[:0] = [str(ROOT), str(ROOT / "oracle")]
    import torch
    import torch.distributed as dist
    import oracle_lib
    from yscv_b200 import sharding, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        o = oracle_lib.load()
        n, k, g, m = 64, 256, 32, 3
        w = synth.normal(9, 0, n * k, 0.02)
        packed, scales = o.pack_int4(w, n, k, g)
        packed, scales = packed.reshape(n, k // 2), scales.reshape(n, k // g)
        act = synth.normal(9, 1, m * k, 1.0).reshape(m, k)
        full = o.exec_matmul_int4(packed.ravel(), scales.ravel(), act, m, n, k, g)
        # column-parallel: own rows, all-gather the output columns
        p, s = sharding.shard_rows(packed, scales, rank, world)
        part = o.exec_matmul_int4(np.ascontiguousarray(p).ravel(), np.ascontiguousarray(s).ravel(), act, m,
                                  n // world, k, g)
        gathered = [torch.empty(m, n // world) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(part))
        col_ok = np.array_equal(torch.cat(gathered, dim=1).numpy(), full)
        # row-parallel: own K slice, all-reduce the fp32 partials
        p, s = sharding.shard_cols(packed, scales, g, rank, world)
        a = np.ascontiguousarray(sharding.shard_activation_cols(act, g, rank, world))
        part = o.exec_matmul_int4(np.ascontiguousarray(p).ravel(), np.ascontiguousarray(s).ravel(), a, m, n,
                                  k // world, g)
        t = torch.from_numpy(part.copy())
        dist.all_reduce(t)
        err = float(np.max(np.abs(t.numpy() - full)) / np.max(np.abs(full)))
        # int8 QLinearMatMul, N-sharded: own columns of B and of the per-channel vectors,
        # all-gather the requantised bytes
        mi, ki, ni = 5, 48, 32
        a8 = synth.uniform_int(9, 2, mi * ki, -128, 127).astype(np.int8)
        b8 = synth.uniform_int(9, 3, ki * ni, -127, 127).astype(np.int8).reshape(ki, ni)
        corr = synth.uniform_int(9, 4, ni, -500, 500).astype(np.int32)
        comp = (0.001 * (1 + np.arange(ni) % 3)).astype(np.float32)
        full_q = o.requant_i8_per_channel(o.int8_matmul(a8, b8, mi, ki, ni).ravel(), corr, comp, 1.0, ni).reshape(mi, ni)
        bs = np.ascontiguousarray(sharding.shard_i8_b_cols(b8, rank, world))
        acc = o.int8_matmul(a8, bs, mi, ki, ni // world)
        mine = o.requant_i8_per_channel(acc.ravel(), np.ascontiguousarray(sharding.shard_channel_vector(corr, rank, world)),
                                        np.ascontiguousarray(sharding.shard_channel_vector(comp, rank, world)), 1.0,
                                        ni // world).reshape(mi, ni // world)
        parts = [torch.empty(mi, ni // world, dtype=torch.int8) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(mine))
        i8_ok = np.array_equal(sharding.assemble_cols(torch.stack(parts)).numpy(), full_q)
        q.put((rank, col_ok and i8_ok, err))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_matches_single_rank():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, col_ok, err in results:
        assert col_ok, f"rank {rank}: column-parallel shards do not reassemble the full output"
        assert err <= 1e-6, f"rank {rank}: row-parallel partial sums differ by {err}"


def test_shard_ranges_reject_bad_splits():
    from yscv_b200 import sharding
    assert sharding.row_range(64, 1, 4) == (16, 32)
    assert sharding.col_range(256, 32, 3, 4) == (192, 256)
    with pytest.raises(ValueError):
        sharding.row_range(10, 0, 4)
    with pytest.raises(ValueError):
        sharding.col_range(96, 32, 0, 2)  # 48 per rank is not a multiple of the group
    # Llama-3-70B shapes over 8 ranks (BASELINE config 5)
    assert sharding.col_range(8192, 32, 7, 8) == (7168, 8192)
    assert sharding.col_range(28672, 32, 1, 8) == (3584, 7168)


def _tp_worker(rank, world, port, q):
    sys.path[:0] = [str(ROOT), str(ROOT / "oracle")]
    import torch
    import torch.distributed as dist
    import oracle_lib
    from yscv_b200 import sharding, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        o = oracle_lib.load()
        n, k, g, layers, steps, cap = 48, 512, 32, 3, 4, 64
        w = synth.normal(19, 0, n * k, 0.02)
        packed, scales = o.pack_int4(w, n, k, g)
        packed, scales = packed.reshape(n, k // 2), scales.reshape(n, k // g)
        p, s = sharding.shard_cols(packed, scales, g, rank, world)
        p, s = np.ascontiguousarray(p).ravel(), np.ascontiguousarray(s).ravel()
        # the rank's exchange region: [2 parities][world sources][cap rows] of (value, tag)
        values = np.zeros(2 * world * cap, np.float32)
        tags = np.zeros(2 * world * cap, np.uint32)
        ok, sums = True, []
        for step in range(steps):
            for ex in range(2 * layers):
                act = synth.normal(19, 1 + step * 100 + ex, k, 1.0).reshape(1, k)
                a = np.ascontiguousarray(sharding.shard_activation_cols(act, g, rank, world))
                part = o.exec_matmul_int4(p, s, a, 1, n, k // world, g).ravel()
                tag, par = sharding.exchange_tag(step, layers, ex), sharding.exchange_parity(step, layers, ex)
                # "store into every peer's region": the all_gather stands in for the peer stores
                got = [torch.empty(n) for _ in range(world)]
                dist.all_gather(got, torch.from_numpy(part.copy()))
                for src in range(world):
                    sl = sharding.exchange_slot(par, src, 0, world, cap)
                    # the slot set being overwritten was last used two exchanges ago: its tag is old
                    ok &= bool(np.all(tags[sl:sl + n] != tag))
                    values[sl:sl + n] = got[src].numpy()
                    tags[sl:sl + n] = tag
                # "poll until the tags match", then the sum in rank order
                parts = []
                for src in range(world):
                    sl = sharding.exchange_slot(par, src, 0, world, cap)
                    ok &= bool(np.all(tags[sl:sl + n] == tag))
                    parts.append(values[sl:sl + n].copy())
                total = sharding.sum_in_rank_order(parts)
                full = o.exec_matmul_int4(packed.ravel(), scales.ravel(), act, 1, n, k, g).ravel()
                ok &= float(np.max(np.abs(total - full)) / np.max(np.abs(full))) < 1e-5
                sums.append(total)
        # every rank holds the same bits
        mine = torch.from_numpy(np.concatenate(sums))
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        ok &= all(torch.equal(allr[0], t) for t in allr)
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_two_rank_exchange_protocol_of_the_decode_step():
    """The tensor-parallel exchange of the decode step, restated on the host and run by two
    gloo ranks: K-sliced partial GEMVs, slot / tag / parity arithmetic, sums in rank order."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29731
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok in res), res


def test_exchange_tags_and_parities():
    from yscv_b200 import sharding
    for layers in (1, 2, 22, 80):
        seen = {}
        for step in range(6):
            for ex in range(sharding.exchanges_per_step(layers)):
                tag, par = sharding.exchange_tag(step, layers, ex), sharding.exchange_parity(step, layers, ex)
                assert tag != 0
                kind = "token" if ex == 2 * layers else "gemv"
                prev = seen.get((kind, "last"))
                if prev is not None:            # consecutive exchanges of one kind use different slot sets
                    assert prev[1] != par, (layers, step, ex)
                last_same = seen.get((kind, par))
                if last_same is not None:       # and a slot set never sees the same tag twice in a row
                    assert last_same != tag
                seen[(kind, "last")] = (tag, par)
                seen[(kind, par)] = tag
    # tags wrap at 2^32 without ever becoming 0 at the wrap of one step's exchanges
    assert sharding.exchange_tag((1 << 32) // 161, 80, 0) != 0
