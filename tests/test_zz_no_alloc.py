"""The allocation-free int4 matmul entry point (scratch in an array built into the
library) against the regular device entry point. Collected last on purpose."""
import numpy as np
import pytest

import yscv_b200
from yscv_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(16, 4096, 4096), (1, 1024, 2048), (5, 777, 8192)])
def test_static_scratch_matches_regular_entry_point(ctx, oracle, m, n, k):
    """Two calls in a row through the C ABI: the shared scratch array carries the
    previous call's contents into the next one, and the result must not care."""
    import torch
    g = 32
    packed, scales = oracle.pack_int4(synth.normal(71, 0, n * k, 0.02), n, k, g)
    d_p, d_s = torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda()
    w = ctx.int4_weight_wrap(d_p.data_ptr(), d_s.data_ptr(), n, k, g)
    for call in range(2):
        act = synth.normal(72 + call, 1, m * k, 1.0)
        d_a = torch.from_numpy(act).cuda()
        ref = torch.empty(m * n, dtype=torch.float32, device="cuda")
        got = torch.full((m * n,), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        ctx.int4_matmul_dev(w, d_a.data_ptr(), ref.data_ptr(), m)
        ctx.int4_matmul_dev_static(d_p.data_ptr(), d_s.data_ptr(), n, k, g, d_a.data_ptr(), got.data_ptr(), m)
        ctx.synchronize()
        assert "static-scratch" in ctx.last_kernel()
        r, o = ref.cpu().numpy(), got.cpu().numpy()
        assert np.max(np.abs(o - r)) / np.max(np.abs(r)) <= 1e-4, call
        want = oracle.exec_matmul_int4(packed, scales, act, m, n, k, g).ravel()
        assert np.max(np.abs(o - want)) / np.max(np.abs(want)) <= 1e-4, call
    assert ctx.device_status() == 0
    w.free()


def test_static_scratch_allocates_nothing(oracle):
    """A context that never reserved any scratch of its own: the free device memory reported
    by the driver is the same before and after calls through the allocation-free entry point."""
    import torch
    m, n, k, g = 8, 2048, 4096, 32
    packed, scales = oracle.pack_int4(synth.normal(75, 0, n * k, 0.02), n, k, g)
    d_p, d_s = torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda()
    d_a = torch.from_numpy(synth.normal(76, 1, m * k, 1.0)).cuda()
    out = torch.empty(m * n, dtype=torch.float32, device="cuda")
    fresh = yscv_b200.Context(0)
    # first call: looks up the built-in array's address and loads the kernels it needs
    fresh.int4_matmul_dev_static(d_p.data_ptr(), d_s.data_ptr(), n, k, g, d_a.data_ptr(), out.data_ptr(), m)
    fresh.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        fresh.int4_matmul_dev_static(d_p.data_ptr(), d_s.data_ptr(), n, k, g, d_a.data_ptr(), out.data_ptr(), m)
    fresh.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    want = oracle.exec_matmul_int4(packed, scales, synth.normal(76, 1, m * k, 1.0), m, n, k, g).ravel()
    assert np.max(np.abs(out.cpu().numpy() - want)) / np.max(np.abs(want)) <= 1e-4
    assert fresh.device_status() == 0
    fresh.close()


def test_static_scratch_rejects_what_it_cannot_hold(ctx):
    import torch
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    for n, k, g, m in [(8, 65536, 32, 1),    # k beyond the built-in array
                       (8, 256, 32, 17),     # more than 16 rows
                       (8, 256, 64, 1),      # group size the fast kernel does not take
                       (8, 96, 32, 1)]:      # k not a multiple of 256
        with pytest.raises(yscv_b200.YscvCudaError) as e:
            ctx.int4_matmul_dev_static(p, p, n, k, g, p, p, m)
        assert e.value.status == -3
