"""Load-time and bookkeeping entry points on the GPU: the MatMul / Gemm weight path of the
int4 packer with the reference's skip rules, the name-keyed table of resident weights, the
container, the stand-alone requant pass, the counters and the dispatch report. Needs a B200."""
import numpy as np
import pytest

import yscv_b200
from yscv_b200 import synth
from yscv_b200.lib import WEIGHT_GEMM_KN, WEIGHT_GEMM_NK, WEIGHT_MATMUL_KN

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layout", [WEIGHT_MATMUL_KN, WEIGHT_GEMM_NK, WEIGHT_GEMM_KN])
@pytest.mark.parametrize("k,n,g", [(64, 8, 32), (128, 33, 16), (96, 70, 6)])
def test_weight_from_f32_matches_the_reference_packer(ctx, oracle, layout, k, n, g):
    """packed_int4.rs:74-104: MatMul [K,N] and Gemm transB=0 are transposed to [N,K] first,
    Gemm transB=1 is packed as it is; bytes and scales equal the CPU packer's bit for bit."""
    w_nk = synth.normal(41, layout, n * k, 0.02).reshape(n, k)
    given = w_nk if layout == WEIGHT_GEMM_NK else np.ascontiguousarray(w_nk.T)   # [K,N] on disk
    h = ctx.int4_weight_from_f32(given, layout, g)
    assert h is not None and (h.m_w, h.k, h.group_size) == (n, k, g)
    packed, scales = ctx.int4_weight_download(h)
    if layout != WEIGHT_GEMM_NK:   # the oracle's own transpose (packed_int4.rs:76-84)
        t = np.empty(n * k, np.float32)
        oracle.lib.yo_transpose_kn_to_nk(given.ctypes.data, k, n, t.ctypes.data)
        assert np.array_equal(t.reshape(n, k), w_nk)
    want_p, want_s = oracle.pack_int4(w_nk.ravel(), n, k, g)
    assert np.array_equal(packed, want_p) and np.array_equal(scales, want_s)
    # and the handle computes: y = x W^T
    act = synth.normal(42, 0, 3 * k, 1.0)
    got = ctx.int4_matmul(h, act, 3)
    want = oracle.exec_matmul_int4(want_p, want_s, act, 3, n, k, g)
    assert np.max(np.abs(got - want)) / np.max(np.abs(want)) <= 1e-4
    h.free()


def test_weight_from_f32_skip_rules(ctx):
    # packed_int4.rs:102-104: k % group != 0 or k * m_w < 32 -> silently skipped
    assert ctx.int4_weight_from_f32(np.ones((48, 8), np.float32), WEIGHT_MATMUL_KN, 32) is None   # k = 48
    assert ctx.int4_weight_from_f32(np.ones((4, 4), np.float32), WEIGHT_MATMUL_KN, 4) is None     # 16 weights
    assert ctx.int4_weight_from_f32(np.ones((4, 8), np.float32), WEIGHT_GEMM_NK, 8) is not None   # exactly 32
    # packed_int4.rs:54-58: an odd or zero group size is an error
    for g in (0, 7):
        with pytest.raises(yscv_b200.YscvCudaError) as e:
            ctx.int4_weight_from_f32(np.ones((64, 8), np.float32), WEIGHT_MATMUL_KN, g)
        assert e.value.status == -1


def test_registry_routes_by_initializer_name(ctx, oracle):
    """What exec_matmul does with env.packed_int4_weights.get(&node.inputs[1]) (linear.rs:228)
    and exec_qlinear_matmul with env.prepacked_i8_b(name) (tensor_env.rs:178-183)."""
    reg = yscv_b200.Registry()
    k, n, g = 256, 48, 32
    w = synth.normal(43, 0, k * n, 0.02).reshape(k, n)      # MatMul weight [K,N]
    assert reg.register_matmul_weight(ctx, "blk.0.attn_q.weight", w, WEIGHT_MATMUL_KN, g)
    assert not reg.register_matmul_weight(ctx, "blk.0.odd.weight", np.ones((40, 8), np.float32), WEIGHT_MATMUL_KN, g)
    b = synth.uniform_int(44, 0, 64 * 32, -127, 127).astype(np.int8).reshape(64, 32)
    assert reg.register_i8_weight(ctx, "blk.0.q8.weight", b)                 # k >= 4, n % 16 == 0
    assert not reg.register_i8_weight(ctx, "blk.0.q8_odd.weight", b[:, :17].copy())   # gate says no
    assert len(reg) == 2
    assert reg.get_int4("blk.0.odd.weight") is None and reg.get_i8b("blk.0.q8_odd.weight") is None
    h = reg.get_int4("blk.0.attn_q.weight")
    assert (h.m_w, h.k, h.group_size) == (n, k, g)
    act = synth.normal(45, 0, 2 * k, 1.0)
    want_p, want_s = oracle.pack_int4(np.ascontiguousarray(w.T).ravel(), n, k, g)
    want = oracle.exec_matmul_int4(want_p, want_s, act, 2, n, k, g)
    assert np.max(np.abs(ctx.int4_matmul(h, act, 2) - want)) / np.max(np.abs(want)) <= 1e-4
    pb = reg.get_i8b("blk.0.q8.weight")
    assert (pb.k, pb.n) == (64, 32)
    a = synth.uniform_int(46, 0, 5 * 64, -128, 127).astype(np.int8)
    assert np.array_equal(ctx.int8_matmul_prepacked(a, pb, 5), oracle.int8_matmul(a, b, 5, 64, 32))
    # a second put under the same name replaces the first (HashMap::insert)
    assert reg.register_matmul_weight(ctx, "blk.0.attn_q.weight", 2.0 * w, WEIGHT_MATMUL_KN, g)
    assert len(reg) == 2
    h2 = reg.get_int4("blk.0.attn_q.weight")
    assert np.max(np.abs(ctx.int4_matmul(h2, act, 2) - 2.0 * want)) / np.max(np.abs(want)) <= 3e-4
    reg.close()


def test_container_to_device_and_back(ctx, oracle):
    n, k, g = 40, 512, 32
    packed, scales = oracle.pack_int4(synth.normal(47, 0, n * k, 0.02), n, k, g)
    blob = yscv_b200.int4_container_write(packed, scales, n, k, g)
    h = ctx.int4_weight_from_container(blob)
    assert (h.m_w, h.k, h.group_size) == (n, k, g)
    p2, s2 = ctx.int4_weight_download(h)
    assert np.array_equal(p2, packed) and np.array_equal(s2, scales)
    act = synth.normal(48, 0, k, 1.0)
    want = oracle.exec_matmul_int4(packed, scales, act, 1, n, k, g)
    assert np.max(np.abs(ctx.int4_matmul(h, act, 1) - want)) / np.max(np.abs(want)) <= 1e-4
    h.free()
    with pytest.raises(yscv_b200.YscvCudaError):
        ctx.int4_weight_from_container(blob[:100])


def test_standalone_requant_matches_the_reference(ctx, oracle):
    # the reference's known answers (int8_requant.rs:1195-1227)
    acc = np.array([1, -1, 3, -3, 5, -5, 7, -7], np.int32)
    assert ctx.requant_i32_row_to_i8(acc, None, 0.5, 0.0, False, 8).tolist() == [0, 0, 2, -2, 2, -2, 4, -4]
    big = np.array([10 ** 6, -10 ** 6, 0, 1], np.int32)
    assert ctx.requant_i32_row_to_i8(big, None, 1.0, 0.0, False, 4).tolist() == [127, -128, 0, 1]
    # random rows, lane-tail channel counts, bias (wrapping) and ReLU, bit for bit
    rng = np.random.default_rng(9)
    for c in (1, 5, 17, 64):
        for relu in (False, True):
            for with_bias in (False, True):
                acc = rng.integers(-40000, 40000, size=(23, c), dtype=np.int32)
                bias = rng.integers(-5000, 5000, size=c, dtype=np.int32) if with_bias else None
                got = ctx.requant_i32_row_to_i8(acc, bias, 0.0071, 3.0, relu, c)
                want = oracle.requant_i8(acc.ravel(), bias, 0.0071, 3.0, relu, c)
                assert np.array_equal(got, want), (c, relu, with_bias)
    wrap = np.array([2 ** 31 - 1, -2 ** 31], np.int32)
    bias = np.array([1, -1], np.int32)
    assert np.array_equal(ctx.requant_i32_row_to_i8(wrap, bias, 1e-9, 0.0, False, 2),
                          oracle.requant_i8(wrap, bias, 1e-9, 0.0, False, 2))
    assert ctx.requant_i32_row_to_i8(np.zeros(0, np.int32), None, 1.0, 0.0, False, 4).size == 0
    with pytest.raises(yscv_b200.YscvCudaError):
        ctx.requant_i32_row_to_i8(np.zeros(7, np.int32), None, 1.0, 0.0, False, 4)   # len % c != 0


def test_counters_and_dispatch_report(ctx, oracle):
    yscv_b200.quant_stats_reset()
    n, k, g = 256, 512, 32
    packed, scales = oracle.pack_int4(synth.normal(49, 0, n * k, 0.02), n, k, g)
    h = ctx.int4_weight_upload(packed, scales, n, k, g)
    ctx.int4_matmul(h, synth.normal(50, 0, k, 1.0), 1)
    ctx.int4_matmul(h, synth.normal(50, 1, 20 * k, 1.0), 20)          # > 16 rows: tensor-core GEMM
    odd_p, odd_s = oracle.pack_int4(np.ones(8 * 48, np.float32), 8, 48, 6)
    ctx.packed_int4_gemv(odd_p, odd_s, np.ones(48, np.float32), 8, 48, 6)   # group 6: generic kernel
    b = np.ones((32, 32), np.int8)
    pk = ctx.pack_i8_b(b, 32, 32)
    ctx.matmul_integer(np.ones((4, 32), np.uint8), pk, 4, a_zp=3)
    ctx.qlinear_matmul(np.ones((4, 32), np.uint8), pk, 4, ctx.requant(0.1, 0.0, 0, 255, a_unsigned=True))
    st = yscv_b200.quant_stats()
    assert st["int4_gemv_calls"] == 1 and st["int4_gemm_calls"] == 1 and st["int4_generic_calls"] == 1
    assert st["int8_gemm_calls"] == 2 and st["matmul_integer_calls"] == 1 and st["qlinear_matmul_calls"] == 1
    assert st["cpu_fallbacks"] == 0
    rep = ctx.dispatch_report()
    assert "sm_100a" in rep and "int8_gemm_tc" in rep and "cpu fallback: none" in rep
    assert "int4_gemv_generic" in rep and "group=6" in rep    # the last int4 call, with its shape
    h.free()
    pk.free()


def test_operand_alignment_is_checked_not_faulted(ctx):
    """Device pointers that break a kernel's vector width are refused (or take a scalar path)."""
    import torch
    buf = torch.zeros(1 << 16, dtype=torch.float32, device="cuda")
    p = buf.data_ptr()
    tok = torch.zeros(4, dtype=torch.int32, device="cuda")
    for call in (lambda: ctx.f32_matmul_dev(p + 4, p, 1, 8, 64, p + 4096),           # weights off by 4 bytes
                 lambda: ctx.f32_matmul_dev(p, p + 4, 1, 8, 64, p + 4096),           # activations
                 lambda: ctx.embedding_dev(p + 8, 16, 64, tok.data_ptr(), 4, p + 8192),
                 lambda: ctx.embedding_dev(p, 16, 64, tok.data_ptr(), 4, p + 8192 + 4)):
        with pytest.raises(yscv_b200.YscvCudaError) as e:
            call()
        assert e.value.status == -3
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(yscv_b200.YscvCudaError) as e:   # long-cache decode attention reads keys 128 bits at a time
        ctx.gqa_attention_dev(p, 64, 1, 1, 1, 1, 64, p + 4, p + 8192, 256, pos.data_ptr(), True, p + 32768)
    assert e.value.status == -3
    with pytest.raises(yscv_b200.YscvCudaError) as e:   # rotary tables of 16 K entries do not fit shared memory
        ctx.rope_kv_append_dev(p, 1, 1, 1, 1, 32768, 10000.0, pos.data_ptr(), p, p, 4)
    assert e.value.status == -3
    # an int8 GEMM whose output row pitch allows vector stores but whose base does not:
    # the epilogue takes scalar stores, the result is the same
    a = torch.randint(-128, 128, (130, 64), dtype=torch.int8, device="cuda")
    b = np.random.default_rng(3).integers(-127, 128, size=(64, 32), dtype=np.int8)
    pk = ctx.pack_i8_b(b, 64, 32)
    out = torch.zeros(130 * 32 + 1, dtype=torch.int32, device="cuda")
    ref = torch.zeros(130 * 32, dtype=torch.int32, device="cuda")
    ctx.int8_matmul_prepacked_dev(a.data_ptr(), pk, 130, out.data_ptr() + 4)
    ctx.int8_matmul_prepacked_dev(a.data_ptr(), pk, 130, ref.data_ptr())
    ctx.synchronize()
    assert torch.equal(out[1:], ref)
    o8 = torch.zeros(130 * 32 + 3, dtype=torch.uint8, device="cuda")
    r8 = torch.zeros(130 * 32, dtype=torch.uint8, device="cuda")
    rq = ctx.requant(0.01, 128.0, 0, 255)
    ctx.qlinear_matmul_dev(a.data_ptr(), pk, 130, rq, o8.data_ptr() + 3)
    ctx.qlinear_matmul_dev(a.data_ptr(), pk, 130, rq, r8.data_ptr())
    ctx.synchronize()
    assert torch.equal(o8[3:], r8)
    pk.free()
    assert ctx.device_status() == 0
