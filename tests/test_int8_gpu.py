"""Parity of the tcgen05 int8 GEMM and its MatMulInteger / QLinearMatMul epilogues
against the CPU oracle, through the C ABI. Integer results are compared bit for bit."""
import numpy as np
import pytest

import yscv_b200
from yscv_b200 import synth

pytestmark = pytest.mark.gpu


# crates/yscv-kernels/src/ops/int8_matmul.rs:2458-2465
def test_known_small_case(ctx):
    out = ctx.int8_matmul(np.array([1, 2, 3, 4], np.int8), np.array([5, 6, 7, 8], np.int8), 2, 2, 2)
    assert out.ravel().tolist() == [19, 22, 43, 50]


# int8_matmul.rs:2502-2509
def test_extreme_values(ctx):
    a = np.full(128, -128, np.int8)
    assert ctx.int8_matmul(a, a, 1, 128, 1)[0, 0] == 128 * 128 * 128


# int8_matmul.rs:2467-2500: the reference's own shape lists, same LCG seeds, bit-exact
@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (2, 3, 4), (4, 16, 8), (5, 17, 6), (8, 64, 8)])
def test_dispatch_matches_scalar(ctx, oracle, m, k, n):
    a = oracle.lcg_i8(0xDEAD ^ (m * k), m * k)
    b = oracle.lcg_i8(0xBEEF ^ (k * n), k * n)
    assert np.array_equal(ctx.int8_matmul(a, b, m, k, n), oracle.int8_matmul(a, b, m, k, n))


@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (1, 17, 5), (3, 31, 7), (4, 64, 16), (8, 127, 33), (16, 128, 64)])
def test_prepacked_matches_scalar(ctx, oracle, m, k, n):
    a = oracle.lcg_i8(0xA11CE ^ (m * k), m * k)
    b = oracle.lcg_i8(0xB0B ^ (k * n), k * n)
    packed = ctx.pack_i8_b(b, k, n)
    assert (packed.k, packed.n) == (k, n)
    assert np.array_equal(ctx.int8_matmul_prepacked(a, packed, m), oracle.int8_matmul(a, b, m, k, n))
    packed.free()


# ragged tiles: every tail of the 128 x {64,128,256} x 128 tiling, multi-tile persistence
@pytest.mark.parametrize("m,k,n", [(129, 144, 65), (1, 4096, 257), (300, 272, 513), (127, 1000, 130),
                                   (257, 128, 1024), (640, 2048, 768), (2048, 512, 4096)])
def test_ragged_shapes(ctx, oracle, m, k, n):
    a = synth.uniform_int(5, 0, m * k, -128, 127).astype(np.int8)
    b = synth.uniform_int(5, 1, k * n, -128, 127).astype(np.int8)
    packed = ctx.pack_i8_b(b, k, n)
    got = ctx.int8_matmul_prepacked(a, packed, m)
    want = oracle.int8_matmul_prepacked(a, oracle.transpose_b_i8(b, k, n), m, k, n, simd=True, threads=8)
    assert np.array_equal(got, want), ctx.last_kernel()
    assert ctx.device_status() == 0
    packed.free()


# BASELINE config 1: MatMulInteger, A u8 [64,1024] with a_zero_point 128, B i8 [1024,1024], seed 0
def test_config1_matmul_integer(ctx, oracle):
    m, k, n = 64, 1024, 1024
    a = synth.uniform_int(0, 0, m * k, 0, 255).astype(np.uint8)
    b = synth.uniform_int(0, 1, k * n, -127, 127).astype(np.int8)
    packed = ctx.pack_i8_b(b, k, n)
    got = ctx.matmul_integer(a, packed, m, a_zp=128)
    # u8 with zero point 128 == i8 with zero point 0 after flipping the top bit
    want = oracle.int8_matmul((a ^ 0x80).view(np.int8), b, m, k, n)
    assert np.array_equal(got, want)
    # and the runner-level semantics (f32-encoded operands, exact integer result)
    runner = oracle.runner_matmul_integer(a.astype(np.float32), b.astype(np.float32), m, k, n, a_zp=128.0)
    assert np.array_equal(got.astype(np.float32), runner)
    # signed operand, zero point 0: the reference's int8 fast path
    a8 = (a ^ 0x80).view(np.int8)
    assert np.array_equal(ctx.matmul_integer(a8, packed, m), want)
    packed.free()


# crates/yscv-onnx/src/tests/coverage.rs:359-390 (zero-point offset known answer)
def test_matmul_integer_zero_point_known_answer(ctx):
    packed = ctx.pack_i8_b(np.array([1, 0, 0, 1], np.int8), 2, 2)
    got = ctx.matmul_integer(np.array([10, 11, 12, 13], np.uint8), packed, 2, a_zp=10)
    assert got.ravel().tolist() == [0, 1, 2, 3]
    packed.free()


# crates/yscv-kernels/src/ops/int8_requant.rs:1195-1227: round-half-even table and saturation
def test_requant_known_answers(ctx):
    one = ctx.pack_i8_b(np.array([1], np.int8), 1, 1)
    acc = np.array([1, -1, 3, -3, 5, -5, 7, -7], np.int8)
    got = ctx.qlinear_matmul(acc, one, 8, ctx.requant(0.5, 0.0, -128, 127))
    assert got.ravel().tolist() == [0, 0, 2, -2, 2, -2, 4, -4]
    away = ctx.qlinear_matmul(acc, one, 8, ctx.requant(0.5, 0.0, -128, 127, round_mode=1))
    assert away.ravel().tolist() == [1, -1, 2, -2, 3, -3, 4, -4]
    big = ctx.pack_i8_b(np.full(128, 127, np.int8), 128, 1)
    a = np.concatenate([np.full(128, 127, np.int8), np.full(128, -128, np.int8)])
    sat = ctx.qlinear_matmul(a, big, 2, ctx.requant(0.001, 0.0, -128, 127))
    assert sat.ravel().tolist() == [127, -128]
    usat = ctx.qlinear_matmul(a, big, 2, ctx.requant(0.001, 128.0, 0, 255))
    assert usat.ravel().tolist() == [255, 0]
    one.free()
    big.free()


# crates/yscv-onnx/src/tests/qlinear.rs:150-194: the runner's QLinearMatMul (f32::round, i8 clamp)
def test_runner_qlinear_matmul_case(ctx, oracle):
    a_int = (np.arange(32) - 16).astype(np.int8)
    b_int = ((np.arange(32) * 7) % 31 - 15).astype(np.int8)
    composite = np.float32(np.float32(0.05) * np.float32(0.1)) / np.float32(0.25)
    packed = ctx.pack_i8_b(b_int, 8, 4)
    got = ctx.qlinear_matmul(a_int, packed, 4, ctx.requant(composite, 0.0, -128, 127, round_mode=1))
    want = oracle.runner_qlinear_matmul_fast(a_int.astype(np.float32), b_int.astype(np.float32), 4, 8, 4,
                                             0.05, 0.1, 0.25, 0.0)
    assert np.array_equal(got.astype(np.float32), want)
    packed.free()


def config3_inputs(oracle, m, k, n):
    af = synth.normal(2, 0, m * k, 1.0)
    bf = synth.normal(2, 1, k * n, 0.02)
    a = oracle.quantize_linear(af, np.float32(6.0 / 255.0), 128.0, unsigned=True)
    b_scale = np.float32(np.max(np.abs(bf)) / np.float32(127.0))
    b = oracle.quantize_tensor_symmetric(bf, b_scale)
    composite = np.float32(np.float32(np.float32(6.0 / 255.0) * b_scale) / np.float32(0.05))
    return a, b, composite


# BASELINE config 3 (QLinearMatMul, uint8 in / uint8 out, y_zero_point 128), reduced and full size
@pytest.mark.parametrize("m,k,n", [(256, 1024, 512), (2048, 4096, 4096)])
def test_config3_qlinear_matmul(ctx, oracle, m, k, n):
    a, b, composite = config3_inputs(oracle, m, k, n)
    packed = ctx.pack_i8_b(b, k, n)
    got = ctx.qlinear_matmul(a, packed, m, ctx.requant(composite, 128.0, 0, 255, a_unsigned=True, a_zp=128))
    acc = oracle.int8_matmul_prepacked((a ^ 0x80).view(np.int8), oracle.transpose_b_i8(b, k, n), m, k, n,
                                       simd=True, threads=8)
    if m * k * n <= 2 ** 28:  # the scalar oracle proper where it finishes in seconds
        assert np.array_equal(acc, oracle.int8_matmul((a ^ 0x80).view(np.int8), b, m, k, n))
    want = oracle.requant_range(acc, composite, 128.0, 0, 255).astype(np.uint8)
    assert got.dtype == np.uint8 and np.array_equal(got, want)
    assert 0 < np.count_nonzero(got == 128) < got.size  # the output is not saturated garbage
    # raw accumulators through the MatMulInteger epilogue, and a checksum of checksums
    raw = ctx.matmul_integer(a, packed, m, a_zp=128)
    assert np.array_equal(raw, acc)
    lhs = raw.astype(np.int64).sum(axis=1)
    rhs = (a.astype(np.int64) - 128).reshape(m, k) @ b.astype(np.int64).reshape(k, n).sum(axis=1)
    assert np.array_equal(lhs, rhs)
    assert ctx.device_status() == 0
    packed.free()


def test_device_form_and_determinism(ctx, oracle):
    import torch
    m, k, n = 512, 1024, 1024
    a, b, composite = config3_inputs(oracle, m, k, n)
    d_b = torch.from_numpy(b.reshape(k, n)).cuda()
    packed = ctx.pack_i8_b_dev(d_b.data_ptr(), k, n)
    d_a = torch.from_numpy(a.reshape(m, k)).cuda()
    d_out = torch.empty(m, n, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    rq = ctx.requant(composite, 128.0, 0, 255, a_unsigned=True, a_zp=128)
    ctx.qlinear_matmul_dev(d_a.data_ptr(), packed, m, rq, d_out.data_ptr())
    ctx.synchronize()
    first = d_out.cpu().numpy()
    host = ctx.qlinear_matmul(a, packed, m, rq)
    assert np.array_equal(first, host)
    d_acc = torch.empty(m, n, dtype=torch.int32, device="cuda")
    ctx.matmul_integer_dev(d_a.data_ptr(), True, 128, packed, m, d_acc.data_ptr())
    ctx.synchronize()
    want = (a.astype(np.int32).reshape(m, k) - 128) @ b.astype(np.int32).reshape(k, n)
    assert np.array_equal(d_acc.cpu().numpy(), want)
    packed.free()


def test_bad_arguments(ctx):
    with pytest.raises(yscv_b200.YscvCudaError):
        ctx.pack_i8_b(np.zeros(0, np.int8), 0, 4)
    packed = ctx.pack_i8_b(np.zeros(16, np.int8), 4, 4)
    with pytest.raises(yscv_b200.YscvCudaError) as e:
        ctx.qlinear_matmul(np.zeros(4, np.int8), packed, 1, ctx.requant(1.0, 0.0, -200, 127))
    assert e.value.status == -1
    assert ctx.int8_matmul_prepacked(np.zeros(0, np.int8), packed, 0).shape == (0, 4)
    packed.free()


# ---- the i8 requant epilogues of the pointwise QLinearConv path ---------------------------
# crates/yscv-onnx/src/runner/conv/quantized.rs:340-500 = int8 GEMM over NHWC pixels, then
# requant_i8_per_channel (int8_requant.rs:537-556) or requant_i32_row_to_i8 (:81-169)

def conv_case(m, k, n, seed):
    a = synth.uniform_int(seed, 0, m * k, -128, 127).astype(np.int8)      # activations, NHWC pixels
    b = synth.uniform_int(seed, 1, k * n, -127, 127).astype(np.int8)      # weights [c_in][c_out]
    x_zp = int(synth.uniform_int(seed, 2, 1, -20, 20)[0])
    bias = synth.uniform_int(seed, 3, n, -5000, 5000).astype(np.int32)
    colsum = b.reshape(k, n).astype(np.int64).sum(axis=0)
    corr = (bias.astype(np.int64) - x_zp * colsum).astype(np.int32)       # what the reference folds together
    w_scale = (0.002 + 0.001 * (np.arange(n) % 7)).astype(np.float32)
    composite = (np.float32(0.05) * w_scale / np.float32(0.11)).astype(np.float32)
    return a, b, corr, composite, bias


@pytest.mark.parametrize("m,k,n", [(1, 4, 1), (49, 32, 24), (196, 96, 33), (784, 128, 256), (3136, 64, 130),
                                   (1000, 257, 512)])
def test_pointwise_conv_per_channel_requant(ctx, oracle, m, k, n):
    a, b, corr, composite, _ = conv_case(m, k, n, 40 + m)
    packed = ctx.pack_i8_b(b, k, n)
    got = ctx.int8_matmul_requant_per_channel(a, packed, m, corr, composite, -3.0)
    acc = oracle.int8_matmul(a, b, m, k, n)
    want = oracle.requant_i8_per_channel(acc.ravel(), corr, composite, -3.0, n).reshape(m, n)
    assert np.array_equal(got, want), ctx.last_kernel()
    assert ctx.device_status() == 0
    packed.free()


def test_per_channel_requant_wraps_like_the_reference(ctx, oracle):
    # acc + corr overflows i32: the reference's wrapping_add turns it negative, saturating low
    m, k, n = 4, 64, 40
    a = np.full(m * k, 127, np.int8)
    b = np.full(k * n, 127, np.int8)
    corr = np.full(n, 2**31 - 1, np.int32)
    corr[::2] = -7
    composite = np.full(n, 1e-4, np.float32)
    packed = ctx.pack_i8_b(b, k, n)
    got = ctx.int8_matmul_requant_per_channel(a, packed, m, corr, composite, 0.0)
    acc = oracle.int8_matmul(a, b, m, k, n)
    want = oracle.requant_i8_per_channel(acc.ravel(), corr, composite, 0.0, n).reshape(m, n)
    assert np.array_equal(got, want)
    assert got[0, 1] == -128 and got[0, 0] > 0
    packed.free()


@pytest.mark.parametrize("relu,with_bias", [(False, False), (False, True), (True, True), (True, False)])
def test_pointwise_conv_per_tensor_requant(ctx, oracle, relu, with_bias):
    m, k, n = 300, 96, 72
    a, b, _, _, bias = conv_case(m, k, n, 77)
    packed = ctx.pack_i8_b(b, k, n)
    got = ctx.int8_matmul_requant_i8(a, packed, m, bias if with_bias else None, 3.1e-4, 2.0, relu=relu)
    acc = oracle.int8_matmul(a, b, m, k, n)
    want = oracle.requant_i8(acc.ravel(), bias if with_bias else None, 3.1e-4, 2.0, relu, n).reshape(m, n)
    assert np.array_equal(got, want)
    if relu:
        assert got.min() >= 0
    packed.free()


def test_per_channel_requant_device_pointers(ctx, oracle):
    import torch
    m, k, n = 512, 256, 384
    a, b, corr, composite, _ = conv_case(m, k, n, 5)
    packed = ctx.pack_i8_b(b, k, n)
    torch.cuda.synchronize()
    da, dc, dp = (torch.from_numpy(x).cuda() for x in (a, corr, composite))
    out = torch.empty(m, n, dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    ctx.int8_matmul_requant_per_channel_dev(da.data_ptr(), packed, m, dc.data_ptr(), dp.data_ptr(), 1.0,
                                            out.data_ptr())
    ctx.synchronize()
    acc = oracle.int8_matmul(a, b, m, k, n)
    want = oracle.requant_i8_per_channel(acc.ravel(), corr, composite, 1.0, n).reshape(m, n)
    assert np.array_equal(out.cpu().numpy(), want)
    packed.free()


# ---- a zero point on B: exact, where the reference would leave its integer path -------------
# (crates/yscv-onnx/src/runner/linear.rs:701-735 computes (a - a_zp)(b - b_zp) in fp32 then)

@pytest.mark.parametrize("m,k,n,a_unsigned,a_zp,b_zp", [(3, 8, 3, False, 0, 5), (64, 1024, 1024, True, 128, -3),
                                                        (130, 200, 72, True, 7, 11), (257, 333, 65, False, -9, -128),
                                                        (512, 2048, 512, True, 255, 127)])
def test_matmul_integer_with_b_zero_point(ctx, oracle, m, k, n, a_unsigned, a_zp, b_zp):
    if a_unsigned:
        a = synth.uniform_int(9, 0, m * k, 0, 255).astype(np.uint8)
    else:
        a = synth.uniform_int(9, 0, m * k, -128, 127).astype(np.int8)
    b = synth.uniform_int(9, 1, k * n, -128, 127).astype(np.int8)
    packed = ctx.pack_i8_b(b, k, n)
    packed.set_zero_point(b_zp)
    want = ((a.astype(np.int64).reshape(m, k) - a_zp) @ (b.astype(np.int64).reshape(k, n) - b_zp))
    assert np.abs(want).max() < 2**31
    got = ctx.matmul_integer(a, packed, m, a_zp=a_zp)
    assert np.array_equal(got.astype(np.int64), want), ctx.last_kernel()
    # the float-typed MatMulInteger of the runner agrees wherever fp32 is exact
    if np.abs(want).max() < 2**24 and m * k * n < 2**22:
        ref = oracle.runner_matmul_integer(a.astype(np.float32), b.astype(np.float32), m, k, n, float(a_zp), float(b_zp))
        assert np.array_equal(ref.astype(np.int64), want)
    # QLinearMatMul on top of it: exact accumulator, then the requant contract
    comp = float(np.float32(0.4) / np.float32(max(1.0, np.abs(want).max() / 100.0)))
    rq = ctx.requant(comp, 128.0, 0, 255, a_unsigned=a_unsigned, a_zp=a_zp)
    got_q = ctx.qlinear_matmul(a, packed, m, rq)
    want_q = oracle.requant_range(want.astype(np.int32), comp, 128.0, 0, 255).astype(np.uint8)
    assert np.array_equal(got_q, want_q)
    packed.set_zero_point(0)
    assert np.array_equal(ctx.matmul_integer(a, packed, m, a_zp=a_zp).astype(np.int64),
                          (a.astype(np.int64).reshape(m, k) - a_zp) @ b.astype(np.int64).reshape(k, n))
    assert ctx.device_status() == 0
    packed.free()


@pytest.mark.parametrize("m,k,n", [(2048, 1024, 2560), (2000, 300, 2304), (4096, 256, 4096),
                                   (2048, 512, 4136), (1100, 384, 4000), (2048, 640, 4096)])
def test_cta_pair_kernel_is_bit_identical(ctx, oracle, m, k, n):
    """The cta_group::2 kernel (two CTAs per tile of 256 rows x 64..256 columns) against the one-CTA
    kernel and, on a row sample, the oracle: int32 and requantised outputs, ragged M, K not a
    multiple of the stage, N not a multiple of a 64-column unit, tiles of every width, more tiles
    than CTA pairs."""
    import torch
    rng = np.random.default_rng(17)
    a = rng.integers(0, 256, size=(m, k), dtype=np.uint8)
    b = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    pk = ctx.pack_i8_b(b, k, n)
    rq = ctx.requant(3e-4, 128.0, 0, 255, a_unsigned=True, a_zp=128)
    outs = {}
    try:
        for pairs in (False, True):
            ctx.set_int8_cta_pairs(pairs)
            q = ctx.qlinear_matmul(a, pk, m, rq)
            assert ("cta_group::2" in ctx.last_kernel()) == pairs
            outs[pairs] = (q, ctx.matmul_integer(a, pk, m, a_zp=128))
    finally:
        ctx.set_int8_cta_pairs(None)
    assert np.array_equal(outs[False][0], outs[True][0]) and np.array_equal(outs[False][1], outs[True][1])
    rows = rng.choice(m, size=16, replace=False)
    acc = oracle.int8_matmul((a[rows] ^ 0x80).view(np.int8), b, len(rows), k, n)
    assert np.array_equal(outs[True][1][rows], acc)
    assert np.array_equal(outs[True][0][rows], oracle.requant_range(acc, 3e-4, 128.0, 0, 255).astype(np.uint8))
    pk.free()
    assert ctx.device_status() == 0


def test_cta_pair_kernel_is_chosen_where_it_measured_faster(ctx):
    """The default kernel selection (yscv_cuda_ctx_set_int8_cta_pairs(-1)): CTA pairs for a single round of
    the one-CTA kernel on more than half of the SMs and for int32 output from three rounds of pair tiles
    on, the one-CTA kernel for requantised output with full rounds, for K < 2048 and for row counts that
    would leave the 256-row blocks more rounds than the 128-row tiles."""
    import torch
    ctx.set_int8_cta_pairs(None)
    rng = np.random.default_rng(5)
    cases = [((1024, 2048, 4096), True, True),     # 128 tiles of 128 x 256: one partial round
             ((2048, 2048, 4096), False, False),   # config-3-like: 1.73 rounds
             ((4096, 2048, 4096), True, False),    # 256 pair tiles >= 3 x 74: int32 output only
             ((1024, 1024, 4096), False, False),   # K < 2048
             ((300, 2048, 11008), False, False)]   # two 256-row blocks for 300 rows
    for (m, k, n), pair_i32, pair_u8 in cases:
        a = rng.integers(0, 256, size=(m, k), dtype=np.uint8)
        b = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
        pk = ctx.pack_i8_b(b, k, n)
        ctx.matmul_integer(a, pk, m, a_zp=128)
        assert ("cta_group::2" in ctx.last_kernel()) == pair_i32, ((m, k, n), ctx.last_kernel())
        ctx.qlinear_matmul(a, pk, m, ctx.requant(3e-4, 128.0, 0, 255, a_unsigned=True, a_zp=128))
        assert ("cta_group::2" in ctx.last_kernel()) == pair_u8, ((m, k, n), ctx.last_kernel())
        pk.free()
    assert ctx.device_status() == 0


@pytest.mark.parametrize("m,k,n,splits", [(64, 11008, 4096, True), (300, 8200, 700, True),
                                          (130, 16384, 1100, True), (2048, 4096, 4096, False)])
def test_tail_split_is_bit_identical(ctx, oracle, m, k, n, splits):
    """Shapes with far fewer tiles than SMs and K >= 8192 have their K loops cut over all CTAs and
    their int32 partial sums added by the owning CTA: aligned, ragged M / N / K, more than two
    parts per tile; config 3 keeps whole tiles. Outputs equal those of whole tiles per CTA and, on
    a row sample, the oracle; repeated calls reuse the workspace under a new epoch."""
    rng = np.random.default_rng(23)
    a = rng.integers(0, 256, size=(m, k), dtype=np.uint8)
    b = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
    pk = ctx.pack_i8_b(b, k, n)
    rq = ctx.requant(2e-4, 128.0, 0, 255, a_unsigned=True, a_zp=128)
    outs = {}
    try:
        for split in (False, True, True):
            ctx.set_int8_tail_split(split)
            q = ctx.qlinear_matmul(a, pk, m, rq)
            report = ctx.dispatch_report()
            if not split:
                assert "tail split" not in report
            else:
                assert ("tail split" in report) == splits, report
            outs[split] = (q, ctx.matmul_integer(a, pk, m, a_zp=128))
            if split:
                assert np.array_equal(outs[False][0], q) and np.array_equal(outs[False][1], outs[True][1])
    finally:
        ctx.set_int8_tail_split(True)
    rows = rng.choice(m, size=8, replace=False)
    acc = oracle.int8_matmul((a[rows] ^ 0x80).view(np.int8), b, len(rows), k, n)
    assert np.array_equal(outs[True][1][rows], acc)
    assert np.array_equal(outs[True][0][rows], oracle.requant_range(acc, 2e-4, 128.0, 0, 255).astype(np.uint8))
    pk.free()
    assert ctx.device_status() == 0
