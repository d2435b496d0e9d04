"""Parity of the CUDA int4 block-quantized GEMV / small-M GEMM and of the GPU
packer against the CPU oracle, through the C ABI. Needs a B200."""
import numpy as np
import pytest

import yscv_b200
from yscv_b200 import synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-4  # max|diff| / max|ref|, the definition kernel_bench uses (kernel_bench.rs:97-103)
FRO_TOL = 2e-2  # relative Frobenius error allowed for the bf16 tensor-core prefill GEMM (m > 16)


def fro_err(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


def rel_err(got, want):
    return float(np.max(np.abs(got - want)) / max(float(np.max(np.abs(want))), 1e-30))


def make_weights(oracle, seed, n, k, g, std=0.02):
    w = synth.normal(seed, 0, n * k, std)
    return oracle.pack_int4(w, n, k, g)


# ---- the reference's own unit-test cases (int4_matmul.rs:720-944) ------------

@pytest.mark.parametrize("m_w,k,g,sw,sa", [(4, 128, 32, 0xCAFEBABE, 0xF00DBA12),
                                           (8, 256, 32, 0x12345678, 0x9ABCDEF0)])
def test_gemv_reference_cases(ctx, oracle, m_w, k, g, sw, sa):
    packed, scales = oracle.pack_int4(oracle.lcg_f32(sw, m_w * k), m_w, k, g)
    act = oracle.lcg_f32(sa, k)
    want = oracle.int4_gemv(packed, scales, act, m_w, k, g)
    got = ctx.packed_int4_gemv(packed, scales, act, m_w, k, g)
    assert np.max(np.abs(got - want)) <= 1e-4


def test_gemv_zero_weights(ctx, oracle):
    packed, scales = oracle.pack_int4(np.zeros(3 * 32, np.float32), 3, 32, 16)
    out = ctx.packed_int4_gemv(packed, scales, np.full(32, 1.5, np.float32), 3, 32, 16)
    assert np.all(np.abs(out) <= 1e-5)


def test_gemm_reference_cases(ctx, oracle):
    n, k, g = 8, 64, 32
    packed, scales = oracle.pack_int4(oracle.lcg_f32(0x100, n * k), n, k, g)
    for m in (1, 4, 16, 32):
        act = oracle.lcg_f32(0x200 + m, m * k)
        want = oracle.int4_gemm(packed, scales, act, m, n, k, g)
        got = ctx.packed_int4_gemm(packed, scales, act, m, n, k, g)
        if m > 16:  # bf16 tensor-core path, then the exact one
            assert fro_err(got, want) <= FRO_TOL, m
            ctx.set_int4_prefill_exact(True)
            got = ctx.packed_int4_gemm(packed, scales, act, m, n, k, g)
            ctx.set_int4_prefill_exact(False)
        assert np.max(np.abs(got - want)) <= 1e-3, m


# ---- odd / ragged shapes: both kernels, all tails ------------------------------

@pytest.mark.parametrize("m,n,k,g", [
    (1, 5, 96, 32),      # generic vec path (K % 256 != 0)
    (3, 7, 64, 16),      # generic bytewise (group 16)
    (2, 9, 60, 6),       # group not a power of two
    (1, 1, 256, 32),     # fast, a single row
    (1, 17, 256, 32),    # fast, fewer rows than SMs
    (5, 1000, 512, 32),  # fast, padded M
    (3, 300, 2048, 32),
    (1, 2500, 768, 32),  # fast, 256-wide stages
    (7, 2049, 1280, 32),
    (16, 777, 1024, 32),
    (12, 3000, 4096, 32),
    (1, 4096, 1024, 64),  # group 64 -> generic
    (20, 640, 512, 32),   # more than 16 rows: split into chunks of 16
])
def test_odd_shapes(ctx, oracle, m, n, k, g):
    packed, scales = make_weights(oracle, 11, n, k, g)
    act = synth.normal(12, 1, m * k, 1.0)
    want = oracle.exec_matmul_int4(packed, scales, act, m, n, k, g)
    got = ctx.packed_int4_gemm(packed, scales, act, m, n, k, g)
    assert got.shape == (m, n)
    if "prefill" in ctx.last_kernel():
        assert fro_err(got, want) <= FRO_TOL
        ctx.set_int4_prefill_exact(True)
        got = ctx.packed_int4_gemm(packed, scales, act, m, n, k, g)
        ctx.set_int4_prefill_exact(False)
    assert rel_err(got, want) <= REL_TOL, (ctx.last_kernel(), rel_err(got, want))


# ---- prefill shapes: tcgen05 bf16 GEMM, relative Frobenius error <= 2e-2 ----------

@pytest.mark.parametrize("m,n,k", [(17, 128, 64), (128, 2560, 2048), (200, 1000, 1024), (333, 130, 4096),
                                   (512, 4096, 512), (1024, 300, 256), (2048, 1024, 2048), (1100, 8000, 512),
                                   (64, 1024, 4096), (2048, 4608, 1024), (1100, 8000, 448)])
def test_prefill_gemm(ctx, oracle, m, n, k):
    g = 32
    packed, scales = make_weights(oracle, 21, n, k, g)
    act = synth.normal(22, 1, m * k, 1.0)
    want = oracle.exec_matmul_int4(packed, scales, act, m, n, k, g, threads=8)
    got = ctx.packed_int4_gemm(packed, scales, act, m, n, k, g)
    assert "prefill" in ctx.last_kernel()
    report = ctx.dispatch_report()
    if (m, n, k) == (1100, 8000, 512):     # enough tiles for CTA pairs (512 weight rows x 256 tokens), ragged in both
        assert "pair tile 512 rows x 256 tokens, 128 k per stage" in report, report
        ctx.set_int4_prefill_cta_pairs(False)
        try:
            one = ctx.packed_int4_gemm(packed, scales, act, m, n, k, g)
            assert "CTA tile 256 rows x 256 tokens" in ctx.dispatch_report(), ctx.dispatch_report()
        finally:
            ctx.set_int4_prefill_cta_pairs(True)
        # same bf16 products, same order over k
        assert np.array_equal(one, got)
    if (m, n, k) == (1100, 8000, 448):     # K not a multiple of 128: CTA pairs with one 64-k sub-block per stage
        assert "pair tile 512 rows x 256 tokens, 64 k per stage" in report, report
    if (m, n, k) == (64, 1024, 4096):      # a wide decode batch on a narrow matrix: two sub-blocks, K slices
        assert "128 k per stage" in report and "K slice(s)" in report and "1 K slice(s)" not in report, report
    e = fro_err(got, want)
    assert e <= FRO_TOL, e
    assert e > 1e-6          # it really is the bf16 path
    assert ctx.device_status() == 0
    # every row is as good as the whole: no tile is left out or duplicated
    rows = np.linalg.norm(got - want, axis=1) / np.linalg.norm(want, axis=1)
    assert np.max(rows) <= FRO_TOL, int(np.argmax(rows))
    cols = np.linalg.norm(got - want, axis=0) / np.maximum(np.linalg.norm(want, axis=0), 1e-30)
    assert np.max(cols) <= 5 * FRO_TOL, int(np.argmax(cols))


def test_kernel_selection(ctx, oracle):
    packed, scales = make_weights(oracle, 1, 64, 256, 32)
    ctx.packed_int4_gemv(packed, scales, np.ones(256, np.float32), 64, 256, 32)
    assert "fast" in ctx.last_kernel()
    packed, scales = make_weights(oracle, 1, 64, 96, 32)
    ctx.packed_int4_gemv(packed, scales, np.ones(96, np.float32), 64, 96, 32)
    assert "generic" in ctx.last_kernel()


# ---- the benchmark configuration: K=4096, N=14336, M in {1,4,16}, seed 1 -------

@pytest.fixture(scope="module")
def config2(oracle):
    k, n, g = 4096, 14336, 32
    w_kn = synth.normal(1, 0, k * n, 0.02).reshape(k, n)   # ONNX MatMul weight [K,N]
    w_nk = np.ascontiguousarray(w_kn.T)                    # packer transposes first
    packed, scales = oracle.pack_int4(w_nk.ravel(), n, k, g)
    return k, n, g, packed, scales, w_nk


@pytest.mark.parametrize("m", [1, 4, 16])
def test_config2_parity(ctx, oracle, config2, m):
    k, n, g, packed, scales, _ = config2
    act = synth.normal(1, 1, m * k, 1.0)
    want = oracle.exec_matmul_int4(packed, scales, act, m, n, k, g)  # scalar oracle
    got = ctx.packed_int4_gemm(packed, scales, act, m, n, k, g)
    assert "fast" in ctx.last_kernel()
    assert rel_err(got, want) <= REL_TOL, rel_err(got, want)


def test_config2_properties(ctx, config2):
    """Size-independent checks at full size: linearity in the activations and
    row independence (row i of an M=16 call equals the M=1 call on that row)."""
    k, n, g, packed, scales, _ = config2
    a = synth.normal(21, 1, 16 * k, 1.0).reshape(16, k)
    full = ctx.packed_int4_gemm(packed, scales, a, 16, n, k, g)
    one = ctx.packed_int4_gemv(packed, scales, a[5], n, k, g)
    assert rel_err(full[5], one) <= 2e-6
    s = ctx.packed_int4_gemv(packed, scales, a[0] + a[1], n, k, g)
    assert rel_err(s, full[0] + full[1]) <= 1e-5
    z = ctx.packed_int4_gemv(packed, scales, np.zeros(k, np.float32), n, k, g)
    assert np.all(z == 0.0)
    twice = ctx.packed_int4_gemm(packed, scales, a, 16, n, k, g)
    assert np.array_equal(full, twice), "the kernel must be run-to-run deterministic"


def test_quantisation_error_vs_fp32(ctx, config2):
    # the reference's own sanity bound on int4 vs fp32 weights (tests/qlinear.rs:784-842)
    k, n, g, packed, scales, w_nk = config2
    act = synth.normal(3, 1, k, 1.0)
    got = ctx.packed_int4_gemv(packed, scales, act, n, k, g)
    ref = w_nk @ act
    assert rel_err(got, ref) < 0.20


def test_extreme_activations(ctx, oracle):
    n, k, g = 64, 512, 32
    packed, scales = make_weights(oracle, 5, n, k, g)
    act = synth.normal(6, 1, k, 1.0)
    act[::7] *= 1e6      # huge dynamic range between groups
    act[3::11] *= 1e-9
    act[32:64] = 0.0     # an all-zero group
    want = oracle.int4_gemv(packed, scales, act, n, k, g)
    got = ctx.packed_int4_gemv(packed, scales, act, n, k, g)
    assert rel_err(got, want) <= REL_TOL
    act[100] = np.nan
    got = ctx.packed_int4_gemv(packed, scales, act, n, k, g)
    assert np.all(np.isnan(got)), "a NaN activation reaches every output, as in fp32"
    # an infinite activation: the reference's fp32 loop (int4_matmul.rs:61-80) gives q * inf, i.e.
    # +-inf per row, or NaN where a zero nibble or infinities of both signs meet it; the integer
    # path cannot tell these apart and gives NaN for the whole group. Both are non-finite on
    # every row (documented in the header); the fp32 kernel for odd group sizes follows the
    # reference exactly.
    act[100] = np.inf
    want = oracle.int4_gemv(packed, scales, act, n, k, g)
    got = ctx.packed_int4_gemv(packed, scales, act, n, k, g)
    assert not np.any(np.isfinite(want)) and not np.any(np.isfinite(got))
    p16, s16 = oracle.pack_int4(synth.normal(5, 0, n * 48, 0.02), n, 48, 16)   # group 16: fp32 kernel
    a48 = synth.normal(6, 2, 48, 1.0)
    a48[5] = -np.inf
    want = oracle.int4_gemv(p16, s16, a48, n, 48, 16)
    got = ctx.packed_int4_gemv(p16, s16, a48, n, 48, 16)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(want)], want[~np.isnan(want)])


# ---- device-resident form -------------------------------------------------------

def test_device_resident_matches_host_form(ctx, oracle):
    import torch
    n, k, g, m = 1024, 2048, 32, 4
    packed, scales = make_weights(oracle, 31, n, k, g)
    act = synth.normal(32, 1, m * k, 1.0)
    w = ctx.int4_weight_upload(packed, scales, n, k, g)
    d_act = torch.from_numpy(act).cuda()
    d_out = torch.empty(m * n, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    ctx.int4_matmul_dev(w, d_act.data_ptr(), d_out.data_ptr(), m)
    ctx.synchronize()
    host = ctx.packed_int4_gemm(packed, scales, act, m, n, k, g)
    assert np.array_equal(d_out.cpu().numpy().reshape(m, n), host)
    # wrapping memory the caller owns
    d_p = torch.from_numpy(packed).cuda()
    d_s = torch.from_numpy(scales).cuda()
    w2 = ctx.int4_weight_wrap(d_p.data_ptr(), d_s.data_ptr(), n, k, g)
    d_out.zero_()
    torch.cuda.synchronize()
    ctx.int4_matmul_dev(w2, d_act.data_ptr(), d_out.data_ptr(), m)
    ctx.synchronize()
    assert np.array_equal(d_out.cpu().numpy().reshape(m, n), host)
    assert ctx.device_status() == 0
    w.free()
    w2.free()


# ---- packer: bit-exact ------------------------------------------------------------

@pytest.mark.parametrize("m_w,k,g", [(2, 32, 16), (4, 128, 32), (3, 96, 6), (257, 4096, 32),
                                     (64, 512, 128), (5, 64, 64)])
def test_pack_bit_exact(ctx, oracle, m_w, k, g):
    w = synth.normal(40 + m_w, 0, m_w * k, 0.02)
    w[:g] = 0.0            # an all-zero group -> scale 1.0
    w[g:2 * g] = 1e-9      # below f32::EPSILON -> scale 1.0
    w[2 * g] = 0.07        # exact ties appear once scale = abs_max/7
    want_p, want_s = oracle.pack_int4(w, m_w, k, g)
    got_p, got_s = ctx.pack_int4_symmetric_per_group(w, m_w, k, g)
    assert np.array_equal(got_s, want_s)
    assert np.array_equal(got_p, want_p)


def test_pack_lcg_case(ctx, oracle):
    w = oracle.lcg_f32(0xDEADBEEF, 2 * 32)
    want_p, want_s = oracle.pack_int4(w, 2, 32, 16)
    got_p, got_s = ctx.pack_int4_symmetric_per_group(w, 2, 32, 16)
    assert np.array_equal(got_p, want_p) and np.array_equal(got_s, want_s)


# ---- error behaviour (the reference debug_asserts; this library returns a status) ---

def test_bad_arguments(ctx):
    z8, zf = np.zeros(64, np.uint8), np.zeros(64, np.float32)
    with pytest.raises(yscv_b200.YscvCudaError) as e:
        ctx.packed_int4_gemv(z8, zf, zf, 4, 32, 15)       # odd group
    assert e.value.status == -1
    with pytest.raises(yscv_b200.YscvCudaError) as e:
        ctx.packed_int4_gemv(z8, zf, zf, 4, 40, 32)       # k % group != 0
    assert e.value.status == -1
    with pytest.raises(yscv_b200.YscvCudaError):
        ctx.packed_int4_gemv(z8, zf, zf, 0, 32, 32)       # no rows
    assert ctx.packed_int4_gemm(z8, zf, np.zeros(0, np.float32), 0, 2, 32, 32).shape == (0, 2)


def test_matmulnbits_import_on_device(ctx, oracle):
    """Weights given as MatMulNBits bytes (zero point 8): converted on the device, then the same GEMV."""
    import torch
    n, k, g = 296, 512, 32
    w = oracle.lcg_f32(0x4B1D, n * k)
    packed, scales = oracle.pack_int4(w, n, k, g)
    nbits = packed ^ 0x88                      # what an exporter would have written
    torch.cuda.synchronize()
    d_src = torch.from_numpy(nbits).cuda()
    d_dst = torch.empty_like(d_src)
    torch.cuda.synchronize()
    ctx.int4_from_matmulnbits_dev(d_src.data_ptr(), d_dst.data_ptr(), d_src.numel())
    ctx.synchronize()
    assert np.array_equal(d_dst.cpu().numpy(), packed)
    act = oracle.lcg_f32(0x77, k)
    got = ctx.packed_int4_gemv(d_dst.cpu().numpy(), scales, act, n, k, g)
    want = oracle.int4_gemv(packed, scales, act, n, k, g)
    assert np.max(np.abs(got - want)) / np.max(np.abs(want)) <= 1e-4
