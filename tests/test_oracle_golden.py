"""Pins the CPU oracle against the known-answer tests the reference ships for
this path (reference file:line in each test). CPU only."""
import numpy as np
import pytest


# crates/yscv-kernels/src/ops/int4_matmul.rs:665-676
def test_unpack_extreme_nibbles(oracle):
    assert oracle.lib.yo_unpack_low(0x78) == -8
    assert oracle.lib.yo_unpack_high(0x78) == 7
    assert oracle.lib.yo_unpack_low(0x00) == 0 and oracle.lib.yo_unpack_high(0x00) == 0
    assert oracle.lib.yo_unpack_low(0xFF) == -1 and oracle.lib.yo_unpack_high(0xFF) == -1


def test_unpack_all_bytes(oracle):
    for b in range(256):
        lo, hi = b & 15, b >> 4
        assert oracle.lib.yo_unpack_low(b) == (lo - 16 if lo >= 8 else lo)
        assert oracle.lib.yo_unpack_high(b) == (hi - 16 if hi >= 8 else hi)


# int4_matmul.rs:652-662: the test LCG. First values computed by hand from the recurrence.
def test_lcg_f32_recurrence(oracle):
    seed, s, want = 0xCAFEBABE, 0xCAFEBABE, []
    for _ in range(5):
        s = (s * 6364136223846793005 + 1442695040888963407) & (2**64 - 1)
        want.append(np.float32(((s >> 33) % 2001) - 1000) * np.float32(0.001))
    got = oracle.lcg_f32(seed, 5)
    assert np.array_equal(got, np.array(want, np.float32))
    assert np.all(np.abs(oracle.lcg_f32(1, 4096)) <= 1.0)


# int4_matmul.rs:679-717: pack -> GEMV against an fp32 dot, rel < 0.12
def test_pack_then_gemv_close_to_fp32(oracle):
    m_w, k, g = 2, 32, 16
    w = oracle.lcg_f32(0xDEADBEEF, m_w * k)
    packed, scales = oracle.pack_int4(w, m_w, k, g)
    act = np.ones(k, np.float32)
    got = oracle.int4_gemv(packed, scales, act, m_w, k, g)
    want = w.reshape(m_w, k).sum(axis=1)
    assert np.all(np.abs(got - want) / np.maximum(np.abs(want), 1e-6) < 0.12)


# int4_matmul.rs:760-773: zero weights -> scale 1.0, zero output
def test_zero_weights(oracle):
    packed, scales = oracle.pack_int4(np.zeros(3 * 32, np.float32), 3, 32, 16)
    assert np.all(scales == 1.0) and np.all(packed == 0)
    out = oracle.int4_gemv(packed, scales, np.full(32, 1.5, np.float32), 3, 32, 16)
    assert np.all(np.abs(out) <= 1e-5)


# int4_matmul.rs:775-813: GEMM(M=1) == GEMV within 1e-5
def test_gemm_m1_matches_gemv(oracle):
    n, k, g = 4, 64, 32
    packed, scales = oracle.pack_int4(oracle.lcg_f32(0xAA, n * k), n, k, g)
    act = oracle.lcg_f32(0xBB, k)
    a = oracle.int4_gemv(packed, scales, act, n, k, g)
    b = oracle.int4_gemm(packed, scales, act, 1, n, k, g)[0]
    assert np.max(np.abs(a - b)) <= 1e-5


# int4_matmul.rs:720-758, 815-944: the SIMD restatements stay within the
# reference's own tolerances of the scalar oracle
@pytest.mark.parametrize("m_w,k,g,sw,sa,tol", [
    (4, 128, 32, 0xCAFEBABE, 0xF00DBA12, 1e-4),
    (8, 256, 32, 0x12345678, 0x9ABCDEF0, 1e-4),
])
def test_simd_gemv_matches_scalar(oracle, m_w, k, g, sw, sa, tol):
    packed, scales = oracle.pack_int4(oracle.lcg_f32(sw, m_w * k), m_w, k, g)
    act = oracle.lcg_f32(sa, k)
    assert np.max(np.abs(oracle.int4_gemv(packed, scales, act, m_w, k, g) -
                         oracle.int4_gemv(packed, scales, act, m_w, k, g, simd=True))) <= tol


def test_simd_gemm_matches_scalar(oracle):
    n, k, g = 8, 64, 32
    packed, scales = oracle.pack_int4(oracle.lcg_f32(0x100, n * k), n, k, g)
    for m in (1, 4, 16, 32):
        act = oracle.lcg_f32(0x200 + m, m * k)
        d = oracle.int4_gemm(packed, scales, act, m, n, k, g) - \
            oracle.int4_gemm(packed, scales, act, m, n, k, g, simd=True)
        assert np.max(np.abs(d)) <= 1e-3


def test_packer_layout_and_rounding(oracle):
    # one group, abs_max 7 -> scale 1, inv 1: values quantise to themselves; ties go to even
    w = np.array([7.0, -7.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5] + [0.0] * 24, np.float32)
    packed, scales = oracle.pack_int4(w, 1, 32, 32)
    assert scales[0] == 1.0
    q = [7, -7, 0, 2, 2, 0, -2, -2]
    want = [(q[2 * i] & 15) | ((q[2 * i + 1] & 15) << 4) for i in range(4)]
    assert list(packed[:4]) == want
    # abs_max below f32::EPSILON -> scale 1.0
    _, s2 = oracle.pack_int4(np.full(32, 1e-8, np.float32), 1, 32, 32)
    assert s2[0] == 1.0


# crates/yscv-kernels/src/ops/int8_matmul.rs:2458-2465
def test_int8_known_small_case(oracle):
    out = oracle.int8_matmul(np.array([1, 2, 3, 4], np.int8), np.array([5, 6, 7, 8], np.int8), 2, 2, 2)
    assert out.ravel().tolist() == [19, 22, 43, 50]


# int8_matmul.rs:2502-2509
def test_int8_extreme_values(oracle):
    a = np.full(128, -128, np.int8)
    for simd in (False, True):
        assert oracle.int8_matmul(a, a, 1, 128, 1, simd=simd)[0, 0] == 128 * 128 * 128


# int8_matmul.rs:2467-2500: dispatch and prepacked forms are bit-exact vs scalar on odd shapes
@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (2, 3, 4), (4, 16, 8), (5, 17, 6), (8, 64, 8),
                                   (1, 17, 5), (3, 31, 7), (4, 64, 16), (8, 127, 33), (16, 128, 64),
                                   (8, 8192, 32), (4, 70, 48)])
def test_int8_simd_bit_exact(oracle, m, k, n):
    a = oracle.lcg_i8(0xDEAD ^ (m * k), m * k)
    b = oracle.lcg_i8(0xBEEF ^ (k * n), k * n)
    want = oracle.int8_matmul(a, b, m, k, n)
    assert np.array_equal(oracle.int8_matmul(a, b, m, k, n, simd=True), want)
    bt = oracle.transpose_b_i8(b, k, n)
    assert np.array_equal(bt.reshape(n, k), b.reshape(k, n).T)
    assert np.array_equal(oracle.int8_matmul_prepacked(a, bt, m, k, n), want)
    assert np.array_equal(oracle.int8_matmul_prepacked(a, bt, m, k, n, simd=True), want)
    assert np.array_equal(oracle.int8_matmul_prepacked(a, bt, m, k, n, threads=3), want)
    # numpy cross-check of the scalar oracle itself
    assert np.array_equal(want, a.reshape(m, k).astype(np.int32) @ b.reshape(k, n).astype(np.int32))


# crates/yscv-kernels/src/ops/int8_requant.rs:1216-1227
def test_requant_round_half_even(oracle):
    acc = np.array([1, -1, 3, -3, 5, -5, 7, -7], np.int32)
    assert oracle.requant_i8(acc, None, 0.5, 0.0, False, 8).tolist() == [0, 0, 2, -2, 2, -2, 4, -4]
    assert oracle.requant_range(acc, 0.5, 0.0, -128, 127).tolist() == [0, 0, 2, -2, 2, -2, 4, -4]


# int8_requant.rs:1195-1213
def test_requant_saturation(oracle):
    acc = np.array([1_000_000] * 8 + [-1_000_000] * 8, np.int32)
    got = oracle.requant_i8(acc, None, 0.001, 0.0, False, 16)
    assert got[:8].tolist() == [127] * 8 and got[8:].tolist() == [-128] * 8
    u = oracle.requant_range(acc, 0.001, 128.0, 0, 255)
    assert u[:8].tolist() == [255] * 8 and u[8:].tolist() == [0] * 8


# int8_requant.rs:1190-1193 (ReLU clamps negatives to 0) and bias wrapping add
def test_requant_relu_and_bias(oracle):
    acc = np.full(12, -100, np.int32)
    assert np.all(oracle.requant_i8(acc, None, 1.0, 0.0, True, 4) == 0)
    got = oracle.requant_i8(np.array([10, 20], np.int32), np.array([5, -30], np.int32), 1.0, 0.0, False, 2)
    assert got.tolist() == [15, -10]


def test_requant_per_channel(oracle):
    acc = np.array([1, 3, 5, 7, 1, 3, 5, 7], np.int32)
    got = oracle.requant_i8_per_channel(acc, np.array([0, 0, 1, -7], np.int32),
                                        np.array([0.5, 0.5, 1.0, 2.0], np.float32), 0.0, 4)
    assert got.tolist() == [0, 2, 6, 0, 0, 2, 6, 0]


# crates/yscv-kernels/src/ops/quantize.rs:242-254
def test_quantize_linear(oracle):
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, 1000.0, -1000.0], np.float32)
    assert oracle.quantize_linear(x, 1.0, 0.0).tolist() == [0, 2, 2, 0, -2, 127, -128]
    assert oracle.quantize_linear(x, 1.0, 128.0, unsigned=True).tolist() == [128, 130, 130, 128, 126, 255, 0]


# crates/yscv-onnx/src/tests/qlinear.rs:150-194 (QLinearMatMul 4x8x4, scales 0.05/0.1/0.25)
def test_runner_qlinear_matmul_symmetric(oracle):
    a_int = np.arange(32, dtype=np.int32) - 16
    b_int = (np.arange(32, dtype=np.int32) * 7) % 31 - 15
    got = oracle.runner_qlinear_matmul_fast(a_int.astype(np.float32), b_int.astype(np.float32),
                                            4, 8, 4, 0.05, 0.1, 0.25, 0.0)
    composite = np.float32(np.float32(0.05) * np.float32(0.1)) / np.float32(0.25)
    acc = a_int.reshape(4, 8) @ b_int.reshape(8, 4)
    v = acc.astype(np.float32) * composite
    want = np.clip(np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)), -128, 127)
    assert np.max(np.abs(got - want)) <= 1e-4


# crates/yscv-onnx/src/tests/coverage.rs:304-357 (unit scales == plain matmul, clamped)
def test_runner_qlinear_matmul_unit_scales(oracle):
    a = np.array([1, 2, 3, 4, 5, 6], np.float32)
    b = np.array([0.5, -0.5, 1.0, -1.0, 0.0, 2.0], np.float32)
    # the runner casts operands with `as i8` (truncation): 0.5 -> 0, -0.5 -> 0
    got = oracle.runner_qlinear_matmul_fast(a, b, 2, 3, 2, 1.0, 1.0, 1.0, 0.0)
    bi = np.trunc(b).reshape(3, 2)
    assert np.array_equal(got, np.clip(a.reshape(2, 3) @ bi, -128, 127))


# crates/yscv-onnx/src/tests/qlinear.rs:667-705 and coverage.rs:359-390, gemm_matmul.rs:73-87
def test_runner_matmul_integer(oracle):
    a_int = np.arange(24, dtype=np.int32) - 12
    b_int = (np.arange(24, dtype=np.int32) * 5) % 23 - 11
    got = oracle.runner_matmul_integer(a_int.astype(np.float32), b_int.astype(np.float32), 3, 8, 3)
    assert np.array_equal(got, (a_int.reshape(3, 8) @ b_int.reshape(8, 3)).astype(np.float32))
    z = oracle.runner_matmul_integer(np.array([10, 11, 12, 13], np.float32),
                                     np.array([1, 0, 0, 1], np.float32), 2, 2, 2, a_zp=10.0)
    assert z.ravel().tolist() == [0.0, 1.0, 2.0, 3.0]
    y = oracle.runner_matmul_integer(np.array([1, 2, 3, 4], np.float32),
                                     np.array([5, 6, 7, 8], np.float32), 2, 2, 2)
    assert y.ravel().tolist() == [19.0, 22.0, 43.0, 50.0]


# crates/yscv-onnx/src/tests/qlinear.rs:784-842: int4 routing K=64, N=8, g=32, rel < 0.20 vs fp32
def test_runner_int4_matmul_close_to_fp32(oracle):
    k, n = 64, 8
    w = ((np.arange(k * n, dtype=np.float32) / np.float32(k * n)) - np.float32(0.5)) * np.float32(0.3)
    act = (np.arange(k, dtype=np.float32) - 32.0) * np.float32(0.05)
    ref = act @ w.reshape(k, n)
    w_nk = np.ascontiguousarray(w.reshape(k, n).T)
    packed, scales = oracle.pack_int4(w_nk, n, k, 32)
    got = oracle.exec_matmul_int4(packed, scales, act, 1, n, k, 32)[0]
    assert np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-6) < 0.20


def test_exec_matmul_threshold(oracle):
    # M < 8 -> per-row GEMV, M >= 8 -> GEMM (runner/linear.rs:242-267)
    n, k, g = 8, 64, 32
    packed, scales = oracle.pack_int4(oracle.lcg_f32(7, n * k), n, k, g)
    for m in (1, 7, 8, 9):
        act = oracle.lcg_f32(100 + m, m * k)
        got = oracle.exec_matmul_int4(packed, scales, act, m, n, k, g)
        if m >= 8:
            want = oracle.int4_gemm(packed, scales, act, m, n, k, g)
        else:
            want = np.stack([oracle.int4_gemv(packed, scales, act[i * k:(i + 1) * k], n, k, g) for i in range(m)])
        assert np.array_equal(got, want)
        assert np.array_equal(oracle.exec_matmul_int4(packed, scales, act, m, n, k, g, threads=3).shape, want.shape)


def test_decoder_primitives(oracle):
    x = oracle.lcg_f32(5, 2 * 64).reshape(2, 64)
    g = np.ones(64, np.float32)
    y = oracle.rms_norm(x, g, 1e-5)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5)
    assert np.max(np.abs(y - want)) < 1e-5
    # rotate-half RoPE: position 0 is the identity, norms are preserved
    q = oracle.lcg_f32(6, 3 * 2 * 8)
    k = oracle.lcg_f32(7, 3 * 1 * 8)
    q2, k2 = oracle.rope(q, k, 2, 1, 8, 3, 0, 10000.0)
    assert np.allclose(q2[:16], q[:16]) and np.allclose(k2[:8], k[:8])
    assert np.allclose(np.linalg.norm(q2.reshape(6, 8), axis=1), np.linalg.norm(q.reshape(6, 8), axis=1), atol=1e-5)
    # pair (i, i+half): angle = pos / theta^(2i/d)
    ang = 1.0 / 10000.0 ** (2.0 * 1 / 8)
    x0, x1 = q[16 + 1], q[16 + 1 + 4]  # pos 1, head 0 -> offset 16
    assert abs(q2[16 + 1] - (x0 * np.cos(ang) - x1 * np.sin(ang))) < 1e-6
    s = oracle.silu(np.array([0.0, 1.0, -1.0], np.float32))
    assert np.allclose(s, [0.0, 0.7310586, -0.26894143], atol=1e-6)
    assert oracle.argmax_last(np.array([1.0, 3.0, 3.0, 2.0], np.float32)) == 2
    # attention: uniform keys -> output is the mean of V
    qq = np.zeros(1 * 1 * 2 * 4, np.float32)
    kk = oracle.lcg_f32(8, 3 * 1 * 4)
    vv = oracle.lcg_f32(9, 3 * 1 * 4)
    o = oracle.gqa_attention(qq, kk, vv, 1, 1, 3, 2, 1, 4, False)
    assert np.allclose(o.reshape(2, 4), vv.reshape(3, 4).mean(axis=0), atol=1e-6)


def test_kv_cache_int8_reference_cases(oracle):
    # crates/yscv-onnx/src/runner/kv_cache.rs:318-357: the round trip stays within one
    # quantisation step of each row's own scale (abs_max / 127)
    k = np.array([[-3.0, -2.5, -1.0, 0.0, 0.5, 1.5, 2.0, 2.8],
                  [0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8]], np.float32)
    v = np.array([[10.0, 20.0, -30.0, 40.0, -50.0, 60.0, -70.0, 80.0],
                  [1.0, -1.0, 2.0, -2.0, 3.0, -3.0, 4.0, -4.0]], np.float32)
    for rows, maxima in ((k, (3.0, 0.8)), (v, (80.0, 4.0))):
        q, s = oracle.kv_append_i8(rows)
        back = oracle.kv_dequantise_i8(q, s)
        for r, mx in enumerate(maxima):
            assert s[r] == np.float32(mx) / np.float32(127.0)
            assert np.all(np.abs(back[r] - rows[r]) <= mx / 127.0)
        assert q.min() >= -127 and q.max() <= 127
        assert np.all(np.abs(q).max(axis=1) == 127)   # the row maximum maps to +-127
    # kv_cache.rs:360-375: a constant row of 5.0 comes back within 0.05
    q, s = oracle.kv_append_i8(np.full((1, 4), 5.0, np.float32))
    assert abs(float(oracle.kv_dequantise_i8(q, s)[0, 0]) - 5.0) < 0.05
    # a row at or below f32::EPSILON keeps scale 1.0 (kv_cache.rs:50-54) and rounds to zero
    q, s = oracle.kv_append_i8(np.full((1, 4), 1e-8, np.float32))
    assert s[0] == 1.0 and not q.any()
    # f32::round is half away from zero: 0.5 steps of the scale
    row = np.array([[127.0, 0.5, -0.5, 1.5, -2.5]], np.float32)
    q, s = oracle.kv_append_i8(row)
    assert s[0] == 1.0 and q.tolist() == [[127, 1, -1, 2, -3]]
