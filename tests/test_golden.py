"""The committed golden vectors (tests/golden/*.npz, written by tests/golden/make_golden.py).

CPU: the oracle still reproduces every stored output bit for bit (so a change to the
oracle that moves a number is caught against files that were written before it).
GPU: the CUDA library, through the C ABI, reproduces the stored outputs from the stored
inputs without the oracle in the loop: bit-exact for the packer and the int8 operators,
max-relative 1e-4 for the fp32-activation W4 products, 2e-5 absolute for the fp32
decoder operators.
"""
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden"
REL_TOL_W4 = 1e-4      # the reference's own scalar-vs-SIMD bound (int4_matmul.rs:720-758)


def load(name):
    z = np.load(GOLDEN / name)
    cases = {}
    for key in z.files:
        case, arr = key.split("/", 1)
        cases.setdefault(case, {})[arr] = z[key]
    return cases


INT4 = load("int4.npz")
INT8 = load("int8.npz")
OPS = np.load(GOLDEN / "decoder_ops.npz")


def max_rel(got, want):
    return float(np.max(np.abs(got.astype(np.float64) - want)) / max(float(np.max(np.abs(want))), 1e-30))


# ------------------------------------------------------------------ CPU: oracle vs the files

@pytest.mark.parametrize("name", sorted(INT4))
def test_oracle_reproduces_int4(oracle, name):
    c = INT4[name]
    n, k, g, _seed = (int(v) for v in c["meta"])
    if "w" in c:
        packed, scales = oracle.pack_int4(c["w"], n, k, g)
        assert np.array_equal(packed, c["packed"]) and np.array_equal(scales, c["scales"])
    for key in c:
        if key.startswith("act_m"):
            m = int(key[5:])
            got = oracle.exec_matmul_int4(c["packed"], c["scales"], c[key], m, n, k, g)
            assert np.array_equal(got, c[f"out_m{m}"])


@pytest.mark.parametrize("name", sorted(INT8))
def test_oracle_reproduces_int8(oracle, name):
    c = INT8[name]
    m, k, n, unsigned, zp, _seed = (int(v) for v in c["meta"])
    if not unsigned and zp == 0:
        assert np.array_equal(oracle.int8_matmul(c["a"], c["b"], m, k, n), c["acc"])
        bt = oracle.transpose_b_i8(c["b"], k, n)
        assert np.array_equal(oracle.int8_matmul_prepacked(c["a"], bt, m, k, n), c["acc"])
    else:
        # the runner's float-typed MatMulInteger (quantize.rs:1118-1183) agrees where it is exact
        got = oracle.runner_matmul_integer(c["a"].astype(np.float32), c["b"].astype(np.float32), m, k, n, float(zp))
        if np.max(np.abs(c["acc"])) < 2 ** 24:
            assert np.array_equal(got.astype(np.int64), c["acc"].astype(np.int64))
    comp = float(c["composite"][0])
    if "q_pc" in c:
        got = oracle.requant_i8_per_channel(c["acc"].ravel(), c["corr"], c["composite_pc"], 4.0, n).reshape(m, n)
        assert np.array_equal(got, c["q_pc"])
    assert np.array_equal(oracle.requant_range(c["acc"], comp, 128.0, 0, 255), c["q_u8"].astype(np.int32))
    assert np.array_equal(oracle.requant_range(c["acc"], comp, -3.0, -128, 127), c["q_i8"].astype(np.int32))


def test_oracle_reproduces_decoder_ops(oracle):
    assert np.array_equal(oracle.rms_norm(OPS["rms/x"].reshape(5, 64), OPS["rms/gamma"], 1e-5), OPS["rms/y"])
    assert np.array_equal(oracle.silu(OPS["silu/x"]), OPS["silu/y"])
    assert [oracle.argmax_last(r) for r in OPS["argmax/logits"]] == OPS["argmax/idx"].tolist()
    assert OPS["argmax/idx"][1] == 900
    nq, nkv, d, seq, off = (int(v) for v in OPS["attn/meta"])
    rq, rk = oracle.rope(OPS["rope/q"], OPS["rope/k"], nq, nkv, d, seq, off, 10000.0)
    assert np.array_equal(rq, OPS["rope/q_out"]) and np.array_equal(rk, OPS["rope/k_out"])


# ------------------------------------------------------------------ GPU: C ABI vs the files

@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(INT4))
def test_cuda_int4_matches_golden(ctx, name):
    c = INT4[name]
    n, k, g, _seed = (int(v) for v in c["meta"])
    if "w" in c:
        packed, scales = ctx.pack_int4_symmetric_per_group(c["w"], n, k, g)
        assert np.array_equal(np.asarray(packed).ravel(), c["packed"])
        assert np.array_equal(np.asarray(scales).ravel(), c["scales"])
    w = ctx.int4_weight_upload(c["packed"], c["scales"], n, k, g)
    ctx.set_int4_prefill_exact(True)
    try:
        for key in sorted(c):
            if not key.startswith("act_m"):
                continue
            m = int(key[5:])
            want = c[f"out_m{m}"]
            if m == 1:
                got = ctx.packed_int4_gemv(c["packed"], c["scales"], c[key], n, k, g)
                assert max_rel(np.asarray(got).reshape(1, n), want) <= REL_TOL_W4
            got = ctx.packed_int4_gemm(c["packed"], c["scales"], c[key], m, n, k, g)
            assert max_rel(np.asarray(got).reshape(m, n), want) <= REL_TOL_W4
            got = ctx.int4_matmul(w, c[key], m)
            assert max_rel(np.asarray(got).reshape(m, n), want) <= REL_TOL_W4
            if m == 3:     # a zero activation row gives exact zeros
                assert np.all(np.asarray(got).reshape(m, n)[0] == 0.0)
    finally:
        ctx.set_int4_prefill_exact(False)
        w.free()


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(INT8))
def test_cuda_int8_matches_golden(ctx, name):
    c = INT8[name]
    m, k, n, unsigned, zp, _seed = (int(v) for v in c["meta"])
    pk = ctx.pack_i8_b(c["b"], k, n)
    try:
        if not unsigned and zp == 0:
            assert np.array_equal(np.asarray(ctx.int8_matmul(c["a"], c["b"], m, k, n)).reshape(m, n), c["acc"])
            assert np.array_equal(np.asarray(ctx.int8_matmul_prepacked(c["a"], pk, m)).reshape(m, n), c["acc"])
        got = ctx.matmul_integer(c["a"], pk, m, a_zp=zp)
        assert np.array_equal(np.asarray(got).reshape(m, n), c["acc"])
        if "q_pc" in c:
            got = ctx.int8_matmul_requant_per_channel(c["a"], pk, m, c["corr"], c["composite_pc"], 4.0)
            assert np.array_equal(got, c["q_pc"])
        comp = float(c["composite"][0])
        rq = ctx.requant(comp, 128.0, 0, 255, a_unsigned=bool(unsigned), a_zp=zp)
        got = ctx.qlinear_matmul(c["a"], pk, m, rq)
        assert np.array_equal(np.asarray(got).reshape(m, n).view(np.uint8), c["q_u8"])
        rq = ctx.requant(comp, -3.0, -128, 127, a_unsigned=bool(unsigned), a_zp=zp)
        got = ctx.qlinear_matmul(c["a"], pk, m, rq)
        assert np.array_equal(np.asarray(got).reshape(m, n).view(np.int8), c["q_i8"])
    finally:
        pk.free()


@pytest.mark.gpu
def test_cuda_decoder_ops_match_golden(ctx):
    import torch

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    torch.cuda.synchronize()
    # RMSNorm (zero residual delta)
    x, gm = dev(OPS["rms/x"].reshape(5, 64)), dev(OPS["rms/gamma"])
    zero, xo, nm = torch.zeros_like(x), torch.empty_like(x), torch.empty_like(x)
    torch.cuda.synchronize()
    ctx.add_rms_norm_dev(x.data_ptr(), zero.data_ptr(), gm.data_ptr(), 1e-5, 5, 64, xo.data_ptr(), nm.data_ptr())
    ctx.synchronize()
    assert np.max(np.abs(nm.cpu().numpy() - OPS["rms/y"])) < 2e-5
    # SiLU through SwiGLU with an all-ones up half
    sx = OPS["silu/x"]
    gu = dev(np.concatenate([sx, np.ones_like(sx)])[None, :])
    so = torch.empty(1, sx.size, device="cuda")
    torch.cuda.synchronize()
    ctx.swiglu_dev(gu.data_ptr(), 1, sx.size, so.data_ptr())
    ctx.synchronize()
    assert np.max(np.abs(so.cpu().numpy().ravel() - OPS["silu/y"])) < 2e-6
    # argmax-last
    lg = dev(OPS["argmax/logits"])
    am = torch.empty(3, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    ctx.argmax_last_dev(lg.data_ptr(), 3, 1000, am.data_ptr())
    ctx.synchronize()
    assert am.cpu().numpy().tolist() == OPS["argmax/idx"].tolist()
    # RoPE + cache append at position 3; then attention from position 0
    nq, nkv, d, seq, off = (int(v) for v in OPS["attn/meta"])
    q = OPS["rope/q"].reshape(seq, nq * d)
    k = OPS["rope/k"].reshape(seq, nkv * d)
    v = OPS["attn/v"].reshape(seq, nkv * d)
    max_seq = 16
    for start in (off, 0):
        qkv = dev(np.concatenate([q, k, v], axis=1))
        kc = torch.zeros(1, max_seq, nkv * d, device="cuda")
        vc = torch.zeros_like(kc)
        pos = torch.full((1,), start, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        ctx.rope_kv_append_dev(qkv.data_ptr(), 1, seq, nq, nkv, d, 10000.0, pos.data_ptr(), kc.data_ptr(),
                               vc.data_ptr(), max_seq)
        ctx.synchronize()
        if start == off:
            assert np.max(np.abs(qkv[:, :nq * d].cpu().numpy().ravel() - OPS["rope/q_out"])) < 2e-5
            assert np.max(np.abs(kc[0, off:off + seq].cpu().numpy().ravel() - OPS["rope/k_out"])) < 2e-5
            assert np.array_equal(vc[0, off:off + seq].cpu().numpy(), v)
            continue
        for causal, key in ((True, "attn/out_causal"), (False, "attn/out_full")):
            out = torch.empty(seq, nq * d, device="cuda")
            torch.cuda.synchronize()
            ctx.gqa_attention_dev(qkv.data_ptr(), (nq + 2 * nkv) * d, 1, seq, nq, nkv, d, kc.data_ptr(),
                                  vc.data_ptr(), max_seq, pos.data_ptr(), causal, out.data_ptr())
            ctx.synchronize()
            assert np.max(np.abs(out.cpu().numpy().ravel() - OPS[key])) < 2e-5
    assert ctx.device_status() == 0
