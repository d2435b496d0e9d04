"""Writes the golden input/output vectors under tests/golden/ (small .npz files).

    python tests/golden/make_golden.py

The reference is Rust and cannot run where this repository is built, so the vectors come
from the scalar C restatement in oracle/ (itself pinned against the known-answer tests of
the reference, tests/test_oracle_golden.py). Inputs are drawn from the reference's test
LCG (crates/yscv-kernels/src/ops/int4_matmul.rs:652-662 for f32 values,
int8_matmul.rs:880-890 for bytes) with the seeds recorded in each file, so the files can
be regenerated bit for bit. They hold the arrays both sides need: a GPU test feeds the
inputs through the C ABI and compares with the stored outputs without calling the oracle;
a CPU test checks that the oracle still reproduces them.

Shapes cover the reference's own test shapes (int4_matmul.rs:679-944,
int8_matmul.rs:892-1117, quantize.rs:1118-1183) and the edge cases of the CUDA path:
group sizes 16/32/64/128, K that is not a multiple of the 128-byte TMA tile, rows that
are not a multiple of the 8-row tile, M on both sides of GEMM_THRESHOLD = 8 and of the
16-row limit of the decode kernel, int8 K and N not multiples of 16.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent / "oracle"))
import oracle_lib  # noqa: E402

# (name, rows of W, K, group size, M list)
INT4_CASES = [
    ("ref_2x32_g16", 2, 32, 16, [1]),
    ("ref_4x128_g32", 4, 128, 32, [1, 4]),
    ("ref_8x256_g32", 8, 256, 32, [1, 2, 8, 16]),
    ("ref_8x64_g32", 8, 64, 32, [1, 4, 16, 32]),
    ("ragged_37x96_g32", 37, 96, 32, [1, 3, 7, 9, 17]),
    ("g64_24x192", 24, 192, 64, [1, 5]),
    ("g128_16x512", 16, 512, 128, [1, 2, 4, 12]),
    ("tile_264x1024_g32", 264, 1024, 32, [1, 2, 4, 8, 16, 20]),
    ("tile_130x2048_g32", 130, 2048, 32, [1, 16, 33]),
]

# (name, M, K, N, a unsigned, a zero point)
INT8_CASES = [
    ("ref_1x4x1", 1, 4, 1, False, 0),
    ("ref_3x5x7", 3, 5, 7, False, 0),
    ("ref_4x16x4", 4, 16, 4, False, 0),
    ("ref_8x64x16", 8, 64, 16, False, 0),
    ("ref_17x33x19", 17, 33, 19, False, 0),
    ("u8_64x128x48_zp128", 64, 128, 48, True, 128),
    ("u8_130x200x72_zp3", 130, 200, 72, True, 3),
    ("i8_256x256x256_zp-5", 256, 256, 256, False, -5),
]


def int4_fixtures(o):
    out = {}
    for name, n, k, g, ms in INT4_CASES:
        seed = 0x1000 + n * 131 + k
        w = o.lcg_f32(seed, n * k)
        if name.startswith("ragged"):
            w[:k] = 0.0                       # an all-zero row: scale 1.0, nibbles 0
            w[k:k + g] *= 1e-30               # a group with a tiny scale
        packed, scales = o.pack_int4(w, n, k, g)
        out[f"{name}/meta"] = np.array([n, k, g, seed], np.int64)
        if n * k <= 8192:
            out[f"{name}/w"] = w              # for the packer test; the larger cases keep only the packed form
        out[f"{name}/packed"] = packed
        out[f"{name}/scales"] = scales
        for m in ms:
            act = o.lcg_f32(seed ^ (0xA5A5 + m), m * k)
            if m == 3:
                act[:k] = 0.0                 # a zero activation row
            out[f"{name}/act_m{m}"] = act
            # exec_matmul dispatch of the reference: GEMV rows below GEMM_THRESHOLD, else GEMM
            out[f"{name}/out_m{m}"] = o.exec_matmul_int4(packed, scales, act, m, n, k, g)
    return out


def int8_fixtures(o):
    out = {}
    for name, m, k, n, unsigned, zp in INT8_CASES:
        seed = 0x2000 + m * 7 + k * 3 + n
        a = o.lcg_i8(seed, m * k)
        b = o.lcg_i8(seed + 1, k * n)
        if unsigned:
            a_store = (a.astype(np.int16) + 128).astype(np.uint8)    # the same bits ^ 0x80
            a_centered = a_store.astype(np.int64) - zp
        else:
            a_store = a
            a_centered = a.astype(np.int64) - zp
        out[f"{name}/meta"] = np.array([m, k, n, int(unsigned), zp, seed], np.int64)
        out[f"{name}/a"] = a_store
        out[f"{name}/b"] = b
        if zp == 0 and not unsigned:
            acc = o.int8_matmul(a, b, m, k, n).reshape(m, n)
        else:
            # MatMulInteger semantics of the runner (quantize.rs:1118-1183): (a - a_zp) . b in i32
            acc = (a_centered.reshape(m, k) @ b.astype(np.int64).reshape(k, n)).astype(np.int32)
        out[f"{name}/acc"] = acc
        comp = np.float32(0.75 / max(1, k))
        out[f"{name}/composite"] = np.array([comp], np.float32)
        # requant_scalar (int8_matmul.rs): separate multiply and add, ties to even, clamp
        out[f"{name}/q_u8"] = o.requant_range(acc, float(comp), 128.0, 0, 255).astype(np.uint8)
        out[f"{name}/q_i8"] = o.requant_range(acc, float(comp), -3.0, -128, 127).astype(np.int8)
        if zp == 0 and not unsigned:
            # pointwise QLinearConv epilogue (int8_requant.rs:537-556): per-channel composite and
            # correction (bias - x_zp * colsum, here any int32 vector)
            corr = (o.lcg_i8(seed + 2, n).astype(np.int32) * 37)
            comp_pc = (comp * (np.float32(1.0) + np.float32(0.125) * (np.arange(n) % 5).astype(np.float32))).astype(np.float32)
            out[f"{name}/corr"] = corr
            out[f"{name}/composite_pc"] = comp_pc
            out[f"{name}/q_pc"] = o.requant_i8_per_channel(acc.ravel(), corr, comp_pc, 4.0, n).reshape(m, n)
    return out


def decoder_fixture(o):
    """The decoder primitives on one small case each."""
    out = {}
    x = o.lcg_f32(0x3001, 5 * 64)
    gamma = o.lcg_f32(0x3002, 64) + np.float32(1.0)
    out["rms/x"], out["rms/gamma"] = x, gamma
    out["rms/y"] = o.rms_norm(x.reshape(5, 64), gamma, 1e-5)
    s = o.lcg_f32(0x3003, 777) * np.float32(8.0)
    out["silu/x"], out["silu/y"] = s, o.silu(s)
    lg = o.lcg_f32(0x3004, 3 * 1000).reshape(3, 1000)
    lg[1, 17] = lg[1, 900] = 5.0          # a tie: the last index wins
    out["argmax/logits"], out["argmax/idx"] = lg, np.array([o.argmax_last(r) for r in lg], np.int64)
    nq, nkv, d, seq = 4, 2, 16, 6
    q = o.lcg_f32(0x3005, seq * nq * d)
    k = o.lcg_f32(0x3006, seq * nkv * d)
    out["rope/q"], out["rope/k"] = q, k
    rq, rk = o.rope(q, k, nq, nkv, d, seq, 3, 10000.0)
    out["rope/q_out"], out["rope/k_out"] = rq, rk
    v = o.lcg_f32(0x3007, seq * nkv * d)
    out["attn/v"] = v
    # attention over the same q/k rotated from position 0 (the cache then holds exactly these keys)
    q0, k0 = o.rope(q, k, nq, nkv, d, seq, 0, 10000.0)
    out["attn/out_causal"] = o.gqa_attention(q0, k0, v, 1, seq, seq, nq, nkv, d, True)
    out["attn/out_full"] = o.gqa_attention(q0, k0, v, 1, seq, seq, nq, nkv, d, False)
    out["attn/meta"] = np.array([nq, nkv, d, seq, 3], np.int64)
    return out


def main():
    o = oracle_lib.load()
    for fname, fn in (("int4.npz", int4_fixtures), ("int8.npz", int8_fixtures), ("decoder_ops.npz", decoder_fixture)):
        data = fn(o)
        np.savez_compressed(HERE / fname, **data)
        print(fname, len(data), "arrays", (HERE / fname).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
