"""ctypes access to the CPU oracle (libyscv_oracle.so, built from this folder).

TEST INFRASTRUCTURE ONLY: imported by the tests, by the smoke check and by the
benchmark's CPU-baseline leg. The oracle is the checker, never part of the
code path under test, and the shipped package does not import it.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent
_LIB = None

_vp, _sz, _f = C.c_void_p, C.c_size_t, C.c_float


def build() -> Path:
    so = ORACLE_DIR / "libyscv_oracle.so"
    srcs = [ORACLE_DIR / n for n in ("yscv_oracle.c", "yscv_simd_baseline.c", "yscv_oracle.h")]
    if not so.exists() or any(s.stat().st_mtime > so.stat().st_mtime for s in srcs):
        subprocess.run(["make", "-C", str(ORACLE_DIR)], check=True, capture_output=True)
    return so


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        lib.yo_unpack_low.restype = C.c_int8
        lib.yo_unpack_low.argtypes = [C.c_uint8]
        lib.yo_unpack_high.restype = C.c_int8
        lib.yo_unpack_high.argtypes = [C.c_uint8]
        lib.yo_argmax_last.restype = C.c_uint32
        lib.yo_argmax_last.argtypes = [_vp, _sz]
        lib.ysb_isa.restype = C.c_char_p
        sigs = {
            "yo_packed_int4_gemv": [_vp, _vp, _vp, _vp, _sz, _sz, _sz],
            "yo_packed_int4_gemm": [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz],
            "yo_exec_matmul_int4": [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz],
            "yo_pack_int4_symmetric_per_group": [_vp, _sz, _sz, _sz, _vp, _vp],
            "yo_transpose_kn_to_nk": [_vp, _sz, _sz, _vp],
            "yo_int8_matmul": [_vp, _vp, _sz, _sz, _sz, _vp],
            "yo_transpose_b_i8": [_vp, _sz, _sz, _vp],
            "yo_int8_matmul_prepacked": [_vp, _vp, _sz, _sz, _sz, _vp],
            "yo_requant_i8": [_vp, _sz, _vp, _f, _f, C.c_int, _vp, _sz],
            "yo_requant_range": [_vp, _sz, _f, _f, C.c_int32, C.c_int32, _vp],
            "yo_requant_i8_per_channel": [_vp, _sz, _vp, _vp, _f, _vp, _sz],
            "yo_quantize_linear_i8": [_vp, _sz, _f, _f, _vp],
            "yo_quantize_linear_u8": [_vp, _sz, _f, _f, _vp],
            "yo_quantize_tensor_symmetric": [_vp, _sz, _f, _vp],
            "yo_runner_qlinear_matmul_fast": [_vp, _vp, _sz, _sz, _sz, _f, _f, _f, _f, _vp],
            "yo_runner_matmul_integer": [_vp, _vp, _sz, _sz, _sz, _f, _f, _vp],
            "yo_rms_norm": [_vp, _sz, _sz, _vp, _f, _vp],
            "yo_rope": [_vp, _vp, _sz, _sz, _sz, _sz, _sz, _f],
            "yo_gqa_attention": [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, C.c_int, _vp],
            "yo_silu": [_vp, _sz, _vp],
            "yo_kv_append_i8": [_vp, _sz, _sz, _vp, _vp],
            "yo_kv_dequantise_i8": [_vp, _vp, _sz, _sz, _vp],
            "yo_lcg_f32": [C.c_uint64, _sz, _vp],
            "yo_lcg_i8": [C.c_uint64, _sz, _vp],
            "ysb_int4_gemv": [_vp, _vp, _vp, _vp, _sz, _sz, _sz],
            "ysb_int4_gemm": [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz],
            "ysb_int8_matmul": [_vp, _vp, _sz, _sz, _sz, _vp],
            "ysb_int8_matmul_prepacked": [_vp, _vp, _sz, _sz, _sz, _vp],
            "ysb_exec_matmul_int4_mt": [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, C.c_int],
            "ysb_int8_matmul_prepacked_mt": [_vp, _vp, _sz, _sz, _sz, _vp, C.c_int],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.restype = None
            fn.argtypes = args

    # ---- helpers --------------------------------------------------------------
    @staticmethod
    def _p(a: np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data

    def isa(self) -> str:
        return self.lib.ysb_isa().decode()

    def lcg_f32(self, seed, n):
        out = np.empty(n, np.float32)
        self.lib.yo_lcg_f32(seed, n, self._p(out))
        return out

    def lcg_i8(self, seed, n):
        out = np.empty(n, np.int8)
        self.lib.yo_lcg_i8(seed, n, self._p(out))
        return out

    def pack_int4(self, w, m_w, k, gs):
        w = np.ascontiguousarray(w, np.float32)
        packed = np.empty(m_w * k // 2, np.uint8)
        scales = np.empty(m_w * (k // gs), np.float32)
        self.lib.yo_pack_int4_symmetric_per_group(self._p(w), m_w, k, gs, self._p(packed), self._p(scales))
        return packed, scales

    def int4_gemv(self, packed, scales, act, m_w, k, gs, simd=False):
        act = np.ascontiguousarray(act, np.float32)
        out = np.empty(m_w, np.float32)
        fn = self.lib.ysb_int4_gemv if simd else self.lib.yo_packed_int4_gemv
        fn(self._p(packed), self._p(scales), self._p(act), self._p(out), m_w, k, gs)
        return out

    def int4_gemm(self, packed, scales, act, m, n, k, gs, simd=False):
        act = np.ascontiguousarray(act, np.float32)
        out = np.empty((m, n), np.float32)
        fn = self.lib.ysb_int4_gemm if simd else self.lib.yo_packed_int4_gemm
        fn(self._p(packed), self._p(scales), self._p(act), self._p(out), m, n, k, gs)
        return out

    def exec_matmul_int4(self, packed, scales, act, m, n, k, gs, threads=0):
        act = np.ascontiguousarray(act, np.float32)
        out = np.empty((m, n), np.float32)
        if threads:
            self.lib.ysb_exec_matmul_int4_mt(self._p(packed), self._p(scales), self._p(act),
                                             self._p(out), m, n, k, gs, threads)
        else:
            self.lib.yo_exec_matmul_int4(self._p(packed), self._p(scales), self._p(act),
                                         self._p(out), m, n, k, gs)
        return out

    def int8_matmul(self, a, b, m, k, n, simd=False):
        a = np.ascontiguousarray(a, np.int8)
        b = np.ascontiguousarray(b, np.int8)
        out = np.empty((m, n), np.int32)
        fn = self.lib.ysb_int8_matmul if simd else self.lib.yo_int8_matmul
        fn(self._p(a), self._p(b), m, k, n, self._p(out))
        return out

    def transpose_b_i8(self, b, k, n):
        b = np.ascontiguousarray(b, np.int8)
        bt = np.empty(n * k, np.int8)
        self.lib.yo_transpose_b_i8(self._p(b), k, n, self._p(bt))
        return bt

    def int8_matmul_prepacked(self, a, bt, m, k, n, simd=False, threads=0):
        a = np.ascontiguousarray(a, np.int8)
        out = np.empty((m, n), np.int32)
        if threads:
            self.lib.ysb_int8_matmul_prepacked_mt(self._p(a), self._p(bt), m, k, n, self._p(out), threads)
        else:
            fn = self.lib.ysb_int8_matmul_prepacked if simd else self.lib.yo_int8_matmul_prepacked
            fn(self._p(a), self._p(bt), m, k, n, self._p(out))
        return out

    def requant_i8(self, acc, bias, composite, y_zp, relu, c):
        acc = np.ascontiguousarray(acc, np.int32)
        out = np.empty(acc.size, np.int8)
        bp = None if bias is None else self._p(np.ascontiguousarray(bias, np.int32))
        self.lib.yo_requant_i8(self._p(acc), acc.size, bp, composite, y_zp, int(relu), self._p(out), c)
        return out

    def requant_range(self, acc, composite, y_zp, lo, hi):
        acc = np.ascontiguousarray(acc, np.int32)
        out = np.empty(acc.shape, np.int32)
        self.lib.yo_requant_range(self._p(acc), acc.size, composite, y_zp, lo, hi, self._p(out))
        return out

    def requant_i8_per_channel(self, acc, corr, composite, y_zp, c):
        acc = np.ascontiguousarray(acc, np.int32)
        corr = np.ascontiguousarray(corr, np.int32)
        composite = np.ascontiguousarray(composite, np.float32)
        out = np.empty(acc.size, np.int8)
        self.lib.yo_requant_i8_per_channel(self._p(acc), acc.size, self._p(corr), self._p(composite),
                                           y_zp, self._p(out), c)
        return out

    def quantize_linear(self, data, scale, zp, unsigned=False):
        data = np.ascontiguousarray(data, np.float32)
        out = np.empty(data.shape, np.uint8 if unsigned else np.int8)
        fn = self.lib.yo_quantize_linear_u8 if unsigned else self.lib.yo_quantize_linear_i8
        fn(self._p(data), data.size, scale, zp, self._p(out))
        return out

    def quantize_tensor_symmetric(self, data, scale):
        data = np.ascontiguousarray(data, np.float32)
        out = np.empty(data.shape, np.int8)
        self.lib.yo_quantize_tensor_symmetric(self._p(data), data.size, scale, self._p(out))
        return out

    def runner_qlinear_matmul_fast(self, a, b, m, k, n, a_s, b_s, y_s, y_zp):
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        out = np.empty((m, n), np.float32)
        self.lib.yo_runner_qlinear_matmul_fast(self._p(a), self._p(b), m, k, n, a_s, b_s, y_s, y_zp, self._p(out))
        return out

    def runner_matmul_integer(self, a, b, m, k, n, a_zp=0.0, b_zp=0.0):
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        out = np.empty((m, n), np.float32)
        self.lib.yo_runner_matmul_integer(self._p(a), self._p(b), m, k, n, a_zp, b_zp, self._p(out))
        return out

    def rms_norm(self, x, gamma, eps):
        x = np.ascontiguousarray(x, np.float32)
        gamma = np.ascontiguousarray(gamma, np.float32)
        out = np.empty_like(x)
        self.lib.yo_rms_norm(self._p(x), x.shape[0], x.shape[1], self._p(gamma), eps, self._p(out))
        return out

    def rope(self, q, k, n_q, n_kv, d, seq, offset, theta):
        q = np.ascontiguousarray(q, np.float32).copy()
        k = np.ascontiguousarray(k, np.float32).copy()
        self.lib.yo_rope(self._p(q), self._p(k), n_q, n_kv, d, seq, offset, theta)
        return q, k

    def gqa_attention(self, q, k, v, batch, sq, sk, n_q, n_kv, d, causal):
        q, k, v = (np.ascontiguousarray(t, np.float32) for t in (q, k, v))
        out = np.empty(batch * sq * n_q * d, np.float32)
        self.lib.yo_gqa_attention(self._p(q), self._p(k), self._p(v), batch, sq, sk, n_q, n_kv, d,
                                  int(causal), self._p(out))
        return out

    def kv_append_i8(self, rows):
        """rows f32 [n, kv_dim] -> (int8 [n, kv_dim], scales f32 [n]) as KvDtype::I8 stores them."""
        rows = np.ascontiguousarray(rows, np.float32)
        n, kv_dim = rows.shape
        data = np.empty((n, kv_dim), np.int8)
        scales = np.empty(n, np.float32)
        self.lib.yo_kv_append_i8(self._p(rows), n, kv_dim, self._p(data), self._p(scales))
        return data, scales

    def kv_dequantise_i8(self, data, scales):
        data = np.ascontiguousarray(data, np.int8)
        scales = np.ascontiguousarray(scales, np.float32)
        out = np.empty(data.shape, np.float32)
        self.lib.yo_kv_dequantise_i8(self._p(data), self._p(scales), data.shape[0], data.shape[1], self._p(out))
        return out

    def silu(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        self.lib.yo_silu(self._p(x), x.size, self._p(out))
        return out

    def argmax_last(self, logits):
        logits = np.ascontiguousarray(logits, np.float32)
        return int(self.lib.yo_argmax_last(self._p(logits), logits.size))


def load() -> Oracle:
    global _LIB
    if _LIB is None:
        _LIB = Oracle(C.CDLL(str(build())))
    return _LIB
