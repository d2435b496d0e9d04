"""ctypes binding of include/yscv_cuda.h.

Every call goes through the C ABI of ``libyscv_cuda.so``. Loading fails loudly
when the library has not been built; nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

_LIB = None


class YscvCudaError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"yscv_cuda status {status}: {message}")
        self.status = status


def library_path() -> Path:
    return Path(__file__).resolve().parent / "libyscv_cuda.so"


_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)
_vp = C.c_void_p
_sz = C.c_size_t

# name -> (restype, argtypes); mirrors include/yscv_cuda.h one to one
SIGNATURES = {
    "yscv_cuda_ctx_create": (C.c_int, [C.c_int, C.POINTER(_vp)]),
    "yscv_cuda_ctx_create_on_stream": (C.c_int, [C.c_int, _vp, C.POINTER(_vp)]),
    "yscv_cuda_ctx_destroy": (None, [_vp]),
    "yscv_cuda_ctx_synchronize": (C.c_int, [_vp]),
    "yscv_cuda_ctx_device_status": (C.c_int, [_vp, C.POINTER(C.c_int)]),
    "yscv_cuda_last_error": (C.c_char_p, []),
    "yscv_cuda_last_kernel": (C.c_char_p, [_vp]),
    "yscv_cuda_ctx_launch_count": (C.c_uint64, [_vp]),
    "yscv_cuda_ctx_set_int4_prefill_exact": (C.c_int, [_vp, C.c_int]),
    "yscv_cuda_ctx_set_int8_cta_pairs": (C.c_int, [_vp, C.c_int]),
    "yscv_cuda_ctx_set_int4_prefill_cta_pairs": (C.c_int, [_vp, C.c_int]),
    "yscv_cuda_ctx_set_int8_tail_split": (C.c_int, [_vp, C.c_int]),
    "yscv_cuda_ctx_set_attention_tensor_cores": (C.c_int, [_vp, C.c_int]),
    "yscv_cuda_ctx_set_f32_tensor_cores": (C.c_int, [_vp, C.c_int]),
    "yscv_cuda_ctx_profile_enable": (C.c_int, [_vp, C.c_int]),
    "yscv_cuda_ctx_profile_read": (C.c_int, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_double)]),
    "yscv_cuda_int4_matmul": (C.c_int, [_vp, _vp, _vp, _vp, _sz]),
    "yscv_cuda_packed_int4_gemv": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "yscv_cuda_packed_int4_gemm": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz]),
    "yscv_cuda_pack_int4_symmetric_per_group": (C.c_int, [_vp, _vp, _sz, _sz, _sz, _vp, _vp]),
    "yscv_cuda_int4_weight_upload": (C.c_int, [_vp, _vp, _vp, _sz, _sz, _sz, C.POINTER(_vp)]),
    "yscv_cuda_int4_weight_wrap": (C.c_int, [_vp, _vp, _sz, _sz, _sz, C.POINTER(_vp)]),
    "yscv_cuda_int4_weight_free": (None, [_vp]),
    "yscv_cuda_int4_matmul_dev": (C.c_int, [_vp, _vp, _vp, _vp, _sz]),
    "yscv_cuda_int4_matmul_act_dev": (C.c_int, [_vp, _vp, _vp, _vp, _sz]),
    "yscv_cuda_pack_int4_dev": (C.c_int, [_vp, _vp, _sz, _sz, _sz, _vp, _vp]),
    "yscv_cuda_int4_matmul_dev_static": (C.c_int, [_vp, _vp, _vp, _sz, _sz, _sz, _vp, _vp, _sz]),
    "yscv_cuda_int8_matmul": (C.c_int, [_vp, _vp, _vp, _sz, _sz, _sz, _vp]),
    "yscv_cuda_pack_i8_b_for_matmul": (C.c_int, [_vp, _vp, _sz, _sz, C.POINTER(_vp)]),
    "yscv_cuda_pack_i8_b_dev": (C.c_int, [_vp, _vp, _sz, _sz, C.POINTER(_vp)]),
    "yscv_cuda_i8b_free": (None, [_vp]),
    "yscv_cuda_i8b_k": (_sz, [_vp]),
    "yscv_cuda_i8b_n": (_sz, [_vp]),
    "yscv_cuda_int8_matmul_prepacked": (C.c_int, [_vp, _vp, _vp, _sz, _vp]),
    "yscv_cuda_int8_matmul_prepacked_dev": (C.c_int, [_vp, _vp, _vp, _sz, _vp]),
    "yscv_cuda_qlinear_matmul": (C.c_int, [_vp, _vp, _vp, _sz, _vp, _vp]),
    "yscv_cuda_qlinear_matmul_dev": (C.c_int, [_vp, _vp, _vp, _sz, _vp, _vp]),
    "yscv_cuda_matmul_integer": (C.c_int, [_vp, _vp, C.c_int, C.c_int32, _vp, _sz, _vp]),
    "yscv_cuda_matmul_integer_dev": (C.c_int, [_vp, _vp, C.c_int, C.c_int32, _vp, _sz, _vp]),
    "yscv_cuda_embedding_dev": (C.c_int, [_vp, _vp, _sz, _sz, _vp, _sz, _vp]),
    "yscv_cuda_add_rms_norm_dev": (C.c_int, [_vp, _vp, _vp, _vp, C.c_float, _sz, _sz, _vp, _vp]),
    "yscv_cuda_add_rms_norm_act_dev": (C.c_int, [_vp, _vp, _vp, _vp, C.c_float, _sz, _sz, _vp, _vp]),
    "yscv_cuda_rope_kv_append_dev": (C.c_int, [_vp, _vp, _sz, _sz, _sz, _sz, _sz, C.c_float, _vp, _vp, _vp, _sz]),
    "yscv_cuda_gqa_attention_dev": (C.c_int, [_vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp, _sz, _vp, C.c_int, _vp]),
    "yscv_cuda_swiglu_dev": (C.c_int, [_vp, _vp, _sz, _sz, _vp]),
    "yscv_cuda_swiglu_act_dev": (C.c_int, [_vp, _vp, _sz, _sz, _vp]),
    "yscv_cuda_f32_matmul_dev": (C.c_int, [_vp, _vp, _vp, _sz, _sz, _sz, _vp]),
    "yscv_cuda_argmax_last_dev": (C.c_int, [_vp, _vp, _sz, _sz, _vp]),
    "yscv_cuda_advance_pos_dev": (C.c_int, [_vp, _vp, C.c_int]),
    "yscv_cuda_i8b_set_zero_point": (C.c_int, [_vp, C.c_int32]),
    "yscv_cuda_int4_from_matmulnbits": (C.c_int, [_vp, _vp, _sz]),
    "yscv_cuda_int4_from_matmulnbits_dev": (C.c_int, [_vp, _vp, _vp, _sz]),
    "yscv_cuda_int8_matmul_requant_per_channel_dev": (C.c_int, [_vp, _vp, _vp, _sz, _vp, _vp, C.c_float, _vp]),
    "yscv_cuda_int8_matmul_requant_per_channel": (C.c_int, [_vp, _vp, _vp, _sz, _vp, _vp, C.c_float, _vp]),
    "yscv_cuda_int8_matmul_requant_i8_dev": (C.c_int, [_vp, _vp, _vp, _sz, _vp, C.c_float, C.c_float, C.c_int, _vp]),
    "yscv_cuda_int8_matmul_requant_i8": (C.c_int, [_vp, _vp, _vp, _sz, _vp, C.c_float, C.c_float, C.c_int, _vp]),
    "yscv_cuda_decode_plan_create": (C.c_int, [_vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz, C.c_float, C.c_float,
                                               C.POINTER(_vp)]),
    "yscv_cuda_decode_plan_step_dev": (C.c_int, [_vp, _vp, _vp, _sz, _vp, _vp, _vp]),
    "yscv_cuda_decode_plan_step_token_dev": (C.c_int, [_vp, _vp, _vp, _sz, _vp, _vp, _vp, _vp, _vp, _vp]),
    "yscv_cuda_decode_plan_free": (None, [_vp]),
    "yscv_cuda_decode_plan_create_ex": (C.c_int, [_vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz, C.c_float, C.c_float,
                                                  _vp, C.POINTER(_vp)]),
    "yscv_cuda_decode_plan_check": (C.c_int, [_vp, _vp]),
    "yscv_cuda_decode_plan_step_token_shard_dev": (C.c_int, [_vp, _vp, _vp, _sz, _vp, _vp, _vp, _vp, _sz, _sz, _vp,
                                                             _vp]),
    "yscv_cuda_tp_comm_create": (C.c_int, [_vp, C.c_int, C.c_int, _sz, C.POINTER(_vp), _vp]),
    "yscv_cuda_tp_comm_connect": (C.c_int, [_vp, _vp]),
    "yscv_cuda_tp_comm_connect_unanswered": (C.c_int, [_vp]),
    "yscv_cuda_tp_comm_destroy": (None, [_vp]),
    "yscv_cuda_dispatch_report": (C.c_char_p, [_vp]),
    "yscv_cuda_quant_stats_read": (None, [_vp]),
    "yscv_cuda_quant_stats_reset": (None, []),
    "yscv_cuda_int4_to_matmulnbits": (C.c_int, [_vp, _vp, _sz]),
    "yscv_cuda_int4_weight_from_f32": (C.c_int, [_vp, _vp, _sz, _sz, C.c_int, _sz, C.POINTER(_vp)]),
    "yscv_cuda_int4_weight_rows": (_sz, [_vp]),
    "yscv_cuda_int4_weight_k": (_sz, [_vp]),
    "yscv_cuda_int4_weight_group_size": (_sz, [_vp]),
    "yscv_cuda_int4_weight_download": (C.c_int, [_vp, _vp, _vp, _vp]),
    "yscv_cuda_int4_container_size": (_sz, [_sz, _sz, _sz]),
    "yscv_cuda_int4_container_write": (C.c_int, [_vp, _vp, _sz, _sz, _sz, _vp, _sz, C.POINTER(_sz)]),
    "yscv_cuda_int4_container_read": (C.c_int, [_vp, _sz, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz),
                                                C.POINTER(_vp), C.POINTER(_vp)]),
    "yscv_cuda_int4_weight_from_container": (C.c_int, [_vp, _vp, _sz, C.POINTER(_vp)]),
    "yscv_cuda_requant_i32_row_to_i8": (C.c_int, [_vp, _vp, _vp, C.c_float, C.c_float, C.c_int, _vp, _sz, _sz]),
    "yscv_cuda_requant_i32_row_to_i8_dev": (C.c_int, [_vp, _vp, _vp, C.c_float, C.c_float, C.c_int, _vp, _sz, _sz]),
    "yscv_cuda_registry_create": (C.c_int, [C.POINTER(_vp)]),
    "yscv_cuda_registry_destroy": (None, [_vp]),
    "yscv_cuda_registry_put_int4": (C.c_int, [_vp, C.c_char_p, _vp]),
    "yscv_cuda_registry_put_i8b": (C.c_int, [_vp, C.c_char_p, _vp]),
    "yscv_cuda_registry_get_int4": (_vp, [_vp, C.c_char_p]),
    "yscv_cuda_registry_get_i8b": (_vp, [_vp, C.c_char_p]),
    "yscv_cuda_registry_len": (_sz, [_vp]),
    "yscv_cuda_registry_register_matmul_weight": (C.c_int, [_vp, _vp, C.c_char_p, _vp, _sz, _sz, C.c_int, _sz,
                                                            C.POINTER(C.c_int)]),
    "yscv_cuda_registry_register_i8_weight": (C.c_int, [_vp, _vp, C.c_char_p, _vp, _sz, _sz, C.POINTER(C.c_int)]),
    "yscv_cuda_should_prepack_i8_b": (C.c_int, [_sz, _sz]),
    "yscv_cuda_should_use_prepacked_i8_b": (C.c_int, [_sz, _sz, _sz]),
    "yscv_cuda_rope_kv_append_i8_dev": (C.c_int, [_vp, _vp, _sz, _sz, _sz, _sz, _sz, C.c_float, _vp, _vp, _vp, _vp,
                                                  _vp, _sz]),
    "yscv_cuda_gqa_attention_i8_dev": (C.c_int, [_vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp, _vp, _vp, _sz, _vp,
                                                 C.c_int, _vp]),
}

WEIGHT_MATMUL_KN, WEIGHT_GEMM_NK, WEIGHT_GEMM_KN = 0, 1, 2
TP_HANDLE_BYTES = 64


class Requant(C.Structure):
    """yscv_cuda_requant."""
    _fields_ = [("a_is_unsigned", C.c_int), ("a_zero_point", C.c_int32), ("composite", C.c_float),
                ("y_zero_point", C.c_float), ("qmin", C.c_int32), ("qmax", C.c_int32),
                ("round_mode", C.c_int)]


class QuantStats(C.Structure):
    """yscv_cuda_quant_stats."""
    _fields_ = [(n, C.c_uint64) for n in ("int4_gemv_calls", "int4_gemm_calls", "int4_generic_calls",
                                          "int8_gemm_calls", "qlinear_matmul_calls", "matmul_integer_calls",
                                          "requant_calls", "decode_step_calls", "cpu_fallbacks")]


class DecodeOptions(C.Structure):
    """yscv_cuda_decode_options."""
    _fields_ = [("variant", C.c_int), ("max_tiles", C.c_int), ("k_chunk", C.c_int), ("attention_form", C.c_int),
                ("spin_limit", C.c_int), ("tp", _vp), ("kv_int8", C.c_int), ("batch", C.c_int)]


class DecodeLayer(C.Structure):
    """yscv_cuda_decode_layer."""
    _fields_ = [("qkv", _vp), ("o", _vp), ("gate_up", _vp), ("down", _vp), ("d_gamma_attn", _vp),
                ("d_gamma_mlp", _vp), ("d_kcache", _vp), ("d_vcache", _vp), ("d_kscale", _vp), ("d_vscale", _vp)]


def load_library():
    """dlopen libyscv_cuda.so and attach the prototypes. Raises if it is missing."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not path.exists():
        raise FileNotFoundError(
            f"{path} is missing: build it with `python -m yscv_b200.build` "
            "(there is no CPU fallback)")
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


def _check(rc: int):
    if rc != 0:
        raise YscvCudaError(rc, load_library().yscv_cuda_last_error().decode())


def _host(a: np.ndarray, dtype) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def _ptr(a) -> int:
    """Address of a numpy array's data, or a raw device pointer passed as int."""
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    return int(a)


class Int4Weight:
    """PackedInt4Weight resident in HBM (owning or wrapping device memory)."""

    borrowed = False  # a view of a handle a Registry owns

    def __init__(self, handle: int, m_w: int, k: int, group_size: int):
        self.handle = handle
        self.m_w, self.k, self.group_size = m_w, k, group_size

    def free(self):
        if self.handle and not self.borrowed:
            load_library().yscv_cuda_int4_weight_free(self.handle)
        self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class I8B:
    """PackedI8B resident in HBM."""

    borrowed = False  # a view of a handle a Registry owns

    def __init__(self, handle: int):
        self.handle = handle
        lib = load_library()
        self.k = int(lib.yscv_cuda_i8b_k(handle))
        self.n = int(lib.yscv_cuda_i8b_n(handle))

    def set_zero_point(self, b_zp: int):
        """b_zero_point of MatMulInteger / QLinearMatMul for this weight (default 0)."""
        _check(load_library().yscv_cuda_i8b_set_zero_point(self.handle, int(b_zp)))

    def free(self):
        if self.handle and not self.borrowed:
            load_library().yscv_cuda_i8b_free(self.handle)
        self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def int4_from_matmulnbits(src) -> np.ndarray:
    """MatMulNBits bytes (unsigned nibbles, zero point 8) -> two's-complement nibbles; host only."""
    a = _host(src, np.uint8)
    out = np.empty_like(a)
    _check(load_library().yscv_cuda_int4_from_matmulnbits(_ptr(a), _ptr(out), a.size))
    return out


def quant_stats() -> dict:
    """Process-wide operator counters since the last reset."""
    st = QuantStats()
    load_library().yscv_cuda_quant_stats_read(C.byref(st))
    return {n: int(getattr(st, n)) for n, _ in QuantStats._fields_}


def quant_stats_reset():
    load_library().yscv_cuda_quant_stats_reset()


def int4_to_matmulnbits(src) -> np.ndarray:
    """Two's-complement nibbles -> MatMulNBits bytes (unsigned nibbles, zero point 8); host only."""
    a = _host(src, np.uint8)
    out = np.empty_like(a)
    _check(load_library().yscv_cuda_int4_to_matmulnbits(_ptr(a), _ptr(out), a.size))
    return out


def int4_container_write(packed, scales, m_w: int, k: int, group_size: int) -> bytes:
    """Serialise one packed int4 weight (header + packed bytes + scales)."""
    lib = load_library()
    p8, sc = _host(packed, np.uint8), _host(scales, np.float32)
    size = int(lib.yscv_cuda_int4_container_size(m_w, k, group_size))
    buf = np.empty(max(size, 64), dtype=np.uint8)
    written = _sz(0)
    _check(lib.yscv_cuda_int4_container_write(_ptr(p8), _ptr(sc), m_w, k, group_size, _ptr(buf), buf.size,
                                              C.byref(written)))
    return buf[:written.value].tobytes()


def int4_container_read(blob: bytes):
    """-> (packed uint8 [m_w*k/2], scales f32, m_w, k, group_size); validates the header."""
    lib = load_library()
    src = np.frombuffer(blob, dtype=np.uint8)
    m_w, k, g = _sz(0), _sz(0), _sz(0)
    pp, sp = _vp(), _vp()
    _check(lib.yscv_cuda_int4_container_read(_ptr(src) if src.size else None, src.size, C.byref(m_w), C.byref(k),
                                             C.byref(g), C.byref(pp), C.byref(sp)))
    base = src.ctypes.data
    p_off, s_off = pp.value - base, sp.value - base
    n_p, n_s = m_w.value * k.value // 2, m_w.value * (k.value // g.value)
    packed = src[p_off:p_off + n_p].copy()
    scales = np.frombuffer(blob, dtype=np.float32, count=n_s, offset=s_off).copy()
    return packed, scales, m_w.value, k.value, g.value


class Registry:
    """yscv_cuda_registry: resident weights keyed by initializer name."""

    def __init__(self):
        self.lib = load_library()
        h = _vp()
        _check(self.lib.yscv_cuda_registry_create(C.byref(h)))
        self.handle = h.value

    def put_int4(self, name: str, w: "Int4Weight"):
        """The table takes the handle over (the wrapper no longer frees it)."""
        _check(self.lib.yscv_cuda_registry_put_int4(self.handle, name.encode(), w.handle))
        w.handle = 0

    def put_i8b(self, name: str, b: "I8B"):
        _check(self.lib.yscv_cuda_registry_put_i8b(self.handle, name.encode(), b.handle))
        b.handle = 0

    def get_int4(self, name: str):
        """A borrowed Int4Weight view (never freed by the wrapper), or None."""
        h = self.lib.yscv_cuda_registry_get_int4(self.handle, name.encode())
        if not h:
            return None
        w = Int4Weight(h, int(self.lib.yscv_cuda_int4_weight_rows(h)), int(self.lib.yscv_cuda_int4_weight_k(h)),
                       int(self.lib.yscv_cuda_int4_weight_group_size(h)))
        w.borrowed = True
        return w

    def get_i8b(self, name: str):
        h = self.lib.yscv_cuda_registry_get_i8b(self.handle, name.encode())
        if not h:
            return None
        b = I8B(h)
        b.borrowed = True
        return b

    def register_matmul_weight(self, ctx: "Context", name: str, weight, layout: int, group_size: int) -> bool:
        """One weight of quantize_matmul_weights_int4_packed; False when the rules skip it."""
        w = _host(weight, np.float32)
        assert w.ndim == 2
        packed = C.c_int(0)
        _check(self.lib.yscv_cuda_registry_register_matmul_weight(ctx.handle, self.handle, name.encode(), _ptr(w),
                                                                  w.shape[0], w.shape[1], layout, group_size,
                                                                  C.byref(packed)))
        return bool(packed.value)

    def register_i8_weight(self, ctx: "Context", name: str, b) -> bool:
        """Load-time prepack of a QLinearMatMul / MatMulInteger weight b [k][n]; False when the gate says no."""
        b8 = _host(b, np.int8)
        done = C.c_int(0)
        _check(self.lib.yscv_cuda_registry_register_i8_weight(ctx.handle, self.handle, name.encode(), _ptr(b8),
                                                              b8.shape[0], b8.shape[1], C.byref(done)))
        return bool(done.value)

    def __len__(self):
        return int(self.lib.yscv_cuda_registry_len(self.handle))

    def close(self):
        if self.handle:
            self.lib.yscv_cuda_registry_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class TpComm:
    """yscv_cuda_tp_comm: this rank's exchange region and the peers' mapped ones."""

    def __init__(self, ctx: "Context", rank: int, world: int, max_rows: int):
        self.lib, self.rank, self.world = ctx.lib, rank, world
        h = _vp()
        self.handle_bytes = np.zeros(TP_HANDLE_BYTES, dtype=np.uint8)
        _check(self.lib.yscv_cuda_tp_comm_create(ctx.handle, rank, world, max_rows, C.byref(h),
                                                 _ptr(self.handle_bytes)))
        self.handle = h.value

    def connect(self, all_handles: np.ndarray):
        """all_handles: uint8 [world, 64], every rank's handle in rank order."""
        a = _host(all_handles, np.uint8)
        assert a.size == self.world * TP_HANDLE_BYTES
        _check(self.lib.yscv_cuda_tp_comm_connect(self.handle, _ptr(a)))

    def connect_unanswered(self):
        """Test form: peers that never answer (every wait for them runs out)."""
        _check(self.lib.yscv_cuda_tp_comm_connect_unanswered(self.handle))

    def close(self):
        if self.handle:
            self.lib.yscv_cuda_tp_comm_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DecodePlan:
    """yscv_cuda_decode_plan: one launch per single-token decode step (batch 1)."""

    def __init__(self, ctx: "Context", handle: int):
        self.ctx, self.handle = ctx, handle

    def step_dev(self, d_embedding: int, vocab: int, d_token: int, d_pos: int, d_x: int):
        _check(self.ctx.lib.yscv_cuda_decode_plan_step_dev(self.ctx.handle, self.handle, _vp(d_embedding), vocab,
                                                           _vp(d_token), _vp(d_pos), _vp(d_x)))

    def step_token_dev(self, d_embedding: int, vocab: int, d_token: int, d_pos: int, d_final_gamma: int,
                       d_lm_head: int, d_x: int, d_logits: int):
        """The step plus final norm, fp32 LM head, greedy token into *d_token and *d_pos += 1."""
        _check(self.ctx.lib.yscv_cuda_decode_plan_step_token_dev(
            self.ctx.handle, self.handle, _vp(d_embedding), vocab, _vp(d_token), _vp(d_pos), _vp(d_final_gamma),
            _vp(d_lm_head), _vp(d_x), _vp(d_logits)))

    def step_token_shard_dev(self, d_embedding: int, vocab: int, d_token: int, d_pos: int, d_final_gamma: int,
                             d_lm_head_rows: int, lm_row0: int, lm_rows: int, d_x: int, d_logits: int):
        """Tensor-parallel form: this rank's rows of the LM head, the token agreed between the ranks."""
        _check(self.ctx.lib.yscv_cuda_decode_plan_step_token_shard_dev(
            self.ctx.handle, self.handle, _vp(d_embedding), vocab, _vp(d_token), _vp(d_pos), _vp(d_final_gamma),
            _vp(d_lm_head_rows), lm_row0, lm_rows, _vp(d_x), _vp(d_logits)))

    def check(self):
        """Synchronises; raises YscvCudaError(-4) if a bounded wait ran out in a step of this plan."""
        _check(self.ctx.lib.yscv_cuda_decode_plan_check(self.ctx.handle, self.handle))

    def free(self):
        if self.handle:
            self.ctx.lib.yscv_cuda_decode_plan_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Context:
    """One CUDA stream on one sm_100 device (yscv_cuda_ctx)."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self.lib = load_library()
        h = _vp()
        if stream is None:
            _check(self.lib.yscv_cuda_ctx_create(device, C.byref(h)))
        else:
            _check(self.lib.yscv_cuda_ctx_create_on_stream(device, _vp(stream), C.byref(h)))
        self.handle = h.value
        self.device = device
        self.prefill_exact = False   # mirrors yscv_cuda_ctx_set_int4_prefill_exact

    def close(self):
        if getattr(self, "handle", None):
            self.lib.yscv_cuda_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- bookkeeping -------------------------------------------------------
    def synchronize(self):
        _check(self.lib.yscv_cuda_ctx_synchronize(self.handle))

    def device_status(self) -> int:
        s = C.c_int(0)
        _check(self.lib.yscv_cuda_ctx_device_status(self.handle, C.byref(s)))
        return s.value

    def last_kernel(self) -> str:
        return self.lib.yscv_cuda_last_kernel(self.handle).decode()

    def launch_count(self) -> int:
        return int(self.lib.yscv_cuda_ctx_launch_count(self.handle))

    def set_int4_prefill_exact(self, exact: bool):
        """m > 16 int4 matmuls: fp32-exact kernel (True) or bf16 tensor-core GEMM (False, default)."""
        _check(self.lib.yscv_cuda_ctx_set_int4_prefill_exact(self.handle, int(exact)))
        self.prefill_exact = bool(exact)

    def set_int4_prefill_cta_pairs(self, on: bool):
        """bf16 prefill GEMM: allow the CTA-pair kernel (cta_group::2) for large prefills (default) or not."""
        _check(self.lib.yscv_cuda_ctx_set_int4_prefill_cta_pairs(self.handle, int(bool(on))))

    def set_int8_cta_pairs(self, on):
        """int8 GEMM: None = the CTA-pair kernel (cta_group::2) where it measured faster (default),
        False = the one-CTA kernel everywhere, True = the pair kernel on every shape it supports."""
        _check(self.lib.yscv_cuda_ctx_set_int8_cta_pairs(self.handle, -1 if on is None else int(bool(on))))

    def set_f32_tensor_cores(self, on: bool):
        """fp32 matmul with more than 8 rows: the 3xTF32 tensor-core kernel (default) or the tiled FMA kernel."""
        _check(self.lib.yscv_cuda_ctx_set_f32_tensor_cores(self.handle, int(bool(on))))

    def set_attention_tensor_cores(self, on: bool):
        """Decode attention over int8 caches: fp16 tensor-core kernel (default) or the fp32 loop."""
        _check(self.lib.yscv_cuda_ctx_set_attention_tensor_cores(self.handle, int(on)))

    def set_int8_tail_split(self, on: bool):
        """int8 GEMM: cut the K loops of the tiles beyond the last full wave over all CTAs (default) or not."""
        _check(self.lib.yscv_cuda_ctx_set_int8_tail_split(self.handle, int(on)))

    def profile_enable(self, on: bool):
        _check(self.lib.yscv_cuda_ctx_profile_enable(self.handle, int(on)))

    def profile_read(self):
        """(bracketed launches, summed device ms) since the last read."""
        n, ms = C.c_uint64(0), C.c_double(0.0)
        _check(self.lib.yscv_cuda_ctx_profile_read(self.handle, C.byref(n), C.byref(ms)))
        return int(n.value), float(ms.value)

    # -- int4, host drop-ins -------------------------------------------------
    def packed_int4_gemv(self, weight_packed, scales, activation, m_w, k, group_size):
        wp, sc, act = _host(weight_packed, np.uint8), _host(scales, np.float32), _host(activation, np.float32)
        out = np.empty(m_w, dtype=np.float32)
        _check(self.lib.yscv_cuda_packed_int4_gemv(self.handle, _ptr(wp), _ptr(sc), _ptr(act),
                                                   _ptr(out), m_w, k, group_size))
        return out

    def packed_int4_gemm(self, weight_packed, scales, activation, m, n, k, group_size):
        wp, sc, act = _host(weight_packed, np.uint8), _host(scales, np.float32), _host(activation, np.float32)
        out = np.empty((m, n), dtype=np.float32)
        _check(self.lib.yscv_cuda_packed_int4_gemm(self.handle, _ptr(wp), _ptr(sc), _ptr(act),
                                                   _ptr(out), m, n, k, group_size))
        return out

    def pack_int4_symmetric_per_group(self, weights, m_w, k, group_size):
        w = _host(weights, np.float32)
        packed = np.empty(m_w * k // 2, dtype=np.uint8)
        scales = np.empty(m_w * (k // max(group_size, 1)), dtype=np.float32)
        _check(self.lib.yscv_cuda_pack_int4_symmetric_per_group(
            self.handle, _ptr(w), m_w, k, group_size, _ptr(packed), _ptr(scales)))
        return packed, scales

    # -- int4, device-resident ------------------------------------------------
    def int4_weight_upload(self, packed, scales, m_w, k, group_size) -> Int4Weight:
        wp, sc = _host(packed, np.uint8), _host(scales, np.float32)
        h = _vp()
        _check(self.lib.yscv_cuda_int4_weight_upload(self.handle, _ptr(wp), _ptr(sc), m_w, k,
                                                     group_size, C.byref(h)))
        return Int4Weight(h.value, m_w, k, group_size)

    def int4_weight_wrap(self, d_packed: int, d_scales: int, m_w, k, group_size) -> Int4Weight:
        h = _vp()
        _check(self.lib.yscv_cuda_int4_weight_wrap(_vp(d_packed), _vp(d_scales), m_w, k,
                                                   group_size, C.byref(h)))
        return Int4Weight(h.value, m_w, k, group_size)

    def int4_matmul_dev(self, w: Int4Weight, d_activation: int, d_output: int, m: int):
        _check(self.lib.yscv_cuda_int4_matmul_dev(self.handle, w.handle, _vp(d_activation),
                                                  _vp(d_output), m))

    def int4_matmul_act_dev(self, w: Int4Weight, d_activation_bf16: int, d_output: int, m: int):
        """int4_matmul_dev for m > 16 on activations already in the tensor-core GEMM's bf16 form."""
        _check(self.lib.yscv_cuda_int4_matmul_act_dev(self.handle, w.handle, _vp(d_activation_bf16),
                                                      _vp(d_output), m))

    def int4_matmul(self, w: Int4Weight, activation, m: int, out=None):
        """Resident weights, host activation [m,k] -> host output [m,n]."""
        act = _host(activation, np.float32)
        if out is None:
            out = np.empty((m, w.m_w), dtype=np.float32)
        _check(self.lib.yscv_cuda_int4_matmul(self.handle, w.handle, _ptr(act), _ptr(out), m))
        return out

    # -- int8 -------------------------------------------------------------------
    def int8_matmul(self, a, b, m, k, n):
        a8, b8 = _host(a, np.int8), _host(b, np.int8)
        out = np.empty((m, n), dtype=np.int32)
        _check(self.lib.yscv_cuda_int8_matmul(self.handle, _ptr(a8), _ptr(b8), m, k, n, _ptr(out)))
        return out

    def pack_i8_b(self, b, k, n) -> "I8B":
        b8 = _host(b, np.int8)
        h = _vp()
        _check(self.lib.yscv_cuda_pack_i8_b_for_matmul(self.handle, _ptr(b8), k, n, C.byref(h)))
        return I8B(h.value)

    def pack_i8_b_dev(self, d_b: int, k, n) -> "I8B":
        h = _vp()
        _check(self.lib.yscv_cuda_pack_i8_b_dev(self.handle, _vp(d_b), k, n, C.byref(h)))
        return I8B(h.value)

    def int8_matmul_prepacked(self, a, b: "I8B", m):
        a8 = _host(a, np.int8)
        out = np.empty((m, b.n), dtype=np.int32)
        _check(self.lib.yscv_cuda_int8_matmul_prepacked(self.handle, _ptr(a8), b.handle, m, _ptr(out)))
        return out

    def int8_matmul_prepacked_dev(self, d_a: int, b: "I8B", m, d_out: int):
        _check(self.lib.yscv_cuda_int8_matmul_prepacked_dev(self.handle, _vp(d_a), b.handle, m, _vp(d_out)))

    @staticmethod
    def requant(composite, y_zp, qmin, qmax, a_unsigned=False, a_zp=0, round_mode=0) -> "Requant":
        return Requant(int(a_unsigned), int(a_zp), float(composite), float(y_zp), int(qmin), int(qmax),
                       int(round_mode))

    def qlinear_matmul(self, a, b: "I8B", m, rq: "Requant"):
        """a: uint8 or int8 [m,k] host; returns uint8 (qmin >= 0) or int8 [m,n]."""
        a = np.ascontiguousarray(a)
        assert a.dtype in (np.uint8, np.int8)
        out = np.empty((m, b.n), dtype=np.uint8 if rq.qmin >= 0 else np.int8)
        _check(self.lib.yscv_cuda_qlinear_matmul(self.handle, _ptr(a), b.handle, m, C.byref(rq), _ptr(out)))
        return out

    def qlinear_matmul_dev(self, d_a: int, b: "I8B", m, rq: "Requant", d_out: int):
        _check(self.lib.yscv_cuda_qlinear_matmul_dev(self.handle, _vp(d_a), b.handle, m, C.byref(rq), _vp(d_out)))

    def int8_matmul_requant_per_channel(self, a, b: "I8B", m, corr, composite, y_zp):
        """i8 A [m,k] host -> i8 [m,n]; corr int32 [n], composite f32 [n]."""
        a8, cr, cp = _host(a, np.int8), _host(corr, np.int32), _host(composite, np.float32)
        out = np.empty((m, b.n), dtype=np.int8)
        _check(self.lib.yscv_cuda_int8_matmul_requant_per_channel(self.handle, _ptr(a8), b.handle, m, _ptr(cr),
                                                                   _ptr(cp), y_zp, _ptr(out)))
        return out

    def int8_matmul_requant_per_channel_dev(self, d_a: int, b: "I8B", m, d_corr: int, d_composite: int, y_zp,
                                            d_out: int):
        _check(self.lib.yscv_cuda_int8_matmul_requant_per_channel_dev(self.handle, _vp(d_a), b.handle, m,
                                                                       _vp(d_corr), _vp(d_composite), y_zp,
                                                                       _vp(d_out)))

    def int8_matmul_requant_i8(self, a, b: "I8B", m, bias, composite, y_zp, relu=False):
        a8 = _host(a, np.int8)
        bs = None if bias is None else _host(bias, np.int32)
        out = np.empty((m, b.n), dtype=np.int8)
        _check(self.lib.yscv_cuda_int8_matmul_requant_i8(self.handle, _ptr(a8), b.handle, m,
                                                          None if bs is None else _ptr(bs), composite, y_zp,
                                                          int(relu), _ptr(out)))
        return out

    def int8_matmul_requant_i8_dev(self, d_a: int, b: "I8B", m, d_bias, composite, y_zp, relu, d_out: int):
        _check(self.lib.yscv_cuda_int8_matmul_requant_i8_dev(self.handle, _vp(d_a), b.handle, m, _vp(d_bias or 0),
                                                              composite, y_zp, int(relu), _vp(d_out)))

    def matmul_integer(self, a, b: "I8B", m, a_zp=0):
        a = np.ascontiguousarray(a)
        assert a.dtype in (np.uint8, np.int8)
        out = np.empty((m, b.n), dtype=np.int32)
        _check(self.lib.yscv_cuda_matmul_integer(self.handle, _ptr(a), int(a.dtype == np.uint8), a_zp,
                                                 b.handle, m, _ptr(out)))
        return out

    def matmul_integer_dev(self, d_a: int, a_unsigned: bool, a_zp: int, b: "I8B", m, d_out: int):
        _check(self.lib.yscv_cuda_matmul_integer_dev(self.handle, _vp(d_a), int(a_unsigned), a_zp, b.handle,
                                                     m, _vp(d_out)))

    def int4_matmul_dev_static(self, d_packed: int, d_scales: int, n, k, group_size,
                               d_activation: int, d_output: int, m: int):
        """Allocation-free variant: scratch is an array built into the library."""
        _check(self.lib.yscv_cuda_int4_matmul_dev_static(
            self.handle, _vp(d_packed), _vp(d_scales), n, k, group_size, _vp(d_activation),
            _vp(d_output), m))

    # -- decoder operators (device pointers) ----------------------------------------
    def embedding_dev(self, d_weight, vocab, dim, d_tokens, rows, d_out):
        _check(self.lib.yscv_cuda_embedding_dev(self.handle, _vp(d_weight), vocab, dim, _vp(d_tokens), rows, _vp(d_out)))

    def add_rms_norm_dev(self, d_x, d_delta, d_gamma, eps, rows, hidden, d_x_out, d_normed):
        _check(self.lib.yscv_cuda_add_rms_norm_dev(self.handle, _vp(d_x), _vp(d_delta or 0), _vp(d_gamma), eps,
                                                   rows, hidden, _vp(d_x_out or 0), _vp(d_normed)))

    def add_rms_norm_act_dev(self, d_x, d_delta, d_gamma, eps, rows, hidden, d_x_out, d_normed_act):
        """add_rms_norm_dev with the normalised rows written as bf16 activations for int4_matmul_act_dev."""
        _check(self.lib.yscv_cuda_add_rms_norm_act_dev(self.handle, _vp(d_x), _vp(d_delta or 0), _vp(d_gamma), eps,
                                                       rows, hidden, _vp(d_x_out or 0), _vp(d_normed_act)))

    def rope_kv_append_dev(self, d_qkv, batch, seq, n_q, n_kv, d_head, theta, d_pos, d_kc, d_vc, max_seq):
        _check(self.lib.yscv_cuda_rope_kv_append_dev(self.handle, _vp(d_qkv), batch, seq, n_q, n_kv, d_head, theta,
                                                     _vp(d_pos), _vp(d_kc), _vp(d_vc), max_seq))

    def gqa_attention_dev(self, d_q, q_stride, batch, seq_q, n_q, n_kv, d_head, d_kc, d_vc, max_seq, d_pos,
                          causal, d_out):
        _check(self.lib.yscv_cuda_gqa_attention_dev(self.handle, _vp(d_q), q_stride, batch, seq_q, n_q, n_kv, d_head,
                                                    _vp(d_kc), _vp(d_vc), max_seq, _vp(d_pos), int(causal), _vp(d_out)))

    def swiglu_dev(self, d_gate_up, rows, inter, d_out):
        _check(self.lib.yscv_cuda_swiglu_dev(self.handle, _vp(d_gate_up), rows, inter, _vp(d_out)))

    def swiglu_act_dev(self, d_gate_up, rows, inter, d_out_act):
        """swiglu_dev with the result written as bf16 activations for int4_matmul_act_dev."""
        _check(self.lib.yscv_cuda_swiglu_act_dev(self.handle, _vp(d_gate_up), rows, inter, _vp(d_out_act)))

    def f32_matmul_dev(self, d_w, d_x, m, n, k, d_out):
        _check(self.lib.yscv_cuda_f32_matmul_dev(self.handle, _vp(d_w), _vp(d_x), m, n, k, _vp(d_out)))

    def argmax_last_dev(self, d_logits, rows, vocab, d_out):
        _check(self.lib.yscv_cuda_argmax_last_dev(self.handle, _vp(d_logits), rows, vocab, _vp(d_out)))

    def advance_pos_dev(self, d_pos, by=1):
        _check(self.lib.yscv_cuda_advance_pos_dev(self.handle, _vp(d_pos), by))

    def dispatch_report(self) -> str:
        return self.lib.yscv_cuda_dispatch_report(self.handle).decode()

    def int4_weight_from_f32(self, weight, layout: int, group_size: int):
        """fp32 MatMul / Gemm weight -> resident packed int4, or None when the reference's rules skip it."""
        w = _host(weight, np.float32)
        assert w.ndim == 2
        h = _vp()
        _check(self.lib.yscv_cuda_int4_weight_from_f32(self.handle, _ptr(w), w.shape[0], w.shape[1], layout,
                                                       group_size, C.byref(h)))
        if not h.value:
            return None
        return Int4Weight(h.value, int(self.lib.yscv_cuda_int4_weight_rows(h.value)),
                          int(self.lib.yscv_cuda_int4_weight_k(h.value)), group_size)

    def int4_weight_download(self, w: Int4Weight):
        packed = np.empty(w.m_w * w.k // 2, dtype=np.uint8)
        scales = np.empty(w.m_w * (w.k // w.group_size), dtype=np.float32)
        _check(self.lib.yscv_cuda_int4_weight_download(self.handle, w.handle, _ptr(packed), _ptr(scales)))
        return packed, scales

    def int4_weight_from_container(self, blob: bytes) -> Int4Weight:
        src = np.frombuffer(blob, dtype=np.uint8)
        h = _vp()
        _check(self.lib.yscv_cuda_int4_weight_from_container(self.handle, _ptr(src) if src.size else None, src.size,
                                                             C.byref(h)))
        return Int4Weight(h.value, int(self.lib.yscv_cuda_int4_weight_rows(h.value)),
                          int(self.lib.yscv_cuda_int4_weight_k(h.value)),
                          int(self.lib.yscv_cuda_int4_weight_group_size(h.value)))

    def requant_i32_row_to_i8(self, acc, bias, composite, y_zp, relu, c):
        a = _host(acc, np.int32)
        b = None if bias is None else _host(bias, np.int32)
        out = np.empty(a.size, dtype=np.int8)
        _check(self.lib.yscv_cuda_requant_i32_row_to_i8(self.handle, _ptr(a) if a.size else None,
                                                         None if b is None else _ptr(b), composite, y_zp, int(relu),
                                                         _ptr(out) if a.size else None, a.size, c))
        return out

    def rope_kv_append_i8_dev(self, d_qkv, batch, seq, n_q, n_kv, d_head, theta, d_pos, d_kc, d_ks, d_vc, d_vs, max_seq):
        _check(self.lib.yscv_cuda_rope_kv_append_i8_dev(self.handle, _vp(d_qkv), batch, seq, n_q, n_kv, d_head, theta,
                                                        _vp(d_pos), _vp(d_kc), _vp(d_ks), _vp(d_vc), _vp(d_vs), max_seq))

    def gqa_attention_i8_dev(self, d_q, q_stride, batch, seq_q, n_q, n_kv, d_head, d_kc, d_ks, d_vc, d_vs, max_seq,
                             d_pos, causal, d_out):
        _check(self.lib.yscv_cuda_gqa_attention_i8_dev(self.handle, _vp(d_q), q_stride, batch, seq_q, n_q, n_kv, d_head,
                                                       _vp(d_kc), _vp(d_ks), _vp(d_vc), _vp(d_vs), max_seq, _vp(d_pos),
                                                       int(causal), _vp(d_out)))

    def decode_plan(self, layers, hidden, inter, n_q, n_kv, d_head, max_seq, eps, rope_theta, *, variant=-1,
                    max_tiles=0, k_chunk=0, attention_form=-1, spin_limit=0, tp: "TpComm | None" = None,
                    kv_int8=False, batch=1) -> DecodePlan:
        """layers: list of dicts with Int4Weight `qkv`, `o`, `gate_up`, `down` and device
        pointers `gamma_attn`, `gamma_mlp`, `kcache`, `vcache` (with kv_int8 also `kscale`,
        `vscale`). The keyword arguments are the fields of yscv_cuda_decode_options (defaults: the
        library's own choices)."""
        arr = (DecodeLayer * len(layers))()
        for dst, l in zip(arr, layers):
            dst.qkv, dst.o, dst.gate_up, dst.down = (l["qkv"].handle, l["o"].handle, l["gate_up"].handle,
                                                     l["down"].handle)
            dst.d_gamma_attn, dst.d_gamma_mlp = l["gamma_attn"], l["gamma_mlp"]
            dst.d_kcache, dst.d_vcache = l["kcache"], l["vcache"]
            dst.d_kscale, dst.d_vscale = l.get("kscale"), l.get("vscale")
        h = _vp()
        opt = DecodeOptions(variant, max_tiles, k_chunk, attention_form, spin_limit, tp.handle if tp else None,
                            1 if kv_int8 else 0, int(batch))
        _check(self.lib.yscv_cuda_decode_plan_create_ex(self.handle, C.cast(arr, _vp), len(layers), hidden, inter,
                                                        n_q, n_kv, d_head, max_seq, eps, rope_theta,
                                                        C.cast(C.byref(opt), _vp), C.byref(h)))
        return DecodePlan(self, h.value)

    def int4_from_matmulnbits_dev(self, d_src: int, d_dst: int, nbytes: int):
        _check(self.lib.yscv_cuda_int4_from_matmulnbits_dev(self.handle, _vp(d_src), _vp(d_dst), nbytes))

    def pack_int4_dev(self, d_weights: int, m_w, k, group_size, d_packed: int, d_scales: int):
        _check(self.lib.yscv_cuda_pack_int4_dev(self.handle, _vp(d_weights), m_w, k, group_size,
                                                _vp(d_packed), _vp(d_scales)))
