"""The C-ABI library loads and exports every symbol include/yscv_cuda.h declares.
CPU only: no compute call is made."""
import ctypes
import re
from pathlib import Path

import yscv_b200
from yscv_b200 import lib as binding

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "yscv_cuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(yscv_cuda_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert "yscv_cuda_packed_int4_gemv" in names and len(names) >= 10


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(yscv_b200.library_path()))
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_binding_covers_header_exactly():
    assert sorted(binding.SIGNATURES) == declared_functions()
    yscv_b200.load_library()


def test_matmulnbits_nibbles_become_twos_complement(oracle):
    # (q_u - 8) for every unsigned nibble pair equals the sign-extended nibbles of byte ^ 0x88
    import numpy as np
    src = np.arange(256, dtype=np.uint8)
    got = yscv_b200.int4_from_matmulnbits(src)
    assert np.array_equal(got, src ^ 0x88)
    for u, s in zip(src.tolist(), got.tolist()):
        assert oracle.lib.yo_unpack_low(s) == (u & 15) - 8
        assert oracle.lib.yo_unpack_high(s) == (u >> 4) - 8


def test_no_fallback_without_device():
    # On a machine without a B200 the library must refuse, not compute on the CPU.
    import torch
    if torch.cuda.is_available():
        return
    try:
        yscv_b200.Context(0)
    except yscv_b200.YscvCudaError as e:
        assert e.status in (-5, -2)
    else:
        raise AssertionError("context creation succeeded without a GPU")


def test_product_does_not_import_oracle():
    for p in (ROOT / "yscv_b200").rglob("*"):
        if p.suffix in {".py", ".cu", ".cuh", ".cpp", ".hpp", ".h"}:
            text = p.read_text()
            assert "oracle" not in text.lower() or p.name == "__none__", f"{p} mentions the oracle"
