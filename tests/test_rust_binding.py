"""The Rust sys crate under bindings/rust is generated from include/yscv_cuda.h: the committed
file must be what the generator produces from the current header, and must declare every
function the header does. CPU only (no Rust toolchain is needed or used)."""
import importlib.util
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _gen():
    spec = importlib.util.spec_from_file_location("gen_sys", ROOT / "bindings" / "rust" / "gen_sys.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_sys_crate_is_generated_from_the_header():
    gen = _gen()
    assert gen.OUT.read_text() == gen.generate(), "run `python bindings/rust/gen_sys.py`"


def test_sys_crate_declares_every_header_function():
    gen = _gen()
    text = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / "yscv_cuda.h").read_text(), flags=re.S)
    declared = set(re.findall(r"\b(yscv_cuda_[a-z0-9_]+)\s*\(", text))
    rust = set(re.findall(r"pub fn (yscv_cuda_[a-z0-9_]+)\(", gen.OUT.read_text()))
    assert declared == rust, (declared - rust, rust - declared)


def test_wrappers_only_call_declared_functions():
    gen = _gen()
    rust = set(re.findall(r"pub fn (yscv_cuda_[a-z0-9_]+)\(", gen.OUT.read_text()))
    consts = set(re.findall(r"pub const (YSCV_CUDA_[A-Z0-9_]+)", gen.OUT.read_text()))
    for rel in ("yscv-kernels-cuda/src/lib.rs",):
        src = (ROOT / "bindings" / "rust" / rel).read_text()
        used = set(re.findall(r"sys::(yscv_cuda_[a-z0-9_]+)\s*\(", src))
        assert used <= rust, used - rust
        assert set(re.findall(r"sys::(YSCV_CUDA_[A-Z0-9_]+)", src)) <= consts
