"""Builds libyscv_cuda.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Usage: ``python -m yscv_b200.build`` (cross-compiles without a GPU).
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libyscv_cuda.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-diag-suppress", "177",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    deps = sources() + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.hpp")) + \
        sorted((PKG_DIR.parent / "include").glob("*.h"))
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    # one object per source file, compiled side by side (no device symbol crosses a file), then
    # one link step; the objects live in a scratch directory outside the tree
    import tempfile
    from concurrent.futures import ThreadPoolExecutor
    objdir = Path(tempfile.gettempdir()) / "yscv_b200_obj"
    objdir.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.hpp")) + sorted((PKG_DIR.parent / "include").glob("*.h"))
    newest_header = max((p.stat().st_mtime for p in headers), default=0.0)

    def compile_one(src: Path):
        obj = objdir / (src.stem + ".o")
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, newest_header):
            return obj, None
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        return obj, subprocess.run(cmd, capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, sources()))
    failed = False
    for obj, proc in results:
        if proc is None:
            continue
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            failed = True
        elif verbose:
            sys.stderr.write(proc.stderr)
    if failed:
        raise RuntimeError("nvcc failed building libyscv_cuda.so")
    link = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC",
            "-o", str(LIB_PATH), *[str(o) for o, _ in results]]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("nvcc failed linking libyscv_cuda.so")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
