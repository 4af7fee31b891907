"""Builds libpitch_b200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m pitch_b200.build [--force] [-v]

The library is written for B200 only: one -gencode for compute_100a / sm_100a.
-fmad=false keeps every float operation a separate IEEE rounding (the codec's
codes are compared bit for bit with a CPU restatement); fused operations are
written explicitly where wanted.  Every ``csrc/abi_*.cu`` is one translation unit;
they are compiled side by side and only the stale ones are rebuilt.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
OBJ_DIR = LIB_DIR / "obj"
LIB = LIB_DIR / "libpitch_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "-fmad=false",
    "-Xcompiler", "-fPIC",
]


def sources():
    return sorted(CSRC.glob("*.cu"))


def _headers():
    return list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG.parent / "include" / "pitch_b200.h"]


def _obj(src: Path) -> Path:
    return OBJ_DIR / (src.stem + ".o")


def _stale_objects():
    newest_header = max(p.stat().st_mtime for p in _headers())
    out = []
    for src in sources():
        o = _obj(src)
        if not o.exists() or o.stat().st_mtime < max(src.stat().st_mtime, newest_header):
            out.append(src)
    return out


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in sources() + _headers())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    todo = sources() if force else _stale_objects()

    def compile_one(src: Path):
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(_obj(src))]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
            print(" ".join(cmd), file=sys.stderr)
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4) or 1) as pool:
        for src, r in pool.map(compile_one, todo):
            if verbose or r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode:
                raise subprocess.CalledProcessError(r.returncode, f"nvcc {src.name}")
    live = {_obj(s) for s in sources()}
    for o in OBJ_DIR.glob("*.o"):
        if o not in live:
            o.unlink()
    subprocess.run([nvcc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
                    "-o", str(LIB), *map(str, sorted(live))], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
