"""Builds LitInfer, unmodified, for the reference arm of bench.py.

LitInfer's own build needs xmake, which this image does not have, so `pip install` of it yields its Python layer only
(``baseline/_ref/llaisys``, git-ignored).  Its native library is plain C++17 with OpenMP and AVX2; this script compiles
every .cpp / .cc under its ``src/`` with g++, with the flags of its xmake files (xmake/cpu.lua:43-58 for the two AVX
files), into ``baseline/_ref/llaisys/libllaisys/libllaisys.so``, where its Python layer looks for it.  Nothing of
LitInfer is changed, and nothing of this repository's engine is involved.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_PKG = HERE / "_ref" / "llaisys"
LIB = REF_PKG / "libllaisys" / "libllaisys.so"
DEFAULT_SOURCE = Path(os.environ.get("LITINFER_SOURCE", "/root/reference"))


def have_library() -> bool:
    return LIB.is_file()


def build(source: Path = DEFAULT_SOURCE, verbose: bool = True) -> Path:
    """Compile the reference's native library beside its installed Python layer; returns the library's path."""
    if have_library():
        return LIB
    cxx = shutil.which("g++")
    if cxx is None:
        raise RuntimeError("g++ not found: LitInfer's native library cannot be built")
    source = Path(source)
    if not (source / "src").is_dir():
        raise RuntimeError(f"LitInfer's sources not found at {source}")
    if not REF_PKG.is_dir():
        # the Python layer as pip would install it from python/ (the project root has no setup.py / pyproject.toml)
        shutil.copytree(source / "python" / "llaisys", REF_PKG)
        for p in REF_PKG.rglob("*"):
            os.chmod(p, 0o755 if p.is_dir() else 0o644)
    files = sorted(list((source / "src").rglob("*.cpp")) + list((source / "src").rglob("*.cc")))
    with tempfile.TemporaryDirectory() as tmp:
        def compile_one(job):
            i, f = job
            extra = []
            # `-include immintrin.h` first: include/llaisys.h defines __C, which GCC's intrinsics headers use as a parameter name
            if f.name == "linear_cpu_avx.cpp":
                extra = ["-include", "immintrin.h", "-mavx2", "-mfma", "-mf16c", "-DLLAISYS_COMPILE_AVX_LINEAR"]
            elif f.name == "quantize_cpu_avx.cpp":
                extra = ["-include", "immintrin.h", "-mavx2", "-mfma", "-mf16c", "-DLLAISYS_COMPILE_AVX_QUANT"]
            o = Path(tmp) / f"{i}.o"
            r = subprocess.run([cxx, "-std=c++17", "-O3", "-fPIC", "-fopenmp", "-Wno-unknown-pragmas", f"-I{source / 'include'}",
                                f"-I{source / 'src'}", *extra, "-c", str(f), "-o", str(o)], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"g++ failed on {f}:\n{r.stderr[-2000:]}")
            return str(o)

        if verbose:
            print(f"[reference] compiling {len(files)} files of LitInfer with g++", file=sys.stderr, flush=True)
        with ThreadPoolExecutor(max_workers=min(len(files), os.cpu_count() or 4)) as ex:
            objs = list(ex.map(compile_one, enumerate(files)))
        LIB.parent.mkdir(parents=True, exist_ok=True)
        tmp_lib = LIB.with_suffix(f".{os.getpid()}.tmp")
        r = subprocess.run([cxx, "-shared", "-fopenmp", "-o", str(tmp_lib), *objs], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking LitInfer failed:\n{r.stderr[-2000:]}")
        os.replace(tmp_lib, LIB)
    if verbose:
        print(f"[reference] built {LIB}", file=sys.stderr, flush=True)
    return LIB


if __name__ == "__main__":
    print(build())
