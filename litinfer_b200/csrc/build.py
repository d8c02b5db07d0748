"""Builds the CUDA kernels of this package into one shared library with nvcc.

The sources are plain CUDA with a C interface (no torch headers), compiled for
sm_100a only, one object per ``.cu`` file in parallel, then linked.  The
library lands in ``csrc/_build/`` inside the package; if that is not writable,
in a per-user folder under the system's temporary directory.  It is rebuilt
when a source file, a header or the flags change (a hash of them is part of
the file name).  Nothing is compiled at import: the first kernel call, or
:func:`ensure_built`, does it and prints a line per file meanwhile.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Optional

CSRC = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fvisibility=hidden"]
LIB_STEM = "liblitinfer_b200"


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc not found (set NVCC or put it on PATH); the kernels cannot be built")


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dirs() -> List[Path]:
    dirs = [CSRC / "_build"]
    env = os.environ.get("LITINFER_B200_BUILD_DIR")
    if env:
        dirs.insert(0, Path(env))
    dirs.append(Path(tempfile.gettempdir()) / f"litinfer_b200_build_{os.getuid()}")
    return dirs


def library_path(must_exist: bool = True) -> Optional[Path]:
    name = f"{LIB_STEM}_{_fingerprint()}.so"
    for d in _build_dirs():
        if (d / name).is_file():
            return d / name
    return None if must_exist else _build_dirs()[0] / name


def _writable_dir() -> Path:
    for d in _build_dirs():
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".probe_{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return d
        except OSError:
            continue
    raise BuildError("no writable folder for the built kernels: tried " + ", ".join(str(d) for d in _build_dirs()))


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[litinfer_b200 build] {msg}", file=sys.stderr, flush=True)


def ensure_built(verbose: bool = True, extra_flags: Optional[List[str]] = None) -> Path:
    """Path of the up-to-date library, compiling it first if need be."""
    have = library_path()
    if have is not None and not extra_flags:
        return have
    nvcc = find_nvcc()
    out_dir = _writable_dir()
    name = f"{LIB_STEM}_{_fingerprint()}.so"
    target = out_dir / name
    obj_dir = out_dir / f"obj_{_fingerprint()}_{os.getpid()}"
    obj_dir.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    if not srcs:
        raise BuildError(f"no .cu sources in {CSRC}")
    t0 = time.time()
    _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first call only)", verbose)

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *(extra_flags or []), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        t = time.time()
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        if extra_flags and (r.stdout or r.stderr):
            _say(f"{src.name}:\n{r.stdout}{r.stderr}", True)
        _say(f"  {src.name} done in {time.time() - t:.1f} s", verbose)
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
            objs = list(ex.map(compile_one, srcs))
        tmp = out_dir / f".{name}.{os.getpid()}.tmp"
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *[str(o) for o in objs]]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, target)            # atomic: concurrent builders never see a half-written library
    finally:
        shutil.rmtree(obj_dir, ignore_errors=True)
    # older builds of other source versions are of no use any more
    for old in out_dir.glob(f"{LIB_STEM}_*.so"):
        if old != target:
            try:
                old.unlink()
            except OSError:
                pass
    _say(f"built {target.name} in {time.time() - t0:.1f} s", verbose)
    return target


# ---------------------------------------------------------------------------
# the host runtime (csrc/host/*.cpp): plain C++, built with g++ into a library of its own, so that the engine's
# bookkeeping also runs (and is tested) where there is neither a GPU nor nvcc
# ---------------------------------------------------------------------------

HOST_DIR = CSRC / "host"
HOST_STEM = "liblitinfer_host"
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall"]


def _host_fingerprint() -> str:
    h = hashlib.sha256()
    for f in sorted(list(HOST_DIR.glob("*.cpp")) + list(HOST_DIR.glob("*.h"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(HOST_FLAGS).encode())
    return h.hexdigest()[:16]


def ensure_host_built(verbose: bool = True) -> Path:
    """Path of the up-to-date host runtime library, compiling it first if need be (a second or two)."""
    name = f"{HOST_STEM}_{_host_fingerprint()}.so"
    for d in _build_dirs():
        if (d / name).is_file():
            return d / name
    cxx = next((c for c in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")) if c), None)
    if cxx is None:
        raise BuildError("no C++ compiler found (set CXX or install g++); the host runtime cannot be built")
    srcs = sorted(HOST_DIR.glob("*.cpp"))
    if not srcs:
        raise BuildError(f"no .cpp sources in {HOST_DIR}")
    out_dir = _writable_dir()
    target = out_dir / name
    tmp = out_dir / f".{name}.{os.getpid()}.tmp"
    _say(f"compiling the host runtime ({len(srcs)} C++ file{'s' if len(srcs) > 1 else ''}) into {out_dir}", verbose)
    r = subprocess.run([cxx, *HOST_FLAGS, "-I", str(HOST_DIR), *[str(s) for s in srcs], "-o", str(tmp)], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"{cxx} failed on the host runtime:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, target)
    for old in out_dir.glob(f"{HOST_STEM}_*.so"):
        if old != target:
            try:
                old.unlink()
            except OSError:
                pass
    return target


if __name__ == "__main__":
    print(ensure_host_built())
    print(ensure_built())
