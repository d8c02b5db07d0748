"""The C headers of the two libraries say what the sources export: every exported function is declared with the
signature it is defined with, and nothing else is declared."""

from __future__ import annotations

import re
import shutil
import subprocess
from pathlib import Path

import pytest

CSRC = Path(__file__).resolve().parent.parent / "litinfer_b200" / "csrc"


def exported(files, macro):
    """name -> signature (whitespace squeezed) of every definition marked with the export macro."""
    out = {}
    for f in files:
        for m in re.finditer(re.escape(macro) + r"\s+([^;{]*?\))\s*\{", f.read_text(), re.S):
            sig = " ".join(m.group(1).split())
            out[re.match(r".*?(\w+)\(", sig).group(1)] = sig
    return out


def declared(header):
    text = re.sub(r"/\*.*?\*/", lambda m: m.group(0) if m.group(0).startswith("/* R_real") else "", header.read_text(), flags=re.S)
    out = {}
    for m in re.finditer(r"^([\w \*]+?\b(li_\w+)\([^;]*\));", text, re.S | re.M):
        out[m.group(2)] = " ".join(m.group(1).split())
    return out


@pytest.mark.parametrize("header,sources,macro", [
    ("litinfer_b200.h", "*.cu", "LI_EXPORT"),
    ("host/litinfer_host.h", "host/*.cpp", "LI_HOST_EXPORT"),
])
def test_header_declares_what_the_sources_export(header, sources, macro):
    have = exported(sorted(CSRC.glob(sources)), macro)
    want = declared(CSRC / header)
    assert sorted(have) == sorted(want), f"only in the sources: {sorted(set(have) - set(want))}; only in the header: {sorted(set(want) - set(have))}"
    for name, sig in have.items():
        assert want[name] == sig, f"{name}: defined as\n  {sig}\ndeclared as\n  {want[name]}"


def test_the_host_library_has_every_declared_function():
    from litinfer_b200.cache import native

    lib = native.library()
    for name in declared(CSRC / "host" / "litinfer_host.h"):
        assert hasattr(lib, name), name


def test_headers_compile(tmp_path):
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        pytest.skip("no C++ compiler")
    (tmp_path / "h.cpp").write_text('#include "host/litinfer_host.h"\nint main() { return li_pool_num_free(nullptr) * 0; }\n')
    r = subprocess.run([cxx, "-std=c++17", "-fsyntax-only", "-I", str(CSRC), str(tmp_path / "h.cpp")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    (tmp_path / "h.c").write_text('#include "host/litinfer_host.h"\nint f(void) { return LI_HOST_OK; }\n')
    r = subprocess.run([shutil.which("gcc") or cxx, "-fsyntax-only", "-I", str(CSRC), str(tmp_path / "h.c")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    nvcc = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if Path("/usr/local/cuda/bin/nvcc").is_file() else None)
    if nvcc is None:
        pytest.skip("no nvcc: the kernel library's header needs cuda_runtime.h")
    (tmp_path / "k.cu").write_text('#include "litinfer_b200.h"\n#include "no_alloc.h"\nint main() { return li_tcgen05_status(); }\n')
    r = subprocess.run([nvcc, "-std=c++17", "-I", str(CSRC), "-c", str(tmp_path / "k.cu"), "-o", str(tmp_path / "k.o")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
