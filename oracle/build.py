"""Builds the checker: the C restatement (liboracle.so, next to this file) and — only where the reference tree is
mounted — the reference's own CPU silicon family, compiled from its sources where they lie, into oracle/_ref/.

TEST INFRASTRUCTURE.  The reference family is built with the reference's own recipe for it (one translation unit that
includes silicon_families/x86_avx2/unit.cuh; g++ -O3 -mavx2 -mfma -mf16c, engine/scripts/build_silicon_families.sh:
196-201 of that tree); no reference source is copied anywhere.  oracle/_ref/ is git-ignored and still travels to a GPU
box with the rest of the working tree, where the reference tree itself does not exist.

build_engine() compiles the reference's engine (evaluator, boot, C interface and Python module) the same way, from its
one translation unit engine/src/manifest.cu with the command its own build script uses (scripts/build.sh:25-26 of that
tree), into oracle/_ref/ as the Python module silvann_engine_cpu.  It is there for one job: to load THIS repository's
family into the unmodified engine and run the nn verbs through it (tests/test_engine_dropin.py).
"""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
PORT = HERE / "liboracle.so"
REF_DIR = HERE / "_ref"
REF = REF_DIR / "libsilvann_x86_avx2.so"
# where the reference tree is mounted: SILVANN_REFERENCE, else a directory named "reference" beside this repository's own
REFERENCE_TREE = Path(os.environ.get("SILVANN_REFERENCE") or HERE.parent.parent / "reference")


def build_port(force: bool = False) -> Path:
    src = HERE / "silvann_oracle.c"
    if force or not PORT.exists() or PORT.stat().st_mtime < src.stat().st_mtime:
        cmd = ["gcc", "-O2", "-mavx2", "-mfma", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", str(src), "-lm", "-o", str(PORT)]
        subprocess.run(cmd, check=True)
    return PORT


def build_reference(force: bool = False) -> Path | None:
    """The reference CPU family, or None when its sources are not on this machine and no earlier build is present."""
    unit = REFERENCE_TREE / "engine" / "src" / "silicon_families" / "x86_avx2" / "unit.cuh"
    if not unit.exists():
        return REF if REF.exists() else None
    if REF.exists() and not force:
        return REF
    REF_DIR.mkdir(exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        tu = Path(tmp) / "x86_avx2.cpp"
        tu.write_text('#include "silicon_families/x86_avx2/unit.cuh"\n')
        cmd = ["g++", "-O3", "-mavx2", "-mfma", "-mf16c", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
               "-I", str(REFERENCE_TREE / "engine" / "src"), str(tu), "-lpthread", "-o", str(REF)]
        subprocess.run(cmd, check=True)
    return REF


REF_CUDA = REF_DIR / "libsilvann_nvidia_cuda12.so"


def build_reference_cuda(force: bool = False) -> Path | None:
    """The reference's own CUDA family for sm_100 — the same-card baseline the B200 family is measured beside — built
    with the reference's recipe for it (engine/scripts/build_silicon_families.sh:141-156 of that tree: one translation
    unit that includes silicon_families/nvidia_cuda12/unit.cuh; nvcc -O2 -std=c++17 -cudart static).  None when the
    sources are not on this machine and no earlier build is present."""
    unit = REFERENCE_TREE / "engine" / "src" / "silicon_families" / "nvidia_cuda12" / "unit.cuh"
    if not unit.exists():
        return REF_CUDA if REF_CUDA.exists() else None
    if REF_CUDA.exists() and not force:
        return REF_CUDA
    REF_DIR.mkdir(exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        tu = Path(tmp) / "nvidia_cuda12.cu"
        tu.write_text('#include "silicon_families/nvidia_cuda12/unit.cuh"\n')
        cmd = ["nvcc", "-gencode", "arch=compute_100,code=sm_100", "-O2", "-std=c++17", "-cudart", "static", "-w",
               "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared", "-I", str(REFERENCE_TREE / "engine" / "src"), str(tu), "-o", str(REF_CUDA)]
        subprocess.run(cmd, check=True)
    return REF_CUDA


def engine_path() -> Path:
    import sysconfig
    return REF_DIR / ("silvann_engine_cpu" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_engine(force: bool = False) -> Path | None:
    """The reference engine as a Python module, or None when its sources are not here and no earlier build is present."""
    import sysconfig
    out = engine_path()
    unit = REFERENCE_TREE / "engine" / "src" / "manifest.cu"
    if not unit.exists():
        return out if out.exists() else None
    if out.exists() and not force:
        return out
    import pybind11
    REF_DIR.mkdir(exist_ok=True)
    cmd = ["g++", "-x", "c++", "-O2", "-std=c++17", "-pthread", "-fPIC", "-shared", "-ftls-model=initial-exec", "-w",
           "-DSILVANN_MODULE_NAME=silvann_engine_cpu", "-I", str(REFERENCE_TREE / "engine" / "src"), "-I", pybind11.get_include(),
           "-I", sysconfig.get_path("include"), str(unit), "-o", str(out)]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    print(build_port(force="-f" in sys.argv))
    print(build_reference(force="-f" in sys.argv))
    print(build_engine(force="-f" in sys.argv))
    print(build_reference_cuda(force="-f" in sys.argv))
