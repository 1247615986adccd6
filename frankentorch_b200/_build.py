"""In-tree build of the native libraries.

Two shared objects are produced next to the sources (they are git-ignored build
artefacts):

* ``lib/libftk_sm100.so``  - the hand-written sm_100a CUDA kernels (plain C ABI,
  no PyTorch dependency), compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``.
* ``lib/libftcore.so``     - the host runtime in C++ (deterministic autograd tape,
  evidence ledger, dispatch key resolution, FNV fingerprints, FTSV codec, PRNGs).

``nvcc`` cross-compiles without a GPU, so the build also serves as the
"does it compile" check on a CPU-only machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC=/path/to/nvcc")


def _newer(src_list, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in src_list)


def _run(cmd):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), proc.stdout, proc.stderr))
    return proc.stdout + proc.stderr


def kernel_sources():
    return sorted(CSRC.glob("*.cu"))


def core_sources():
    return sorted((CSRC / "core").glob("*.cpp"))


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libftk_sm100.so``."""
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    out = LIB / "libftk_sm100.so"
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    srcs = kernel_sources()
    nvcc = _nvcc()
    jobs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if force or _newer([s] + headers, o):
            jobs.append([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(s), "-o", str(o)])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for log in ex.map(_run, jobs):
                if verbose and log.strip():
                    print(log)
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if force or jobs or _newer(objs, out):
        _run([nvcc, "-shared", "-o", str(out), *map(str, objs), "-lcudart"])
    return out


def build_core(force: bool = False) -> Path:
    """Compile the host runtime (``csrc/core/*.cpp``) into ``libftcore.so``."""
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    out = LIB / "libftcore.so"
    srcs = core_sources()
    headers = list((CSRC / "core").glob("*.h")) + list((CSRC / "core").glob("*.hpp"))
    if not srcs:
        return out
    if force or _newer(srcs + headers, out):
        cxx = os.environ.get("CXX", "g++")
        _run([cxx, *CXX_FLAGS, "-shared", "-o", str(out), *map(str, srcs), "-lpthread"])
    return out


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force, verbose), build_core(force)


if __name__ == "__main__":
    k, c = build_all(force="--force" in sys.argv, verbose=True)
    print("built", k, c)
