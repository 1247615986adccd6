"""In-tree build of the native libraries.

Two shared objects are produced next to the sources (they are git-ignored build
artefacts, together with ``lib/build_manifest.json``, which records the sha256 of the
sources and flags each one was built from; a library is rebuilt when that differs from
what is on disk now, whatever the modification times say):

* ``lib/libftk_sm100.so``  - the hand-written sm_100a CUDA kernels (plain C ABI,
  no PyTorch dependency), compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``.
* ``lib/libftcore.so``     - the host runtime in C++ (deterministic autograd tape,
  evidence ledger, dispatch key resolution, FNV fingerprints, FTSV codec, PRNGs).

``nvcc`` cross-compiles without a GPU, so the build also serves as the
"does it compile" check on a CPU-only machine.
"""
from __future__ import annotations

import fcntl
import hashlib
import json
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
# FT_BUILD_DEBUG_BOUNDS=1: a debug build in which the kernels' FT_IDX() index guards are compiled in (an index
# outside its range is reported through the status word and replaced by 0 instead of being dereferenced).  The
# flags are part of the build manifest, so switching the variable rebuilds the library.
if os.environ.get("FT_BUILD_DEBUG_BOUNDS", "0") == "1":
    NVCC_FLAGS.append("-DFT_DEBUG_BOUNDS")
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC=/path/to/nvcc")


def _digest(paths, extra=()) -> str:
    """sha256 over the contents of ``paths`` (in sorted order) and the strings in ``extra``."""
    h = hashlib.sha256()
    for x in extra:
        h.update(str(x).encode())
        h.update(b"\0")
    for p in sorted(map(str, paths)):
        h.update(os.path.basename(p).encode())
        h.update(b"\0")
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _manifest() -> dict:
    try:
        return json.loads((LIB / "build_manifest.json").read_text())
    except Exception:
        return {}


def _save_manifest(m: dict) -> None:
    (LIB / "build_manifest.json").write_text(json.dumps(m, indent=1, sort_keys=True))


def _stale(key: str, digest: str, target: Path, manifest: dict) -> bool:
    """A target is rebuilt when it is missing or was built from different source bytes or flags.

    Modification times are not consulted: a binary that is newer than its sources but was built
    from other sources (a checkout, a copied tree) would otherwise be used as is.
    """
    return (not target.exists()) or manifest.get(key) != digest


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
    man = _manifest()
    digests = {(s.stem + ".o"): _digest([s] + headers, NVCC_FLAGS) for s in srcs}
    so_digest = _digest([], sorted(digests.values()))
    if not force and not _stale(out.name, so_digest, out, man):
        return out          # the library on disk was built from exactly these sources and flags
    with _Lock():
        return _build_kernels_locked(force, verbose, out, srcs, nvcc, digests, so_digest)


def _build_kernels_locked(force, verbose, out, srcs, nvcc, digests, so_digest) -> Path:
    man = _manifest()
    if not force and not _stale(out.name, so_digest, out, man):
        return out          # another process built it while this one waited for the lock
    jobs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if force or _stale(o.name, digests[o.name], o, man):
            jobs.append([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(s), "-o", str(o)])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for log in ex.map(_run, jobs):
                if verbose and log.strip():
                    print(log)
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    _run([nvcc, "-shared", "-o", str(out), *map(str, objs), "-lcudart"])
    man = _manifest()
    man.update(digests)
    man[out.name] = so_digest
    _save_manifest(man)
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
    man = _manifest()
    d = _digest(srcs + headers, CXX_FLAGS)
    if force or _stale(out.name, d, out, man):
        with _Lock():
            if force or _stale(out.name, d, out, _manifest()):
                cxx = os.environ.get("CXX", "g++")
                _run([cxx, *CXX_FLAGS, "-shared", "-o", str(out), *map(str, srcs), "-lpthread"])
                man = _manifest()
                man[out.name] = d
                _save_manifest(man)
    return out


def is_current() -> bool:
    """True when both libraries exist and were built from the sources now on disk."""
    man = _manifest()
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    ds = sorted(_digest([s] + headers, NVCC_FLAGS) for s in kernel_sources())
    k_ok = (LIB / "libftk_sm100.so").exists() and man.get("libftk_sm100.so") == _digest([], ds)
    ch = list((CSRC / "core").glob("*.h")) + list((CSRC / "core").glob("*.hpp"))
    c_ok = (LIB / "libftcore.so").exists() and man.get("libftcore.so") == _digest(core_sources() + ch, CXX_FLAGS)
    return k_ok and c_ok


class _Lock:
    """Inter-process lock: the ranks of one job may all find a stale library at import time."""

    def __enter__(self):
        LIB.mkdir(exist_ok=True)
        self.f = open(LIB / ".build.lock", "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force, verbose), build_core(force)


if __name__ == "__main__":
    k, c = build_all(force="--force" in sys.argv, verbose=True)
    print("built", k, c)
