

def test_debug_bounds_variant_compiles(tmp_path):
    """The guarded-index debug build (-DFT_DEBUG_BOUNDS) of a kernel file that uses FT_IDX compiles for sm_100a."""
    import shutil
    import subprocess

    from frankentorch_b200 import _build
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    src = _build.CSRC / "elementwise.cu"
    assert "FT_IDX(" in src.read_text()
    out = tmp_path / "elementwise_dbg.o"
    flags = [f for f in _build.NVCC_FLAGS if f != "-DFT_DEBUG_BOUNDS"]
    p = subprocess.run([nvcc, *flags, "-DFT_DEBUG_BOUNDS", "-I", str(_build.CSRC), "-c", str(src), "-o", str(out)],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and out.exists(), p.stderr[-2000:]
