"""ctypes binding of ``libftk_sm100.so`` (the hand-written sm_100a kernels).

The library is built in-tree by :mod:`frankentorch_b200._build`.  On a machine
with a GPU a missing library is a hard error: the CUDA path is the only path, a
silent PyTorch fallback would hide a broken build.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libftk_sm100.so"


class KernelLibraryMissing(RuntimeError):
    pass


class FtkGemmDesc(C.Structure):
    _fields_ = [
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("L0", C.c_int), ("L1", C.c_int),
        ("a_mn", C.c_int), ("b_mn", C.c_int),
        ("A", C.c_void_p), ("lda", C.c_longlong), ("a_s0", C.c_longlong), ("a_s1", C.c_longlong),
        ("B", C.c_void_p), ("ldb", C.c_longlong), ("b_s0", C.c_longlong), ("b_s1", C.c_longlong),
        ("D", C.c_void_p), ("ldd", C.c_longlong), ("d_s0", C.c_longlong), ("d_s1", C.c_longlong),
        ("bias", C.c_void_p),
        ("resid", C.c_void_p), ("ldr", C.c_longlong), ("r_s0", C.c_longlong), ("r_s1", C.c_longlong),
        ("aux", C.c_void_p),
        ("alpha", C.c_float), ("epi", C.c_int), ("out_fp32", C.c_int), ("accumulate", C.c_int),
        ("force_bn", C.c_int), ("max_ctas", C.c_int),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_longlong), ("split_k", C.c_int),
        ("reduce_stream", C.c_void_p),
        ("seg_counts", C.c_void_p), ("seg_rows", C.c_int),
    ]


class FtkAttnDesc(C.Structure):
    _fields_ = [
        ("B", C.c_int), ("H", C.c_int), ("S", C.c_int), ("hd", C.c_int), ("causal", C.c_int),
        ("scale", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_bs", C.c_longlong), ("q_ss", C.c_longlong), ("q_hs", C.c_longlong),
        ("k_bs", C.c_longlong), ("k_ss", C.c_longlong), ("k_hs", C.c_longlong),
        ("v_bs", C.c_longlong), ("v_ss", C.c_longlong), ("v_hs", C.c_longlong),
        ("o", C.c_void_p),
        ("o_bs", C.c_longlong), ("o_ss", C.c_longlong), ("o_hs", C.c_longlong),
        ("lse", C.c_void_p),
        ("d_o", C.c_void_p), ("delta", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
    ]


FTK_MAX_RANKS = 8
COMM_GATHER_A, COMM_GATHER_B, COMM_SCATTER_D = 1, 2, 3


class FtkCommDesc(C.Structure):
    _fields_ = [
        ("mode", C.c_int), ("rank", C.c_int), ("world", C.c_int), ("comm_ctas", C.c_int),
        ("chunk_rows", C.c_int),
        ("src", C.c_void_p * FTK_MAX_RANKS),
        ("sub_flags", C.c_void_p), ("ready_local", C.c_void_p),
        ("ready_peer", C.c_void_p * FTK_MAX_RANKS),
        ("inbox", C.c_void_p * FTK_MAX_RANKS),
        ("arrive", C.c_void_p * FTK_MAX_RANKS),
        ("epoch", C.c_void_p),
        ("push", C.c_int),
        ("full_peer", C.c_void_p * FTK_MAX_RANKS),
        ("flags_peer", C.c_void_p * FTK_MAX_RANKS),
    ]


class FtkMoeDesc(C.Structure):
    _fields_ = [
        ("T", C.c_int), ("d", C.c_int), ("E", C.c_int), ("capacity", C.c_int), ("rank", C.c_int),
        ("world", C.c_int),
        ("idx", C.c_void_p), ("slot", C.c_void_p), ("counts", C.c_void_p), ("ticket", C.c_void_p),
        ("epoch", C.c_void_p),
    ]


def lib_path() -> Path:
    return _LIB_PATH


def load(build_if_missing: bool = True):
    """Return the loaded kernel library, building it first if it is absent."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if build_if_missing and os.environ.get("FT_NO_AUTOBUILD") != "1":
        # also rebuilds a library that was built from other sources than the ones on disk
        from .. import _build
        _build.build_kernels()
    if not _LIB_PATH.exists():
        raise KernelLibraryMissing(
            f"{_LIB_PATH} is missing; run `python -m frankentorch_b200._build` "
            "(the sm_100a kernels are the only GPU backend, there is no fallback)")
    lib = C.CDLL(str(_LIB_PATH))
    lib.ftk_status_word.restype = C.c_void_p
    lib.ftk_read_status.argtypes = [C.c_int]
    lib.ftk_gemm_bf16.argtypes = [C.POINTER(FtkGemmDesc), C.c_void_p]
    lib.ftk_gemm_plan.argtypes = [C.POINTER(FtkGemmDesc), C.POINTER(C.c_int), C.POINTER(C.c_int)]
    lib.ftk_gemm_plan.restype = C.c_int
    lib.ftk_gemm_group_bf16.argtypes = [C.POINTER(FtkGemmDesc), C.c_int, C.c_void_p]
    lib.ftk_gemm_group_bf16.restype = C.c_int
    lib.ftk_gemm_comm_bf16.argtypes = [C.POINTER(FtkGemmDesc), C.POINTER(FtkCommDesc), C.c_void_p]
    lib.ftk_tick_i32.argtypes = [C.c_void_p, C.c_void_p]
    lib.ftk_set_flags_sys.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    lib.ftk_copy_async.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]
    lib.ftk_set_flags_sys.restype = lib.ftk_copy_async.restype = C.c_int
    lib.ftk_attn_fwd.argtypes = [C.POINTER(FtkAttnDesc), C.c_void_p]
    lib.ftk_attn_bwd.argtypes = [C.POINTER(FtkAttnDesc), C.c_void_p]
    vp, i, f, ll, ull = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_ulonglong
    pm, pv = C.POINTER(FtkMoeDesc), C.POINTER(C.c_void_p)
    sigs = {
        "ftk_moe_route": [vp, vp, vp, vp, i, i, i, vp],
        "ftk_moe_route_bwd": [vp, vp, vp, vp, i, i, i, vp],
        "ftk_moe_gate_grad": [vp, vp, vp, i, i, vp],
        "ftk_moe_slots": [vp, vp, vp, i, i, i, vp],
        "ftk_moe_dispatch": [pm, vp, vp, pv, pv, pv, vp],
        "ftk_moe_combine": [pm, pv, pv, vp, vp, vp, vp, vp],
        "ftk_layernorm_fwd": [vp, vp, vp, vp, vp, vp, vp, vp, i, i, f, vp],
        "ftk_layernorm_bwd_blocks": [i],
        "ftk_layernorm_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, vp],
        "ftk_rmsnorm_fwd": [vp, vp, vp, vp, i, i, f, vp],
        "ftk_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, vp, i, i, i, vp],
        "ftk_softmax_rows": [vp, vp, i, i, i, vp],
        "ftk_softmax_causal_bf16": [vp, vp, i, i, f, vp],
        "ftk_softmax_bwd_bf16": [vp, vp, vp, ll, i, f, vp],
        "ftk_cross_entropy_fwd_bwd": [vp, vp, vp, vp, i, i, i, f, vp],
        "ftk_reduce_mean_f32": [vp, vp, ll, f, vp],
        "ftk_sumsq_f32": [vp, vp, vp, ll, i, vp],
        "ftk_gelu_fwd": [vp, vp, ll, i, vp],
        "ftk_gelu_bwd": [vp, vp, vp, ll, i, vp],
        "ftk_add_bf16": [vp, vp, vp, ll, vp],
        "ftk_cast_f32_to_bf16": [vp, vp, ll, vp],
        "ftk_cast_bf16_to_f32": [vp, vp, ll, i, vp],
        "ftk_dropout_bf16": [vp, vp, ll, f, ull, ull, vp],
        "ftk_colsum_bf16": [vp, vp, vp, i, i, ll, i, vp],
        "ftk_colsum_blocks": [i],
        "ftk_embedding_fwd": [vp, vp, vp, vp, i, i, i, ll, vp],
        "ftk_embedding_bwd": [vp, vp, vp, vp, vp, i, i, i, ll, vp],
        "ftk_embedding_bwd_scan": [vp, vp, vp, vp, i, i, i, ll, vp],
        "ftk_adamw": [vp, vp, vp, vp, vp, ll, f, f, f, f, f, f, f, f, vp],
        "ftk_adamw_tick": [vp, vp, C.c_double, C.c_double, vp],
        "ftk_clip_scale": [vp, f, vp, vp, vp],
        "ftk_adamw_dev": [vp, vp, vp, vp, vp, ll, vp, f, f, f, f, vp],
        "ftk_fill_f32": [vp, ll, f, vp],
        "ftk_timestamp": [vp, vp],
        "ftk_present_rgba8": [vp, vp, i, i, ll, i, vp],
        "ftk_im2col_1d": [vp, vp, i, i, i, i, i, i, vp],
        "ftk_wait_probe": [vp, i, ll, vp, vp],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_int
    _LIB = lib
    return lib


def is_loaded() -> bool:
    return _LIB is not None
