"""ctypes binding of ``libftcore.so``: the C++ host runtime (tape scheduler, ledger,
fingerprints, PRNGs, dispatch resolution, CPU reference kernels)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB = None
_PATH = Path(__file__).resolve().parent.parent / "lib" / "libftcore.so"


def load():
    global _LIB
    if _LIB is not None:
        return _LIB
    import os
    if os.environ.get("FT_NO_AUTOBUILD") != "1":
        from .. import _build
        _build.build_core()     # no-op when the library was built from the sources on disk
    lib = C.CDLL(str(_PATH))
    vp, i64, u64, i32, dbl = C.c_void_p, C.c_int64, C.c_uint64, C.c_int, C.c_double
    P = C.POINTER
    sig = {
        "ftc_tape_new": ([], vp), "ftc_tape_free": ([vp], None), "ftc_tape_len": ([vp], i64),
        "ftc_tape_add_node": ([vp, P(i64), i32, i32, i32], i64),
        "ftc_tape_set_requires_grad": ([vp, i64, i32], i32),
        "ftc_tape_truncate": ([vp, i64], i64), "ftc_tape_mark_consumed": ([vp], None),
        "ftc_tape_is_consumed": ([vp, i64], i32),
        "ftc_tape_schedule": ([vp, i64, i32, P(i64), P(i64), P(i64)], i64),
        "ftc_ledger_new": ([i64], vp), "ftc_ledger_free": ([vp], None),
        "ftc_ledger_record": ([vp, i32, C.c_char_p, i64], i64), "ftc_ledger_len": ([vp], i64),
        "ftc_ledger_total": ([vp], i64),
        "ftc_ledger_get": ([vp, i64, P(i64), P(i32), C.c_char_p, i64], i64),
        "ftc_ledger_clear": ([vp], None),
        "ftc_fnv1a64": ([C.c_char_p, i64, u64], u64),
        "ftc_xoshiro_seed": ([P(u64), u64], None), "ftc_xoshiro_next_u64": ([P(u64)], u64),
        "ftc_xoshiro_fill_uniform": ([P(u64), vp, i64], None),
        "ftc_xoshiro_fill_normal": ([P(u64), vp, i64], None),
        "ftc_lcg_next": ([P(u64)], u64), "ftc_lcg_shuffle": ([P(u64), vp, i64], None),
        "ftc_dispatch_resolve": ([u64, i32, P(i32)], i32),
        "ftc_pairwise_sum": ([vp, i64], dbl),
        "ftc_linear_f64": ([vp, vp, vp, vp, i64, i64, i64], None),
        "ftc_linear_backward_f64": ([vp, vp, vp, vp, vp, vp, i64, i64, i64], None),
        "ftc_layer_norm_f64": ([vp, vp, vp, vp, vp, vp, i64, i64, dbl], None),
        "ftc_cross_entropy_f64": ([vp, vp, vp, vp, vp, i64, i64], None),
        "ftc_sdpa_f64": ([vp, vp, vp, vp, i64, i64, i64, dbl, i32], None),
        "ftc_adamw_f64": ([vp, vp, vp, vp, i64, dbl, dbl, dbl, dbl, dbl, i64], None),
        "ftc_gelu_tanh_clamped_f32": ([vp, vp, i64], None),
        "ftc_softmax_guarded_f32": ([vp, vp, i64, i64], None),
        "ftc_pool_configure": ([C.c_char_p, P(i32)], i32), "ftc_pool_width": ([], i32),
        "ftc_pool_physical_cores": ([], i32), "ftc_pool_auto_width": ([], i32),
        "ftc_pool_reset_for_tests": ([], None), "ftc_pool_set_min_work": ([i64], i64),
        "ftc_pool_set_target_workers": ([C.c_int], C.c_int), "ftc_pool_target_workers": ([], C.c_int),
        "ftc_pairwise_sum_par": ([vp, i64], dbl),
        "ftc_linear_f64_par": ([vp, vp, vp, vp, i64, i64, i64], None),
        "ftc_layer_norm_f64_par": ([vp, vp, vp, vp, i64, i64, dbl], None),
        "ftc_adamw_f64_par": ([vp, vp, vp, vp, i64, dbl, dbl, dbl, dbl, dbl, i64], None),
        "ftc_set_sdpa_br": ([i32], i32), "ftc_get_sdpa_br": ([], i32), "ftc_sdpa_br_for": ([i64, i64], i32),
        "ftc_sdpa_f64_blocked": ([vp, vp, vp, vp, i64, i64, i64, i64, dbl, i32], None),
    }
    for name, (args, res) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = res
    _LIB = lib
    return lib


def fnv1a64(data: bytes, seed: int = 0) -> int:
    return int(load().ftc_fnv1a64(data, len(data), seed))
