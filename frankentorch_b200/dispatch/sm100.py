"""Kernel registry of the single GPU backend (sm_100a): which session operators run on a
hand-written kernel, and what the dispatcher does with the ones that have none.

``FrankenTorchSession(device="cuda")`` consults this table in its operator entry point
(the counterpart of the typed dispatch functions, ft-dispatch/src/lib.rs:4123, reached from
``Linear::forward`` at ft-nn/src/lib.rs:1067-1100):

* an operator with a route whose operands qualify (bf16, on the device, unit inner stride,
  extents compatible with 16-byte TMA rows) is executed by the fused kernels of
  :mod:`frankentorch_b200.ops.fused`; the dispatch decision written to the ledger carries the
  name of the kernel that was launched and, for GEMMs, its tile configuration
  (``ftk::gemm_bf16_sm100<128x192,splitK=1>``);
* layout operators (views and index bookkeeping) carry no arithmetic and are recorded as
  ``layout::<op>``;
* everything else has no sm_100a kernel.  Strict mode refuses it (``NoKernelForBackend``);
  hardened mode runs PyTorch's CUDA operator, marks the decision ``fallback_path=true`` with the
  kernel string ``torch::<op>`` and the deviation id ``dispatch.sm100_missing_kernel_fallback``,
  which must be listed in ``HARDENED_DEVIATION_ALLOWLIST_V1.json`` (next to this file's package,
  under ``conformance/``) like every other strict/hardened difference
  (artifacts/phase2c/HARDENED_DEVIATION_ALLOWLIST_V1.json in the reference).
"""
from __future__ import annotations

import ctypes as C
import json
import os
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

DEVIATION_ID = "dispatch.sm100_missing_kernel_fallback"
ALLOWLIST_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "conformance",
                              "HARDENED_DEVIATION_ALLOWLIST_V1.json")

# operators that only rearrange metadata or move bytes (no arithmetic kernel of the backend)
LAYOUT_OPS = frozenset({
    "reshape", "view", "squeeze", "unsqueeze", "transpose", "permute", "flatten", "unflatten", "narrow", "expand",
    "contiguous", "detach", "split", "chunk", "unbind", "movedim", "cat", "stack", "select", "slice", "t",
    "cast_f32", "cast_f64", "cast_f16", "cast_bf16", "to_dtype", "clone", "index_select", "gather", "flip", "roll",
    "repeat", "tile", "pad", "diagonal", "tril", "triu", "sum_to_shape", "hstack", "vstack", "dstack",
})


class NoKernelForBackend(RuntimeError):
    """Strict mode: the operator has no sm_100a kernel for these operands."""

    def __init__(self, op: str, why: str):
        super().__init__(f"op '{op}' has no sm_100a kernel for these operands ({why}); strict mode does not fall "
                         f"back - use hardened mode to run the library operator with fallback_path=true")
        self.op, self.why = op, why


def load_allowlist() -> Dict:
    with open(ALLOWLIST_PATH) as f:
        return json.load(f)


def fallback_allowed(mode_value: str) -> bool:
    """True when the allow-list permits the missing-kernel fallback in this mode."""
    for d in load_allowlist().get("deviations", []):
        if d.get("id") == DEVIATION_ID and mode_value in d.get("modes", []):
            return True
    return False


# ------------------------------------------------------------------------------------ eligibility
def _bf16_cuda(*ts: Optional[torch.Tensor]) -> bool:
    return all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in ts)


def _rows_ok(t: torch.Tensor) -> bool:
    """Contiguous with a last extent that is a multiple of 8 elements (16-byte TMA rows)."""
    return t.is_contiguous() and t.dim() >= 1 and t.shape[-1] % 8 == 0 and t.data_ptr() % 16 == 0


def gemm_kernel_name(M: int, N: int, Kd: int, *, a_mn: bool = False, b_mn: bool = False,
                     splittable: bool = True) -> str:
    """Name + tile configuration of the kernel ``ftk_gemm_bf16`` picks for this shape."""
    from ..ops import _lib
    from ..ops import kernels as K
    lib = _lib.load()
    g = _lib.FtkGemmDesc()
    g.M, g.N, g.K, g.L0, g.L1 = M, N, Kd, 1, 1
    g.a_mn, g.b_mn = int(a_mn), int(b_mn)
    g.A = g.B = g.D = 256          # aligned stand-ins: the plan query only looks at extents and alignment
    g.lda = M if a_mn else Kd
    g.ldb = N if b_mn else Kd
    g.ldd = N
    if splittable:
        g.workspace, g.workspace_bytes = 256, K.GEMM_WORKSPACE_BYTES
    bn, sp = C.c_int(0), C.c_int(1)
    lib.ftk_gemm_plan.argtypes = [C.POINTER(_lib.FtkGemmDesc), C.POINTER(C.c_int), C.POINTER(C.c_int)]
    lib.ftk_gemm_plan.restype = C.c_int
    rc = lib.ftk_gemm_plan(C.byref(g), C.byref(bn), C.byref(sp))
    if rc != 0:
        return "ftk::gemm_bf16_sm100<unplanned>"
    if bn.value == 512:
        return f"ftk::gemm2_bf16_sm100<256x256,cta_group2,splitK={sp.value}>"
    return f"ftk::gemm_bf16_sm100<128x{bn.value},splitK={sp.value}>"


# ------------------------------------------------------------------------------------ routes
# route(session, ids, vals, kw) -> (node_id, kernel_string) | None when the operands do not qualify
Route = Callable[[object, Sequence[int], List[torch.Tensor], dict], Optional[Tuple[int, str]]]
ROUTES: Dict[str, Route] = {}


def _route(name: str):
    def deco(fn: Route) -> Route:
        ROUTES[name] = fn
        return fn
    return deco


@_route("linear")
def _linear(s, ids, vals, kw):
    from ..ops import fused as F
    x, w = vals[0], vals[1]
    b = vals[2] if len(vals) > 2 else None
    if kw or not _bf16_cuda(x, w, b) or w.dim() != 2 or not _rows_ok(x) or not _rows_ok(w) or w.shape[0] % 8:
        return None
    nid = F.linear(s.tensor_tape, ids[0], ids[1], ids[2] if b is not None else None)
    rows = x.numel() // x.shape[-1]
    return nid, gemm_kernel_name(rows, w.shape[0], w.shape[1], splittable=b is None)


@_route("matmul")
def _matmul(s, ids, vals, kw):
    from ..ops import fused as F
    a, b = vals
    if kw or not _bf16_cuda(a, b) or a.dim() != 2 or b.dim() != 2 or not _rows_ok(a) or not _rows_ok(b) or \
            a.shape[0] % 8:
        return None
    return F.matmul(s.tensor_tape, ids[0], ids[1]), gemm_kernel_name(a.shape[0], b.shape[1], a.shape[1], b_mn=True)


@_route("bmm")
def _bmm(s, ids, vals, kw):
    from ..ops import fused as F
    a, b = vals
    if kw or not _bf16_cuda(a, b) or a.dim() != 3 or b.dim() != 3 or not _rows_ok(a) or not _rows_ok(b) or \
            a.shape[1] % 8:
        return None
    return F.bmm(s.tensor_tape, ids[0], ids[1]), "ftk::gemm_bf16_sm100<batched>"


@_route("layer_norm")
def _layer_norm(s, ids, vals, kw):
    from ..ops import fused as F
    if len(vals) != 3 or kw.get("ndim", 1) != 1 or not _bf16_cuda(*vals) or not _rows_ok(vals[0]):
        return None
    return F.layernorm(s.tensor_tape, ids[0], ids[1], ids[2], float(kw.get("eps", 1e-5))), \
        "ftk::norm_fwd_kernel<layer_norm>"


@_route("rms_norm")
def _rms_norm(s, ids, vals, kw):
    from ..ops import fused as F
    if len(vals) != 2 or not _bf16_cuda(*vals) or not _rows_ok(vals[0]):
        return None
    return F.rmsnorm(s.tensor_tape, ids[0], ids[1], float(kw.get("eps", 1e-6))), "ftk::norm_fwd_kernel<rms_norm>"


@_route("softmax")
def _softmax(s, ids, vals, kw):
    from ..ops import fused as F
    x = vals[0]
    dim = kw.get("dim", -1)
    if not _bf16_cuda(x) or not x.is_contiguous() or dim not in (-1, x.dim() - 1):
        return None
    return F.softmax_lastdim(s.tensor_tape, ids[0]), "ftk::softmax_rows_kernel"


def _gelu(tanh_form: bool) -> Route:
    def route(s, ids, vals, kw):
        from ..ops import fused as F
        x = vals[0]
        if kw or not _bf16_cuda(x) or not x.is_contiguous():
            return None
        return F.gelu(s.tensor_tape, ids[0], tanh_form=tanh_form), \
            f"ftk::ew_bf16_kernel<gelu_{'tanh' if tanh_form else 'erf'}>"
    return route


ROUTES["gelu"] = _gelu(False)
ROUTES["gelu_tanh"] = _gelu(True)


@_route("add")
def _add(s, ids, vals, kw):
    from ..ops import fused as F
    a, b = vals
    if kw or not _bf16_cuda(a, b) or a.shape != b.shape or not a.is_contiguous() or not b.is_contiguous():
        return None
    return F.add_same_shape(s.tensor_tape, ids[0], ids[1]), "ftk::ew_bf16_kernel<add>"


@_route("embedding")
def _embedding(s, ids, vals, kw):
    from ..ops import fused as F
    w, idx = vals
    if kw or not _bf16_cuda(w) or w.dim() != 2 or not _rows_ok(w) or not idx.is_cuda:
        return None
    return F.embedding_lookup(s.tensor_tape, ids[0], idx), "ftk::embedding_fwd_kernel"


@_route("sdpa")
def _sdpa(s, ids, vals, kw):
    from ..ops import fused as F
    if len(vals) != 3 or kw.get("mask") is not None:
        return None
    q, k, v = vals
    if not _bf16_cuda(q, k, v) or q.shape != k.shape or q.shape != v.shape or q.dim() not in (3, 4):
        return None
    if q.shape[-1] not in (64, 128) or not all(t.is_contiguous() for t in vals) or q.shape[-2] % 8:
        return None
    nid = F.sdpa(s.tensor_tape, ids[0], ids[1], ids[2], causal=bool(kw.get("is_causal", False)), scale=kw.get("scale"))
    return nid, f"ftk::attn_fwd2_kernel<hd={q.shape[-1]}>"


@_route("cross_entropy")
def _cross_entropy(s, ids, vals, kw):
    from ..ops import fused as F
    x, t = vals
    if kw.get("reduction", "mean") != "mean" or not _bf16_cuda(x) or x.dim() != 2 or not _rows_ok(x) or not t.is_cuda:
        return None
    return F.cross_entropy_mean(s.tensor_tape, ids[0], t), "ftk::cross_entropy_kernel"


HOT_OPS = frozenset(ROUTES) | {"dropout"}
