"""Sparse COO products, counting ops, low-rank factorisations, int8 dynamic linear and the
supervised-contrastive loss.

Reference families: ``sparse_coo_matmul_dense_f64`` / ``sparse_coo_coalesce`` / ``sparse_coo_add``
(crates/ft-kernel-cpu/src/lib.rs:42094-42214), ``svd_lowrank`` / ``pca_lowrank`` (``:34571-34761``),
int8 dynamic linear (``:37836-38138``), ``supcon_loss_forward`` (``:10947``).  Sparse tensors are
carried as a pair of dense tape nodes (``indices[nnz, ndim]`` f64-valued like every index tensor
of the session, ``values[nnz]``) plus a static shape, so the rule tables stay dense and real.
Everything here is deterministic: coalescing sorts by linear index with a stable sort and sums
duplicates in storage order.
"""
from __future__ import annotations

import torch

from .functions import OPS, OpDef, local_vjp


def _generic(name, fwd, rule=None):
    OPS[name] = OpDef(name, fwd, local_vjp(fwd), rule or f"d({name})/d_inputs [single-node differentiation]")


def _nograd(name, fwd, rule=None):
    OPS[name] = OpDef(name, fwd, None, rule or f"{name}: integer-valued, no gradient")


# ------------------------------------------------------------------------------------- sparse COO
def linear_index(indices: torch.Tensor, shape) -> torch.Tensor:
    idx = indices.long()
    lin = torch.zeros(idx.shape[0], dtype=torch.int64, device=idx.device)
    for d, n in enumerate(shape):
        if idx.numel() and (idx[:, d].min() < 0 or idx[:, d].max() >= n):
            raise IndexError(f"sparse index out of range in dimension {d}")
        lin = lin * n + idx[:, d]
    return lin


def coalesce(indices: torch.Tensor, values: torch.Tensor, shape):
    """Sorted unique indices and the sum of duplicate values (duplicates added in storage order)."""
    lin = linear_index(indices, shape)
    order = torch.sort(lin, stable=True).indices
    lin_s, val_s = lin[order], values[order]
    uniq, inverse = torch.unique_consecutive(lin_s, return_inverse=True)
    out = torch.zeros((uniq.shape[0],) + tuple(values.shape[1:]), dtype=values.dtype, device=values.device)
    out.index_add_(0, inverse, val_s)          # index_add_ on CPU adds in index order: deterministic
    idx = torch.empty((uniq.shape[0], len(shape)), dtype=indices.dtype, device=indices.device)
    rem = uniq.clone()
    for d in reversed(range(len(shape))):
        idx[:, d] = (rem % shape[d]).to(indices.dtype)
        rem = rem // shape[d]
    return idx, out


def _coo_to_dense(indices, values, shape=()):
    out = torch.zeros(tuple(shape) + tuple(values.shape[1:]), dtype=values.dtype, device=values.device)
    return out.index_put(tuple(indices.long().t()), values, accumulate=True)


def _coo_matmul_dense(indices, values, dense, shape=()):
    """``A[m, k] (COO) @ dense[k, n]``; rows with no entry are zero."""
    m, k = shape
    if dense.shape[0] != k:
        raise ValueError(f"sparse matmul inner size mismatch: {k} vs {dense.shape[0]}")
    idx = indices.long()
    contrib = values[:, None] * dense[idx[:, 1]]
    return torch.zeros((m, dense.shape[1]), dtype=dense.dtype, device=dense.device).index_add(0, idx[:, 0], contrib)


def _coo_values_after_coalesce(indices, values, shape=()):
    return coalesce(indices, values, shape)[1]


OPS["sparse_coo_to_dense"] = OpDef("sparse_coo_to_dense", _coo_to_dense, local_vjp(_coo_to_dense),
                                   "d(dense)/d(values) = gather at the indices")
OPS["sparse_coo_matmul_dense"] = OpDef("sparse_coo_matmul_dense", _coo_matmul_dense, local_vjp(_coo_matmul_dense),
                                       "d(A@B)/d(values)_e = <g[row_e], B[col_e]>; d/dB = A^T g")
OPS["sparse_coo_coalesce_values"] = OpDef("sparse_coo_coalesce_values", _coo_values_after_coalesce,
                                          local_vjp(_coo_values_after_coalesce),
                                          "duplicates share the gradient of their coalesced entry")
_nograd("sparse_coo_coalesce_indices", lambda indices, values, shape=(): coalesce(indices, values, shape)[0])


def csr_from_coo(indices: torch.Tensor, values: torch.Tensor, shape):
    """``(crow[m + 1], col[nnz], values[nnz])`` of a coalesced 2-D COO tensor."""
    idx, val = coalesce(indices, values, shape)
    rows = idx[:, 0].long()
    crow = torch.zeros(shape[0] + 1, dtype=torch.int64, device=idx.device)
    crow[1:] = torch.cumsum(torch.bincount(rows, minlength=shape[0]), 0)
    return crow, idx[:, 1].long(), val


# ------------------------------------------------------------------------------------- counting
_nograd("bincount", lambda x, minlength=0: torch.bincount(x.long(), minlength=minlength).to(torch.float64))
_nograd("histc", lambda x, bins=100, min=0.0, max=0.0: torch.histc(x, bins, min=min, max=max))
_nograd("unique", lambda x: torch.unique(x, sorted=True))
_nograd("unique_counts", lambda x: torch.unique(x, sorted=True, return_counts=True)[1].to(torch.float64))
_nograd("unique_inverse", lambda x: torch.unique(x, sorted=True, return_inverse=True)[1].to(torch.float64))
_nograd("bucketize", lambda x, boundaries, right=False: torch.bucketize(x, boundaries, right=right).to(torch.float64))


# ------------------------------------------------------------------------------------- low rank
def _seeded_normal(rows, cols, seed, like):
    # splitmix-style deterministic test matrix: no dependence on the global torch generator
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    return torch.randn(rows, cols, generator=g, dtype=torch.float64).to(like)


def _range_finder(a, q, niter, seed):
    """Orthonormal basis of an approximate range of ``a`` (Halko et al., subspace iteration)."""
    m, n = a.shape[-2:]
    omega = _seeded_normal(n, q, seed, a)
    Q = torch.linalg.qr(a @ omega).Q
    for _ in range(niter):
        Q = torch.linalg.qr(a.transpose(-1, -2) @ Q).Q
        Q = torch.linalg.qr(a @ Q).Q
    return Q


def svd_lowrank(a, q=6, niter=2, seed=0x4654):
    Q = _range_finder(a, min(q, *a.shape[-2:]), niter, seed)
    B = Q.transpose(-1, -2) @ a
    U, S, Vh = torch.linalg.svd(B, full_matrices=False)
    return Q @ U, S, Vh.transpose(-1, -2)


_generic("svd_lowrank_u", lambda a, q=6, niter=2, seed=0x4654: svd_lowrank(a, q, niter, seed)[0])
_generic("svd_lowrank_s", lambda a, q=6, niter=2, seed=0x4654: svd_lowrank(a, q, niter, seed)[1])
_generic("svd_lowrank_v", lambda a, q=6, niter=2, seed=0x4654: svd_lowrank(a, q, niter, seed)[2])


def pca_lowrank(a, q=6, center=True, niter=2, seed=0x4654):
    if center:
        a = a - a.mean(-2, keepdim=True)
    return svd_lowrank(a, q, niter, seed)


_generic("pca_lowrank_u", lambda a, q=6, center=True, niter=2, seed=0x4654: pca_lowrank(a, q, center, niter, seed)[0])
_generic("pca_lowrank_s", lambda a, q=6, center=True, niter=2, seed=0x4654: pca_lowrank(a, q, center, niter, seed)[1])
_generic("pca_lowrank_v", lambda a, q=6, center=True, niter=2, seed=0x4654: pca_lowrank(a, q, center, niter, seed)[2])


# ------------------------------------------------------------------------------------- int8 dynamic linear
def quantize_rows_int8(x):
    """Symmetric per-row int8 codes and scales: ``x ~ codes * scale[:, None]``."""
    amax = x.abs().amax(-1, keepdim=True).clamp(min=torch.finfo(x.dtype).tiny)
    scale = amax / 127.0
    return torch.clamp(torch.round(x / scale), -127, 127), scale


def _int8_dynamic_linear(x, w, b=None):
    """Activations quantised per row at run time, weights per output row; integer accumulate
    (exact in the float carrier: |sum| < 2^24 for in-features up to 1040), then rescale."""
    xq, xs = quantize_rows_int8(x)
    wq, ws = quantize_rows_int8(w)
    acc = xq.to(torch.float64) @ wq.to(torch.float64).t()
    y = (acc * xs.to(torch.float64) * ws.to(torch.float64).t()).to(x.dtype)
    return y + b if b is not None else y


def _int8_dynamic_linear_vjp(g, inputs, out, kw):
    # straight-through: gradients of the unquantised linear map
    x, w = inputs[0], inputs[1]
    grads = [g @ w, g.reshape(-1, g.shape[-1]).t() @ x.reshape(-1, x.shape[-1])]
    if len(inputs) > 2:
        grads.append(g.reshape(-1, g.shape[-1]).sum(0))
    return grads


OPS["int8_dynamic_linear"] = OpDef("int8_dynamic_linear", _int8_dynamic_linear, _int8_dynamic_linear_vjp,
                                   "straight-through: d/dx = g W, d/dW = g^T x, d/db = sum(g)")


# ------------------------------------------------------------------------------------- supervised contrastive
def _supcon_loss(features, labels, temperature=0.07):
    """Supervised contrastive loss over L2-normalised ``features[N, D]``: for every anchor the mean
    log-probability of its positives (same label, not itself) under a softmax over all others."""
    f = torch.nn.functional.normalize(features, dim=-1)
    n = f.shape[0]
    logits = (f @ f.t()) / temperature
    eye = torch.eye(n, dtype=torch.bool, device=f.device)
    logits = logits.masked_fill(eye, float("-inf"))
    logp = logits - torch.logsumexp(logits, dim=1, keepdim=True)
    pos = (labels.reshape(-1, 1) == labels.reshape(1, -1)) & ~eye
    cnt = pos.sum(1)
    per = -(torch.where(pos, logp, torch.zeros_like(logp)).sum(1)) / cnt.clamp(min=1).to(f.dtype)
    valid = cnt > 0
    return per[valid].mean() if bool(valid.any()) else per.sum() * 0.0


_generic("supcon_loss", _supcon_loss, "d(supcon)/d_features [softmax over non-self pairs]")
