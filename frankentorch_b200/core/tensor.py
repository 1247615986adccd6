"""Tensor value wrappers on top of ``torch.Tensor`` storage.

``DenseTensor`` mirrors the reference's dense tensor (ft-core/src/lib.rs:1063): an id, a
storage id shared by zero-copy views (:1810), and a version counter bumped by every in-place
update (:1715-1805).  Integer / bool tensors are dense tensors of the matching dtype.  Sparse
COO / CSR tensors (:2356, :2765) wrap torch's sparse layouts with the same constructors and
``to_dense`` / ``coalesce`` / ``matmul_dense`` / ``add`` operations
(ft-kernel-cpu/src/lib.rs:42094-42214).
"""
from __future__ import annotations

import itertools
from typing import Callable, Optional, Sequence

import torch

from .dtype import DType
from .meta import Device, TensorMeta, TensorMetaError

_NEXT_TENSOR_ID = itertools.count(1)
_NEXT_STORAGE_ID = itertools.count(1)


class DenseTensorError(ValueError):
    pass


class DenseTensor:
    __slots__ = ("id", "storage_id", "_version", "data")

    def __init__(self, data: torch.Tensor, storage_id: Optional[int] = None, version=None):
        self.id = next(_NEXT_TENSOR_ID)
        self.storage_id = next(_NEXT_STORAGE_ID) if storage_id is None else storage_id
        self._version = version if version is not None else [0]   # shared cell between views
        self.data = data

    # ------------------------------------------------------------------ constructors
    @staticmethod
    def from_values(values: Sequence[float], shape: Sequence[int], dtype: DType = DType.F64) -> "DenseTensor":
        n = 1
        for s in shape:
            n *= s
        if len(values) != n:
            raise DenseTensorError(f"value count {len(values)} does not match shape {tuple(shape)}")
        return DenseTensor(torch.tensor(list(values), dtype=dtype.to_torch()).reshape(tuple(shape)))

    @staticmethod
    def scalar(value: float, dtype: DType = DType.F64) -> "DenseTensor":
        return DenseTensor(torch.tensor(value, dtype=dtype.to_torch()))

    # ------------------------------------------------------------------ metadata
    @property
    def meta(self) -> TensorMeta:
        t = self.data
        dev = Device.Cuda if t.is_cuda else Device.Cpu
        return TensorMeta.from_shape_and_strides(t.shape, t.stride(), t.storage_offset(), DType.from_torch(t.dtype), dev)

    @property
    def version(self) -> int:
        return self._version[0]

    def dtype(self) -> DType:
        return DType.from_torch(self.data.dtype)

    def numel(self) -> int:
        return self.data.numel()

    def contiguous_values(self):
        return self.data.contiguous().reshape(-1).tolist()

    # ------------------------------------------------------------------ views / updates
    def view(self, shape: Sequence[int]) -> "DenseTensor":
        """Zero-copy reshape sharing the storage id and the version counter."""
        if not self.data.is_contiguous():
            raise DenseTensorError("view requires a contiguous tensor")
        return DenseTensor(self.data.view(tuple(shape)), storage_id=self.storage_id, version=self._version)

    def to_dtype(self, dtype: DType) -> "DenseTensor":
        return DenseTensor(self.data.to(dtype.to_torch()))

    def update_contiguous_values(self, values: Sequence[float]) -> None:
        if len(values) != self.data.numel():
            raise DenseTensorError("update length mismatch")
        self.data.copy_(torch.tensor(list(values), dtype=self.data.dtype).reshape(self.data.shape))
        self._version[0] += 1

    def update_contiguous_values_with(self, fn: Callable[[torch.Tensor], None]) -> None:
        fn(self.data)
        self._version[0] += 1


def DenseI64Tensor(values, shape) -> DenseTensor:
    return DenseTensor.from_values(values, shape, DType.I64)


def DenseI32Tensor(values, shape) -> DenseTensor:
    return DenseTensor.from_values(values, shape, DType.I32)


def DenseBoolTensor(values, shape) -> DenseTensor:
    return DenseTensor(torch.tensor(list(values), dtype=torch.bool).reshape(tuple(shape)))


class SparseTensorError(ValueError):
    pass


class SparseCOOTensor:
    """COO tensor: ``indices`` [sparse_dim, nnz] int64, ``values`` [nnz, ...dense dims]."""

    def __init__(self, indices: torch.Tensor, values: torch.Tensor, shape: Sequence[int]):
        indices = torch.as_tensor(indices, dtype=torch.int64)
        values = torch.as_tensor(values)
        if indices.dim() != 2 or indices.shape[1] != values.shape[0]:
            raise SparseTensorError("indices must be [sparse_dim, nnz] matching values' first dim")
        if indices.shape[0] + values.dim() - 1 != len(shape):
            raise SparseTensorError("sparse_dim + dense_dim must equal the rank of the shape")
        for d in range(indices.shape[0]):
            if indices.shape[1] and (indices[d].min() < 0 or indices[d].max() >= shape[d]):
                raise SparseTensorError(f"index out of bounds in sparse dim {d}")
        self.indices, self.values, self.shape = indices, values, tuple(shape)

    @property
    def nnz(self) -> int:
        return int(self.indices.shape[1])

    def _torch(self) -> torch.Tensor:
        return torch.sparse_coo_tensor(self.indices, self.values, self.shape)

    def to_dense(self) -> torch.Tensor:
        return self._torch().to_dense()

    def coalesce(self) -> "SparseCOOTensor":
        c = self._torch().coalesce()
        return SparseCOOTensor(c.indices(), c.values(), self.shape)

    def matmul_dense(self, dense: torch.Tensor) -> torch.Tensor:
        return torch.sparse.mm(self._torch().coalesce(), dense)

    def add(self, other: "SparseCOOTensor") -> "SparseCOOTensor":
        if self.shape != other.shape:
            raise SparseTensorError("shape mismatch in sparse add")
        c = (self._torch() + other._torch()).coalesce()
        return SparseCOOTensor(c.indices(), c.values(), self.shape)


class SparseCSRTensor:
    def __init__(self, crow_indices, col_indices, values, shape: Sequence[int]):
        self.crow = torch.as_tensor(crow_indices, dtype=torch.int64)
        self.col = torch.as_tensor(col_indices, dtype=torch.int64)
        self.values = torch.as_tensor(values)
        self.shape = tuple(shape)
        if len(self.shape) != 2 or self.crow.numel() != self.shape[0] + 1:
            raise SparseTensorError("CSR needs a 2-D shape and rows+1 row pointers")
        if self.col.numel() != self.values.numel() or int(self.crow[-1]) != self.col.numel():
            raise SparseTensorError("CSR column/value/row-pointer lengths disagree")
        if bool((self.crow[1:] < self.crow[:-1]).any()):
            raise SparseTensorError("CSR row pointers must be non-decreasing")
        if self.col.numel() and (self.col.min() < 0 or self.col.max() >= self.shape[1]):
            raise SparseTensorError("CSR column index out of bounds")

    def to_dense(self) -> torch.Tensor:
        return torch.sparse_csr_tensor(self.crow, self.col, self.values, self.shape).to_dense()

    def to_coo(self) -> SparseCOOTensor:
        rows = torch.repeat_interleave(torch.arange(self.shape[0]), self.crow[1:] - self.crow[:-1])
        return SparseCOOTensor(torch.stack([rows, self.col]), self.values, self.shape)
