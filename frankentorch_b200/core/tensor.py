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
    __slots__ = ("id", "storage_id", "_version", "data", "quantization")

    def __init__(self, data: torch.Tensor, storage_id: Optional[int] = None, version=None):
        self.id = next(_NEXT_TENSOR_ID)
        self.storage_id = next(_NEXT_STORAGE_ID) if storage_id is None else storage_id
        self._version = version if version is not None else [0]   # shared cell between views
        self.data = data
        self.quantization = None                                   # QuantizationParams of a quantized tensor

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

    @staticmethod
    def from_typed_storage(meta: TensorMeta, storage) -> "DenseTensor":
        """Tensor over an existing typed buffer (ft-core/src/lib.rs:1151): the dtype of ``meta`` must be the
        storage's variant and the layout must fit inside the buffer.  Quantized tensors keep their integer codes;
        ``meta.quantization`` says how to read them."""
        meta.validate()
        if meta.dtype != storage.dtype:
            raise DenseTensorError(f"meta dtype {meta.dtype.value} does not match storage variant {storage.dtype.value}")
        need = meta.storage_offset + sum((n - 1) * st for n, st in zip(meta.shape, meta.strides) if n) + (1 if meta.numel else 0)
        if meta.numel and need > len(storage):
            raise DenseTensorError(f"layout needs {need} storage elements, the buffer holds {len(storage)}")
        t = DenseTensor(torch.as_strided(storage.data, meta.shape, meta.strides, meta.storage_offset))
        t.quantization = meta.quantization
        return t

    @staticmethod
    def from_storage(meta: TensorMeta, values) -> "DenseTensor":
        """``from_typed_storage`` over a fresh buffer of ``meta.dtype`` holding ``values``
        (``from_storage`` / ``from_storage_f32`` / ``_f16`` / ``_bf16`` / ``_qint8`` / ``_quint8`` of the reference)."""
        from .storage import TensorStorage
        return DenseTensor.from_typed_storage(meta, TensorStorage.from_values(values, meta.dtype))

    @staticmethod
    def from_contiguous_values(values, shape: Sequence[int], device=Device.Cpu, dtype: DType = DType.F64) -> "DenseTensor":
        t = DenseTensor.from_storage(TensorMeta.from_shape(shape, dtype, Device.Cpu), values)
        if Device.parse(device) == Device.Cuda:
            t.data = t.data.cuda()
        return t

    @staticmethod
    def from_contiguous_values_quantized(codes, shape: Sequence[int], dtype: DType, scale: float, zero_point: int) -> "DenseTensor":
        """Quantized tensor from integer codes with per-tensor parameters (``from_contiguous_values_qint8 / _quint8``)."""
        return DenseTensor.from_storage(TensorMeta.quantized_from_shape(shape, dtype, Device.Cpu, scale, zero_point), codes)

    @staticmethod
    def from_contiguous_values_quantized_per_channel(codes, shape: Sequence[int], dtype: DType, scales, zero_points,
                                                     axis: int) -> "DenseTensor":
        meta = TensorMeta.quantized_per_channel_from_shape(shape, dtype, Device.Cpu, scales, zero_points, axis)
        return DenseTensor.from_storage(meta, codes)

    def typed_storage(self):
        """The whole underlying buffer as a :class:`TensorStorage` (views share it)."""
        from .storage import TensorStorage
        base = self.data._base if self.data._base is not None else self.data
        flat = base.reshape(-1) if base.is_contiguous() else base.contiguous().reshape(-1)
        return TensorStorage.from_tensor(flat)

    def shares_storage_with(self, other: "DenseTensor") -> bool:
        return self.storage_id == other.storage_id

    def contiguous_values_as_f64(self) -> list:
        """Values in row-major order as f64; a quantized tensor is dequantized with its parameters."""
        return self.dequantized_values_as_f64() if getattr(self, "quantization", None) is not None else \
            self.data.contiguous().reshape(-1).to(torch.float64).tolist()

    def dequantized_values_as_f64(self) -> list:
        q = getattr(self, "quantization", None)
        if q is None:
            raise DenseTensorError("tensor carries no quantization parameters")
        codes = self.data.to(torch.float64)
        if not q.is_per_channel():
            return ((codes - q.zero_point) * q.scale).contiguous().reshape(-1).tolist()
        shape = [1] * codes.dim()
        shape[q.axis] = len(q)
        sc = torch.tensor(q.scales(), dtype=torch.float64).reshape(shape)
        zp = torch.tensor(q.zero_points(), dtype=torch.float64).reshape(shape)
        return ((codes - zp) * sc).contiguous().reshape(-1).tolist()

    # ------------------------------------------------------------------ per-dtype forms
    # The reference spells one constructor and one accessor per storage variant
    # (ft-core/src/lib.rs:1178-1245 ``from_storage_f64 / _f64_inline4 / _f32 / _f16 / _bf16 / _qint8 / _quint8``,
    # :1247-1370 ``from_contiguous_values_<dtype>``, :1392-1466 ``dispatch_values`` /
    # ``contiguous_values_<dtype>[_mut]``, :1778 ``update_contiguous_values_f32``).  Here they are the generic
    # forms with the dtype pinned and the same refusals: a meta of another dtype, a strided layout.
    @staticmethod
    def _from_storage_of(dtype: DType, meta: TensorMeta, values) -> "DenseTensor":
        if meta.dtype != dtype:
            raise DenseTensorError(f"unsupported dtype {meta.dtype.value} for a {dtype.value} buffer")
        return DenseTensor.from_storage(meta, values)

    @staticmethod
    def from_storage_f64(meta, values): return DenseTensor._from_storage_of(DType.F64, meta, values)          # noqa: E704
    @staticmethod
    def from_storage_f32(meta, values): return DenseTensor._from_storage_of(DType.F32, meta, values)          # noqa: E704
    @staticmethod
    def from_storage_f16(meta, values): return DenseTensor._from_storage_of(DType.F16, meta, values)          # noqa: E704
    @staticmethod
    def from_storage_bf16(meta, values): return DenseTensor._from_storage_of(DType.BF16, meta, values)        # noqa: E704
    @staticmethod
    def from_storage_qint8(meta, values): return DenseTensor._from_storage_of(DType.QInt8, meta, values)      # noqa: E704
    @staticmethod
    def from_storage_quint8(meta, values): return DenseTensor._from_storage_of(DType.QUInt8, meta, values)    # noqa: E704

    @staticmethod
    def from_storage_f64_inline4(meta: TensorMeta, values) -> "DenseTensor":
        """A tensor of at most four f64 values held inline (no heap buffer in the reference; a 4-element buffer
        here): scalar losses and tiny parameters."""
        values = list(values)
        if len(values) != 4:
            raise DenseTensorError(f"inline storage holds exactly 4 values, got {len(values)}")
        return DenseTensor._from_storage_of(DType.F64, meta, values)

    @staticmethod
    def from_contiguous_values_f32(values, shape, device=Device.Cpu): return DenseTensor.from_contiguous_values(values, shape, device, DType.F32)    # noqa: E704
    @staticmethod
    def from_contiguous_values_f16(values, shape, device=Device.Cpu): return DenseTensor.from_contiguous_values(values, shape, device, DType.F16)    # noqa: E704
    @staticmethod
    def from_contiguous_values_bf16(values, shape, device=Device.Cpu): return DenseTensor.from_contiguous_values(values, shape, device, DType.BF16)  # noqa: E704

    @staticmethod
    def from_contiguous_values_qint8(codes, shape, scale: float, zero_point: int) -> "DenseTensor":
        return DenseTensor.from_contiguous_values_quantized(codes, shape, DType.QInt8, scale, zero_point)

    @staticmethod
    def from_contiguous_values_quint8(codes, shape, scale: float, zero_point: int) -> "DenseTensor":
        return DenseTensor.from_contiguous_values_quantized(codes, shape, DType.QUInt8, scale, zero_point)

    @staticmethod
    def from_contiguous_values_qint8_per_channel(codes, shape, scales, zero_points, axis: int) -> "DenseTensor":
        return DenseTensor.from_contiguous_values_quantized_per_channel(codes, shape, DType.QInt8, scales, zero_points, axis)

    @staticmethod
    def from_contiguous_values_quint8_per_channel(codes, shape, scales, zero_points, axis: int) -> "DenseTensor":
        return DenseTensor.from_contiguous_values_quantized_per_channel(codes, shape, DType.QUInt8, scales, zero_points, axis)

    def _typed_view(self, want: DType, contiguous: bool = True) -> torch.Tensor:
        have = self.meta.dtype
        if have != want:
            raise DenseTensorError(f"unsupported dtype {have.value}: this accessor reads {want.value}")
        if contiguous and not self.data.is_contiguous():
            raise DenseTensorError("unsupported layout: the tensor is not contiguous")
        return self.data

    def dispatch_values(self) -> torch.Tensor:
        """The f64 storage span the layout covers, from the view's offset to its last element, as a flat
        zero-copy tensor: what a kernel that applies the strides itself receives (a strided view is allowed)."""
        t = self._typed_view(DType.F64, contiguous=False)
        if t.numel() == 0:
            return t.reshape(-1)
        span = 1 + sum((n - 1) * st for n, st in zip(t.shape, t.stride()))
        return torch.as_strided(t, (span,), (1,), t.storage_offset())

    def contiguous_values_f32(self) -> torch.Tensor:
        """The values of a contiguous f32 tensor as a flat zero-copy tensor."""
        return self._typed_view(DType.F32).reshape(-1)

    def contiguous_values_f32_mut(self) -> torch.Tensor:
        """The same, for writing: an inference-only consumer overwrites a dead intermediate in place.  The
        version counter moves, so a tape node that borrowed the old contents is caught at backward."""
        out = self._typed_view(DType.F32).reshape(-1)
        self._version[0] += 1
        return out

    def contiguous_values_qint8(self) -> torch.Tensor:
        return self._typed_view(DType.QInt8).reshape(-1)

    def contiguous_values_quint8(self) -> torch.Tensor:
        return self._typed_view(DType.QUInt8).reshape(-1)

    def update_contiguous_values_f32(self, values) -> None:
        dst = self._typed_view(DType.F32)
        src = torch.as_tensor(values, dtype=torch.float32).reshape(-1)
        if src.numel() != dst.numel():
            raise DenseTensorError(f"insufficient storage: needed {dst.numel()}, got {src.numel()}")
        dst.reshape(-1).copy_(src)
        self._version[0] += 1

    # ------------------------------------------------------------------ metadata
    @property
    def meta(self) -> TensorMeta:
        t = self.data
        dev = Device.Cuda if t.is_cuda else Device.Cpu
        if self.quantization is not None:
            dt = DType.QInt8 if t.dtype == torch.int8 else DType.QUInt8
            return TensorMeta.from_shape_and_strides(t.shape, t.stride(), t.storage_offset(), dt, dev).with_quantization(self.quantization)
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


def dense_bool_from_bools(values: Sequence[bool], shape: Sequence[int], device=Device.Cpu) -> DenseTensor:
    """``DenseBoolTensor::from_bools`` (ft-core/src/lib.rs:2051)."""
    n = 1
    for s_ in shape:
        n *= s_
    if len(values) != n:
        raise DenseTensorError(f"value count {len(values)} does not match shape {tuple(shape)}")
    t = DenseBoolTensor([bool(v) for v in values], shape)
    if Device.parse(device) == Device.Cuda:
        t.data = t.data.cuda()
    return t


def contiguous_bools(t: DenseTensor) -> list:
    """Row-major ``bool`` list of a bool (or integer) tensor: non-zero is true."""
    return [bool(v) for v in t.data.contiguous().reshape(-1).tolist()]


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

    @staticmethod
    def from_coords(coords: Sequence[Sequence[int]], values, dense_shape: Sequence[int], dtype: DType = DType.F64,
                    device=Device.Cpu) -> "SparseCOOTensor":
        """One coordinate list per non-zero (``coords[k]`` is the index tuple of ``values[k]``); an empty list gives
        an all-zero tensor whose sparse dimension is the full rank (ft-core/src/lib.rs:2515)."""
        nnz = len(coords)
        sd = len(dense_shape) if nnz == 0 else len(coords[0])
        if any(len(c) != sd for c in coords):
            raise SparseTensorError("every coordinate must have the same length")
        if len(values) != nnz:
            raise SparseTensorError(f"{len(values)} values for {nnz} coordinates")
        idx = torch.tensor(list(coords), dtype=torch.int64).reshape(nnz, sd).t().contiguous()
        dev = "cuda" if Device.parse(device) == Device.Cuda else "cpu"
        return SparseCOOTensor(idx.to(dev), torch.tensor(list(values), dtype=dtype.to_torch(), device=dev), dense_shape)

    @property
    def nnz(self) -> int:
        return int(self.indices.shape[1])

    def dense_shape(self):
        return list(self.shape)

    @property
    def sparse_dim(self) -> int:
        return int(self.indices.shape[0])

    def is_coalesced(self) -> bool:
        """True when the coordinates are unique and in row-major order."""
        if self.nnz <= 1:
            return True
        key = torch.zeros(self.nnz, dtype=torch.int64, device=self.indices.device)
        for d in range(self.sparse_dim):
            key = key * int(self.shape[d]) + self.indices[d]
        return bool((key[1:] > key[:-1]).all())

    def _torch(self) -> torch.Tensor:
        return torch.sparse_coo_tensor(self.indices, self.values, self.shape, check_invariants=False)   # bounds were checked at construction

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

    def nrows(self) -> int:
        return self.shape[0]

    def ncols(self) -> int:
        return self.shape[1]

    @property
    def nnz(self) -> int:
        return int(self.col.numel())

    def to_dense(self) -> torch.Tensor:
        return torch.sparse_csr_tensor(self.crow, self.col, self.values, self.shape).to_dense()

    def to_coo(self) -> SparseCOOTensor:
        rows = torch.repeat_interleave(torch.arange(self.shape[0]), self.crow[1:] - self.crow[:-1])
        return SparseCOOTensor(torch.stack([rows, self.col]), self.values, self.shape)
