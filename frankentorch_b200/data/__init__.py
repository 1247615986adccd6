"""Datasets, samplers, the deterministic DataLoader and transforms (mirror of ft-data).

Reference: ft-data/src/lib.rs - ``DataItem`` (named flat tensors) :50, ``Dataset`` trait :82,
``TensorDataset`` with columnar collation :113-209, ``Batch`` :218, the 64-bit LCG
``state*6364136223846793005+1`` with draws ``(state>>33) % bound`` and Fisher-Yates from the
top index down :246-273, samplers :376-760 (default seeds ``0xCAFEBABE12345678`` for
RandomSampler, ``0xFEEDFACEDEADBEEF`` for WeightedRandomSampler), ``DataLoaderConfig`` :761,
``DataLoader`` :794-919 (default seed ``0xDEADBEEFCAFE1234``; the shuffle happens lazily on the
first ``next_batch`` after construction / ``reset`` / ``seed`` and the RNG state carries across
epochs; ``drop_last`` drops a short tail; ``batch_size == 0`` yields nothing), transforms
:1184-1336, ``TransformDataset`` / ``Subset`` / ``random_split`` :1338-1401.
The LCG and the shuffle run in the native runtime so large index sets shuffle quickly.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..runtime import native

DATALOADER_DEFAULT_SEED = 0xDEADBEEFCAFE1234
RANDOM_SAMPLER_DEFAULT_SEED = 0xCAFEBABE12345678
WEIGHTED_SAMPLER_DEFAULT_SEED = 0xFEEDFACEDEADBEEF


class DataError(ValueError):
    pass


class SimpleRng:
    """The data pipeline's LCG (distinct from the session's xoshiro stream)."""

    def __init__(self, seed: int):
        self._lib = native.load()
        self._state = C.c_uint64(seed & ((1 << 64) - 1))

    @property
    def state(self) -> int:
        return int(self._state.value)

    @state.setter
    def state(self, v: int) -> None:
        self._state.value = v & ((1 << 64) - 1)

    def next(self) -> int:
        return int(self._lib.ftc_lcg_next(C.byref(self._state)))

    def below(self, bound: int) -> int:
        return self.next() % bound

    def shuffle(self, idx: List[int]) -> List[int]:
        arr = (C.c_int64 * max(len(idx), 1))(*idx)
        self._lib.ftc_lcg_shuffle(C.byref(self._state), arr, len(idx))
        return [int(arr[i]) for i in range(len(idx))]

    def uniform(self) -> float:
        return self.next() / float(1 << 31)


@dataclass
class DataItem:
    """One sample: named flat value lists with their shapes."""
    tensors: Dict[str, Tuple[List[float], Tuple[int, ...]]] = field(default_factory=dict)

    def insert(self, name: str, values: Sequence[float], shape: Sequence[int]) -> "DataItem":
        n = 1
        for s in shape:
            n *= s
        if n != len(values):
            raise DataError(f"{name}: {len(values)} values do not fill shape {tuple(shape)}")
        self.tensors[name] = (list(values), tuple(shape))
        return self

    @staticmethod
    def input_target(input_values, input_shape, target_values, target_shape) -> "DataItem":
        """One sample with an ``input`` and a ``target`` tensor (ft-data/src/lib.rs:57)."""
        return DataItem().insert("input", input_values, input_shape).insert("target", target_values, target_shape)

    @staticmethod
    def single(name: str, values, shape) -> "DataItem":
        return DataItem().insert(name, values, shape)


class Dataset:
    def __len__(self) -> int:
        raise NotImplementedError

    def get(self, index: int) -> DataItem:
        raise NotImplementedError

    def is_empty(self) -> bool:
        return len(self) == 0


class TensorDataset(Dataset):
    """Columns of equal leading length; collation gathers rows of the pre-packed columns."""

    @staticmethod
    def from_items(items: Sequence[DataItem]) -> "TensorDataset":
        """Columnar dataset from samples that all carry the same named tensors with the same shapes."""
        if not items:
            raise DataError("TensorDataset needs at least one item")
        names = list(items[0].tensors)
        cols = {}
        for n in names:
            shape = items[0].tensors[n][1]
            rows = []
            for k, it in enumerate(items):
                if n not in it.tensors or it.tensors[n][1] != shape:
                    raise DataError(f"item {k}: tensor '{n}' is missing or its shape differs from item 0")
                rows.append(it.tensors[n][0])
            cols[n] = torch.tensor(rows, dtype=torch.float64).reshape((len(items),) + tuple(shape))
        return TensorDataset(cols)

    @staticmethod
    def from_inputs_targets(inputs: Sequence[Tuple[Sequence[float], Sequence[int]]],
                            targets: Sequence[Tuple[Sequence[float], Sequence[int]]]) -> "TensorDataset":
        """Parallel lists of ``(values, shape)``: pair ``k`` becomes sample ``k`` with tensors ``input`` and ``target``
        (ft-data/src/lib.rs:136)."""
        if len(inputs) != len(targets):
            raise DataError("inputs and targets must have same length")
        return TensorDataset.from_items([DataItem.input_target(iv, ish, tv, tsh) for (iv, ish), (tv, tsh) in zip(inputs, targets)])

    def __init__(self, columns: Dict[str, torch.Tensor]):
        if not columns:
            raise DataError("TensorDataset needs at least one column")
        lens = {int(t.shape[0]) for t in columns.values()}
        if len(lens) != 1:
            raise DataError(f"columns disagree on the number of samples: {sorted(lens)}")
        self.columns = {k: v.detach().to(torch.float64) if v.is_floating_point() else v.detach() for k, v in columns.items()}
        self._n = lens.pop()

    def __len__(self):
        return self._n

    def get(self, index: int) -> DataItem:
        if not 0 <= index < self._n:
            raise DataError(f"index {index} out of range for {self._n} samples")
        item = DataItem()
        for k, t in self.columns.items():
            item.insert(k, t[index].reshape(-1).tolist(), tuple(t.shape[1:]))
        return item

    def collate_indices(self, indices: Sequence[int]) -> Dict[str, torch.Tensor]:
        idx = torch.tensor(list(indices), dtype=torch.int64)
        return {k: t.index_select(0, idx) for k, t in self.columns.items()}


@dataclass
class Batch:
    """Named session tensors (node ids) of one collated batch plus the source indices."""
    tensors: Dict[str, int]
    indices: List[int]
    size: int

    def get(self, name: str) -> int:
        return self.tensors[name]


def collate(items: Sequence[DataItem]) -> Dict[str, torch.Tensor]:
    """Stack items along a new leading dim after validating names and shapes."""
    if not items:
        raise DataError("cannot collate an empty list of items")
    names = list(items[0].tensors)
    out = {}
    for n in names:
        shape = items[0].tensors[n][1]
        rows = []
        for it in items:
            if n not in it.tensors or set(it.tensors) != set(names):
                raise DataError("items disagree on tensor names")
            if it.tensors[n][1] != shape:
                raise DataError(f"items disagree on the shape of '{n}'")
            rows.append(torch.tensor(it.tensors[n][0], dtype=torch.float64).reshape(shape))
        out[n] = torch.stack(rows, 0)
    return out


# -------------------------------------------------------------------------------------- samplers
class Sampler:
    def indices(self) -> List[int]:
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError


class SequentialSampler(Sampler):
    def __init__(self, n: int):
        self.n = n

    def indices(self):
        return list(range(self.n))

    def __len__(self):
        return self.n


class RandomSampler(Sampler):
    def __init__(self, n: int, seed: int = RANDOM_SAMPLER_DEFAULT_SEED, replacement: bool = False,
                 num_samples: Optional[int] = None):
        self.n, self.rng, self.replacement, self.num_samples = n, SimpleRng(seed), replacement, num_samples or n

    def indices(self):
        if self.replacement:
            return [self.rng.below(self.n) for _ in range(self.num_samples)] if self.n else []
        return self.rng.shuffle(list(range(self.n)))[: self.num_samples]

    def __len__(self):
        return self.num_samples


class SubsetRandomSampler(Sampler):
    def __init__(self, subset: Sequence[int], seed: int = RANDOM_SAMPLER_DEFAULT_SEED):
        self.subset, self.rng = list(subset), SimpleRng(seed)

    def indices(self):
        return self.rng.shuffle(list(self.subset))

    def __len__(self):
        return len(self.subset)


class WeightedRandomSampler(Sampler):
    def __init__(self, weights: Sequence[float], num_samples: int, replacement: bool = True,
                 seed: int = WEIGHTED_SAMPLER_DEFAULT_SEED):
        if any((w < 0) or (w != w) for w in weights) or sum(weights) <= 0:
            raise DataError("weights must be non-negative with a positive sum")
        if not replacement and num_samples > sum(1 for w in weights if w > 0):
            raise DataError("not enough positive weights to sample without replacement")
        self.weights, self.num_samples, self.replacement, self.rng = list(weights), num_samples, replacement, SimpleRng(seed)

    def indices(self):
        w, out = list(self.weights), []
        for _ in range(self.num_samples):
            total = sum(w)
            x = self.rng.uniform() * total
            acc, pick = 0.0, len(w) - 1
            for i, wi in enumerate(w):
                acc += wi
                if wi > 0 and x < acc:
                    pick = i
                    break
            out.append(pick)
            if not self.replacement:
                w[pick] = 0.0
        return out

    def __len__(self):
        return self.num_samples


class BatchSampler(Sampler):
    def __init__(self, sampler: Sampler, batch_size: int, drop_last: bool = False):
        self.sampler, self.batch_size, self.drop_last = sampler, batch_size, drop_last

    def batches(self) -> List[List[int]]:
        if self.batch_size == 0:
            return []
        idx = self.sampler.indices()
        out = [idx[i: i + self.batch_size] for i in range(0, len(idx), self.batch_size)]
        if self.drop_last and out and len(out[-1]) < self.batch_size:
            out.pop()
        return out

    def indices(self):
        return [i for b in self.batches() for i in b]

    def __len__(self):
        n = len(self.sampler)
        if self.batch_size == 0:
            return 0
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size


# -------------------------------------------------------------------------------------- loader
@dataclass
class DataLoaderConfig:
    batch_size: int = 1
    shuffle: bool = False
    drop_last: bool = False

    @staticmethod
    def new(batch_size: int) -> "DataLoaderConfig":
        return DataLoaderConfig(batch_size)

    def with_shuffle(self, flag: bool) -> "DataLoaderConfig":
        self.shuffle = flag
        return self

    def with_drop_last(self, flag: bool) -> "DataLoaderConfig":
        self.drop_last = flag
        return self


class DataLoader:
    def __init__(self, dataset: Dataset, config: DataLoaderConfig, indices: Optional[Sequence[int]] = None):
        self.dataset, self.config = dataset, config
        self._base = list(indices) if indices is not None else list(range(len(dataset)))
        for i in self._base:
            if not 0 <= i < len(dataset):
                raise DataError(f"index {i} out of range for {len(dataset)} samples")
        self._rng = SimpleRng(DATALOADER_DEFAULT_SEED)
        self._order: Optional[List[int]] = None
        self._cursor = 0

    @staticmethod
    def with_indices(dataset: Dataset, config: DataLoaderConfig, indices: Sequence[int]) -> "DataLoader":
        return DataLoader(dataset, config, indices)

    def seed(self, seed: int) -> None:
        self._rng = SimpleRng(seed)
        self.reset()

    def reset(self) -> None:
        """Start a new epoch; a shuffling loader draws the next permutation on the next batch."""
        self._order, self._cursor = None, 0

    def state_dict(self) -> Dict:
        """Position of the loader: LCG state, cursor and the current epoch's order (plain values),
        so a resumed job draws the same remaining batches and the same later permutations."""
        return {"rng_state": int(self._rng.state), "cursor": int(self._cursor),
                "order": None if self._order is None else [int(i) for i in self._order]}

    def load_state_dict(self, sd: Dict) -> None:
        order = sd.get("order")
        if order is not None and sorted(order) != sorted(self._base):
            raise DataError("the saved order does not index this loader's dataset")
        self._rng.state = int(sd["rng_state"])
        self._cursor = int(sd["cursor"])
        self._order = None if order is None else [int(i) for i in order]

    def num_batches(self) -> int:
        bs, n = self.config.batch_size, len(self._base)
        if bs == 0:
            return 0
        return n // bs if self.config.drop_last else (n + bs - 1) // bs

    def _ensure_order(self) -> None:
        if self._order is None:
            self._order = self._rng.shuffle(list(self._base)) if self.config.shuffle else list(self._base)

    def next_indices(self) -> Optional[List[int]]:
        bs = self.config.batch_size
        if bs == 0:
            return None
        self._ensure_order()
        if self._cursor >= len(self._order):
            return None
        chunk = self._order[self._cursor: self._cursor + bs]
        if self.config.drop_last and len(chunk) < bs:
            self._cursor = len(self._order)
            return None
        self._cursor += len(chunk)
        return chunk

    def next_batch(self, session) -> Optional[Batch]:
        idx = self.next_indices()
        if idx is None:
            return None
        if hasattr(self.dataset, "collate_indices"):
            cols = self.dataset.collate_indices(idx)
        else:
            cols = collate([self.dataset.get(i) for i in idx])
        return Batch({k: session.tensor_variable_from_storage(v, False) for k, v in cols.items()}, idx, len(idx))

    def __iter__(self):
        self.reset()
        while True:
            idx = self.next_indices()
            if idx is None:
                return
            yield idx

    # loader position for checkpoint / resume
    def state_dict(self) -> Dict:
        return {"rng_state": self._rng.state, "order": self._order, "cursor": self._cursor}

    def load_state_dict(self, sd: Dict) -> None:
        self._rng.state = int(sd["rng_state"])
        self._order = None if sd["order"] is None else list(sd["order"])
        self._cursor = int(sd["cursor"])


# -------------------------------------------------------------------------------------- transforms
class Transform:
    def __call__(self, item: DataItem) -> DataItem:
        raise NotImplementedError


class Compose(Transform):
    def __init__(self, transforms: Sequence[Transform]):
        self.transforms = list(transforms)

    def __call__(self, item):
        for t in self.transforms:
            item = t(item)
        return item


class Normalize(Transform):
    def __init__(self, name: str, mean: float, std: float):
        if std == 0:
            raise DataError("Normalize needs a non-zero std")
        self.name, self.mean, self.std = name, mean, std

    def __call__(self, item):
        vals, shape = item.tensors[self.name]
        item.tensors[self.name] = ([(v - self.mean) / self.std for v in vals], shape)
        return item


class Scale(Transform):
    def __init__(self, name: str, factor: float):
        self.name, self.factor = name, factor

    def __call__(self, item):
        vals, shape = item.tensors[self.name]
        item.tensors[self.name] = ([v * self.factor for v in vals], shape)
        return item


class Lambda(Transform):
    def __init__(self, fn: Callable[[DataItem], DataItem]):
        self.fn = fn

    def __call__(self, item):
        return self.fn(item)


class TransformDataset(Dataset):
    def __init__(self, inner: Dataset, transform: Transform):
        self.inner, self.transform = inner, transform

    def __len__(self):
        return len(self.inner)

    def get(self, index):
        return self.transform(self.inner.get(index))


class Subset(Dataset):
    def __init__(self, inner: Dataset, indices: Sequence[int]):
        for i in indices:
            if not 0 <= i < len(inner):
                raise DataError(f"subset index {i} out of range")
        self.inner, self.idx = inner, list(indices)

    def __len__(self):
        return len(self.idx)

    def get(self, index):
        return self.inner.get(self.idx[index])


def random_split(dataset: Dataset, lengths: Sequence[int], seed: int = DATALOADER_DEFAULT_SEED) -> List[Subset]:
    if sum(lengths) != len(dataset):
        raise DataError("split lengths must sum to the dataset length")
    perm = SimpleRng(seed).shuffle(list(range(len(dataset))))
    out, off = [], 0
    for n in lengths:
        out.append(Subset(dataset, perm[off: off + n]))
        off += n
    return out
