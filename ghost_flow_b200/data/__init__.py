"""Datasets, loaders, samplers, transforms (ghostflow-data/src/*) and a synthetic token source.

``Dataset.get(i) -> (x, y)`` / ``len`` (dataset.rs:6-17), ``TensorDataset``, ``Subset``, ``ConcatDataset``,
``InMemoryDataset``; ``DataLoader(ds, batch_size).shuffle().drop_last().num_workers()`` builder
(dataloader.rs:9-151); ``SequentialSampler``, ``RandomSampler``, ``WeightedRandomSampler``, ``BatchSampler``
(sampler.rs:15-174); ``DistributedSampler`` / ``DistributedDataLoader`` with the reference's rank-contiguous
sharding where the last rank takes the remainder (ghostflow-ml/src/distributed.rs:233-307); transforms and
augmentations (transforms.rs:7-226, augmentation.rs:9-253); ``MNIST.load(dir)`` (IDX files) and
``CIFAR10.load(dir)`` (binary batches) (datasets.rs:13-280). Unlike the reference's ``thread_rng`` everywhere,
every random component takes a seed.
"""
from __future__ import annotations

import gzip
import os
import struct
from concurrent.futures import ThreadPoolExecutor

import torch


# ------------------------------------------------------------------------------------------- datasets
class Dataset:
    def get(self, index: int):
        raise NotImplementedError

    def len(self) -> int:
        raise NotImplementedError

    def __getitem__(self, i):
        return self.get(i)

    def __len__(self):
        return self.len()


class TensorDataset(Dataset):
    def __init__(self, data, targets):
        data = getattr(data, "data", data) if not isinstance(data, torch.Tensor) else data
        targets = getattr(targets, "data", targets) if not isinstance(targets, torch.Tensor) else targets
        assert data.shape[0] == targets.shape[0]
        self.data, self.targets = data, targets

    def get(self, i):
        return self.data[i], self.targets[i]

    def len(self):
        return self.data.shape[0]


InMemoryDataset = TensorDataset


class Subset(Dataset):
    def __init__(self, dataset, indices):
        self.dataset, self.indices = dataset, list(indices)

    def get(self, i):
        return self.dataset.get(self.indices[i])

    def len(self):
        return len(self.indices)


class ConcatDataset(Dataset):
    def __init__(self, datasets):
        self.datasets = list(datasets)
        self.offsets = [0]
        for d in self.datasets:
            self.offsets.append(self.offsets[-1] + len(d))

    def get(self, i):
        for k, d in enumerate(self.datasets):
            if i < self.offsets[k + 1]:
                return d.get(i - self.offsets[k])
        raise IndexError(i)

    def len(self):
        return self.offsets[-1]


class TransformedDataset(Dataset):
    def __init__(self, dataset, transform=None, target_transform=None):
        self.dataset, self.transform, self.target_transform = dataset, transform, target_transform

    def get(self, i):
        x, y = self.dataset.get(i)
        return (self.transform(x) if self.transform else x), (self.target_transform(y) if self.target_transform else y)

    def len(self):
        return len(self.dataset)


class SyntheticTokenDataset(Dataset):
    """Uniform random token ids of a fixed shape, reproducible per index; ``get`` returns (inputs, next-token targets)."""

    def __init__(self, vocab_size: int, seq_len: int, num_samples: int, seed: int = 0):
        self.vocab_size, self.seq_len, self.num_samples, self.seed = vocab_size, seq_len, num_samples, seed

    def get(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        t = torch.randint(0, self.vocab_size, (self.seq_len + 1,), generator=g)
        return t[:-1], t[1:]

    def len(self):
        return self.num_samples


# ------------------------------------------------------------------------------------------- samplers
class Sampler:
    """Base of the index samplers (the trait of ghostflow-data/src/sampler.rs:6-12): an iterable of dataset indices
    with a length."""

    def __iter__(self):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError

    def is_empty(self) -> bool:
        return len(self) == 0


class SequentialSampler(Sampler):
    def __init__(self, n: int):
        self.n = n

    def __iter__(self):
        return iter(range(self.n))

    def __len__(self):
        return self.n


class RandomSampler(Sampler):
    def __init__(self, n: int, seed: int = 0, replacement: bool = False, num_samples: int | None = None):
        self.n, self.seed, self.replacement, self.num_samples = n, seed, replacement, num_samples or n
        self.epoch = 0

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        if self.replacement:
            return iter(torch.randint(0, self.n, (self.num_samples,), generator=g).tolist())
        return iter(torch.randperm(self.n, generator=g)[: self.num_samples].tolist())

    def __len__(self):
        return self.num_samples


class WeightedRandomSampler(Sampler):
    def __init__(self, weights, num_samples: int, replacement: bool = True, seed: int = 0):
        self.weights = torch.as_tensor(weights, dtype=torch.float64)
        self.num_samples, self.replacement, self.seed = num_samples, replacement, seed

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed)
        return iter(torch.multinomial(self.weights, self.num_samples, self.replacement, generator=g).tolist())

    def __len__(self):
        return self.num_samples


class BatchSampler:
    def __init__(self, sampler, batch_size: int, drop_last: bool = False):
        self.sampler, self.batch_size, self.drop_last = sampler, batch_size, drop_last

    def __iter__(self):
        batch = []
        for i in self.sampler:
            batch.append(i)
            if len(batch) == self.batch_size:
                yield batch
                batch = []
        if batch and not self.drop_last:
            yield batch

    def __len__(self):
        n = len(self.sampler)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size


class DistributedSampler(Sampler):
    """Rank ``r`` of ``world`` gets the contiguous slice ``[r * n // world ...)``; the last rank takes the
    remainder (the reference's rule). ``even=True`` instead pads so that every rank gets the same count."""

    def __init__(self, n: int, world_size: int, rank: int, shuffle: bool = False, seed: int = 0, even: bool = False):
        self.n, self.world_size, self.rank, self.shuffle, self.seed, self.even = n, world_size, rank, shuffle, seed, even
        self.epoch = 0

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def _indices(self):
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self.epoch)
            order = torch.randperm(self.n, generator=g).tolist()
        else:
            order = list(range(self.n))
        if self.even:
            per = (self.n + self.world_size - 1) // self.world_size
            order = (order + order[: per * self.world_size - self.n])
            return order[self.rank * per:(self.rank + 1) * per]
        per = self.n // self.world_size
        lo = self.rank * per
        hi = self.n if self.rank == self.world_size - 1 else lo + per
        return order[lo:hi]

    def __iter__(self):
        return iter(self._indices())

    def __len__(self):
        return len(self._indices())


# ------------------------------------------------------------------------------------------- loader
def collate_batch(samples):
    """Stacks a list of ``(x, y)`` pairs into batched tensors."""
    xs, ys = zip(*samples)
    xs = [x.data if hasattr(x, "data") and not isinstance(x, torch.Tensor) else x for x in xs]
    ys = [torch.as_tensor(y.data if hasattr(y, "data") and not isinstance(y, torch.Tensor) else y) for y in ys]
    return torch.stack([torch.as_tensor(x) for x in xs]), torch.stack(ys)


class DataLoaderIter:
    """Iterator over the batches of one epoch (ghostflow-data/src/dataloader.rs:72-110): ``next()`` yields
    ``(inputs, targets)``; ``current_batch`` counts what has been handed out, ``len()`` what is left."""

    def __init__(self, loader: "DataLoader"):
        self.loader = loader
        self.current_batch = 0
        self._total = len(loader)
        self._gen = loader._batches()

    def __iter__(self):
        return self

    def __next__(self):
        item = next(self._gen)
        self.current_batch += 1
        return item

    def __len__(self):
        return max(0, self._total - self.current_batch)


class DataLoader:
    def __init__(self, dataset, batch_size: int = 1, shuffle: bool = False, drop_last: bool = False,
                 num_workers: int = 0, sampler=None, seed: int = 0, pin_memory: bool = False, collate_fn=None):
        self.dataset, self.batch_size = dataset, batch_size
        self._shuffle, self._drop_last, self._workers = shuffle, drop_last, num_workers
        self.sampler, self.seed, self.pin_memory = sampler, seed, pin_memory
        self.collate_fn = collate_fn or collate_batch
        self.epoch = 0

    @classmethod
    def new(cls, *args, **kwargs):
        return cls(*args, **kwargs)

    # builder methods of the reference
    def shuffle(self, v: bool = True):
        self._shuffle = v
        return self

    def drop_last(self, v: bool = True):
        self._drop_last = v
        return self

    def num_workers(self, n: int):
        self._workers = n
        return self

    def __len__(self):
        n = len(self.sampler) if self.sampler is not None else len(self.dataset)
        return n // self.batch_size if self._drop_last else (n + self.batch_size - 1) // self.batch_size

    def __iter__(self):
        return DataLoaderIter(self)

    def _batches(self):
        if self.sampler is not None:
            sampler = self.sampler
            if hasattr(sampler, "set_epoch"):
                sampler.set_epoch(self.epoch)
        elif self._shuffle:
            sampler = RandomSampler(len(self.dataset), self.seed)
            sampler.set_epoch(self.epoch)
        else:
            sampler = SequentialSampler(len(self.dataset))
        self.epoch += 1
        pool = ThreadPoolExecutor(self._workers) if self._workers > 0 else None
        try:
            for idxs in BatchSampler(sampler, self.batch_size, self._drop_last):
                samples = list(pool.map(self.dataset.get, idxs)) if pool else [self.dataset.get(i) for i in idxs]
                x, y = self.collate_fn(samples)
                if self.pin_memory and torch.cuda.is_available():
                    x, y = x.pin_memory(), y.pin_memory()
                yield x, y
        finally:
            if pool:
                pool.shutdown()


class DistributedDataLoader(DataLoader):
    """``DistributedDataLoader(dataset, batch_size, world_size, rank)``: each rank iterates its own shard."""

    def __init__(self, dataset, batch_size: int, world_size: int, rank: int, shuffle: bool = False, seed: int = 0,
                 **kw):
        super().__init__(dataset, batch_size, sampler=DistributedSampler(len(dataset), world_size, rank, shuffle, seed),
                         **kw)
        self.world_size, self.rank = world_size, rank


# ------------------------------------------------------------------------------------------- transforms
class Transform:
    """Base of the transforms (the trait of ghostflow-data/src/transforms.rs:6-9): ``apply(tensor) -> tensor``;
    calling the object does the same."""

    def apply(self, x):
        return self(x)

    def __call__(self, x):
        raise NotImplementedError


class Compose(Transform):
    def __init__(self, transforms):
        self.transforms = list(transforms)

    def __call__(self, x):
        for t in self.transforms:
            x = t(x)
        return x


class ToTensor(Transform):
    """uint8 ``[H, W, C]`` (or ``[H, W]``) image -> float ``[C, H, W]`` in [0, 1]."""

    def __call__(self, x):
        t = torch.as_tensor(x)
        if t.dtype == torch.uint8:
            t = t.float() / 255.0
        if t.dim() == 2:
            t = t[None]
        elif t.dim() == 3 and t.shape[-1] in (1, 3, 4) and t.shape[0] not in (1, 3, 4):
            t = t.permute(2, 0, 1)
        return t.float()


class Normalize(Transform):
    def __init__(self, mean, std):
        self.mean, self.std = torch.as_tensor(mean, dtype=torch.float32), torch.as_tensor(std, dtype=torch.float32)

    @classmethod
    def imagenet(cls):
        return cls([0.485, 0.456, 0.406], [0.229, 0.224, 0.225])

    def __call__(self, x):
        return (x - self.mean.view(-1, 1, 1)) / self.std.view(-1, 1, 1)


class _Random(Transform):
    def __init__(self, seed: int = 0):
        self.gen = torch.Generator().manual_seed(seed)

    def _u(self):
        return float(torch.rand(1, generator=self.gen))

    def _i(self, hi):
        return int(torch.randint(0, max(1, hi), (1,), generator=self.gen))


class RandomHorizontalFlip(_Random):
    def __init__(self, p: float = 0.5, seed: int = 0):
        super().__init__(seed)
        self.p = p

    def __call__(self, x):
        return x.flip(-1) if self._u() < self.p else x


class RandomVerticalFlip(RandomHorizontalFlip):
    def __call__(self, x):
        return x.flip(-2) if self._u() < self.p else x


class RandomCrop(_Random):
    def __init__(self, size, padding: int = 0, seed: int = 0):
        super().__init__(seed)
        self.size = (size, size) if isinstance(size, int) else tuple(size)
        self.padding = padding

    def __call__(self, x):
        if self.padding:
            x = torch.nn.functional.pad(x, [self.padding] * 4)
        h, w = self.size
        top, left = self._i(x.shape[-2] - h + 1), self._i(x.shape[-1] - w + 1)
        return x[..., top:top + h, left:left + w]


class RandomRotation(_Random):
    """Rotation by a random multiple of 90 degrees, or by a random angle in ``[-degrees, degrees]`` (bilinear)."""

    def __init__(self, degrees: float = 90.0, seed: int = 0):
        super().__init__(seed)
        self.degrees = degrees

    def __call__(self, x):
        import math

        a = math.radians((self._u() * 2 - 1) * self.degrees)
        theta = torch.tensor([[math.cos(a), -math.sin(a), 0.0], [math.sin(a), math.cos(a), 0.0]])[None]
        xb = x[None] if x.dim() == 3 else x
        grid = torch.nn.functional.affine_grid(theta.expand(xb.shape[0], -1, -1), list(xb.shape), align_corners=False)
        y = torch.nn.functional.grid_sample(xb, grid, align_corners=False)
        return y[0] if x.dim() == 3 else y


class RandomErasing(_Random):
    def __init__(self, p: float = 0.5, scale=(0.02, 0.33), value: float = 0.0, seed: int = 0):
        super().__init__(seed)
        self.p, self.scale, self.value = p, scale, value

    def __call__(self, x):
        if self._u() >= self.p:
            return x
        H, W = x.shape[-2:]
        area = (self.scale[0] + self._u() * (self.scale[1] - self.scale[0])) * H * W
        h = max(1, min(H, int(round(area ** 0.5))))
        w = max(1, min(W, int(round(area / h))))
        top, left = self._i(H - h + 1), self._i(W - w + 1)
        x = x.clone()
        x[..., top:top + h, left:left + w] = self.value
        return x


# ------------------------------------------------------------------------------------------- file datasets
def _open_maybe_gz(path):
    if os.path.exists(path):
        return open(path, "rb")
    if os.path.exists(path + ".gz"):
        return gzip.open(path + ".gz", "rb")
    raise FileNotFoundError(path)


class MNIST(TensorDataset):
    """IDX files ``{train,t10k}-images-idx3-ubyte`` / ``-labels-idx1-ubyte`` (optionally .gz) in ``root``."""

    @classmethod
    def load(cls, root: str, train: bool = True, normalize: bool = True):
        prefix = "train" if train else "t10k"
        with _open_maybe_gz(os.path.join(root, f"{prefix}-images-idx3-ubyte")) as f:
            magic, n, h, w = struct.unpack(">IIII", f.read(16))
            if magic != 2051:
                raise IOError("bad MNIST image file magic")
            imgs = torch.frombuffer(bytearray(f.read(n * h * w)), dtype=torch.uint8).view(n, 1, h, w)
        with _open_maybe_gz(os.path.join(root, f"{prefix}-labels-idx1-ubyte")) as f:
            magic, n2 = struct.unpack(">II", f.read(8))
            if magic != 2049 or n2 != n:
                raise IOError("bad MNIST label file")
            labels = torch.frombuffer(bytearray(f.read(n)), dtype=torch.uint8).long()
        x = imgs.float() / 255.0 if normalize else imgs.float()
        return cls(x, labels)


class CIFAR10(TensorDataset):
    """Binary batches ``data_batch_{1..5}.bin`` / ``test_batch.bin``: records of 1 label byte + 3072 pixel bytes."""

    @classmethod
    def load(cls, root: str, train: bool = True, normalize: bool = True):
        files = [f"data_batch_{i}.bin" for i in range(1, 6)] if train else ["test_batch.bin"]
        xs, ys = [], []
        for name in files:
            raw = torch.frombuffer(bytearray(open(os.path.join(root, name), "rb").read()), dtype=torch.uint8)
            rec = raw.view(-1, 3073)
            ys.append(rec[:, 0].long())
            xs.append(rec[:, 1:].view(-1, 3, 32, 32))
        x = torch.cat(xs).float()
        return cls(x / 255.0 if normalize else x, torch.cat(ys))
