"""``paddle.io``: datasets, samplers and ``DataLoader`` (python/paddle/io/reader.py, dataloader/*).  The
multi-process worker pool, shared-memory transport and pinned-memory staging are PyTorch's; this module
supplies Paddle's classes, collate rules and ``DistributedBatchSampler`` (batch_sampler.py)."""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.utils.data as tud

from .._core.tensor import as_tensor, to_tensor

Dataset = tud.Dataset
IterableDataset = tud.IterableDataset
Sampler = tud.Sampler
SequenceSampler = tud.SequentialSampler
RandomSampler = tud.RandomSampler
WeightedRandomSampler = tud.WeightedRandomSampler
Subset = tud.Subset
ConcatDataset = tud.ConcatDataset
ChainDataset = tud.ChainDataset
get_worker_info = tud.get_worker_info


class TensorDataset(Dataset):
    def __init__(self, tensors):
        self.tensors = list(tensors)

    def __getitem__(self, i):
        return tuple(t[i] for t in self.tensors)

    def __len__(self):
        return self.tensors[0].shape[0]


class ComposeDataset(Dataset):
    def __init__(self, datasets):
        self.datasets = list(datasets)

    def __len__(self):
        return len(self.datasets[0])

    def __getitem__(self, i):
        out = []
        for d in self.datasets:
            s = d[i]
            out.extend(s if isinstance(s, (tuple, list)) else [s])
        return tuple(out)


def random_split(dataset, lengths, generator=None):
    return tud.random_split(dataset, lengths, generator=generator)


class BatchSampler(Sampler):
    def __init__(self, dataset=None, sampler=None, shuffle=False, batch_size=1, drop_last=False):
        self.sampler = sampler if sampler is not None else (RandomSampler(dataset) if shuffle else SequenceSampler(dataset))
        self.batch_size, self.drop_last = batch_size, drop_last

    def __iter__(self):
        batch = []
        for idx in self.sampler:
            batch.append(idx)
            if len(batch) == self.batch_size:
                yield batch
                batch = []
        if batch and not self.drop_last:
            yield batch

    def __len__(self):
        n = len(self.sampler)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size


class DistributedBatchSampler(BatchSampler):
    """Each rank iterates over its own 1/nranks slice of the (optionally shuffled, padded) index list
    (python/paddle/io/dataloader/batch_sampler.py ``DistributedBatchSampler``)."""

    def __init__(self, dataset, batch_size, num_replicas=None, rank=None, shuffle=False, drop_last=False):
        from ..distributed import get_rank, get_world_size
        self.dataset = dataset
        self.batch_size, self.drop_last, self.shuffle = batch_size, drop_last, shuffle
        self.nranks = num_replicas if num_replicas is not None else get_world_size()
        self.local_rank = rank if rank is not None else get_rank()
        self.epoch = 0
        self.num_samples = int(math.ceil(len(dataset) / self.nranks))
        self.total_size = self.num_samples * self.nranks

    def __iter__(self):
        n = len(self.dataset)
        indices = np.arange(n).tolist()
        indices += indices[:self.total_size - n]
        if self.shuffle:
            np.random.RandomState(self.epoch).shuffle(indices)
            self.epoch += 1
        # contiguous blocks of batch_size per rank, as the reference does
        sub = []
        for i in range(self.local_rank * self.batch_size, len(indices) - (len(indices) % (self.batch_size * self.nranks)),
                       self.batch_size * self.nranks):
            sub.extend(indices[i:i + self.batch_size])
        tail = indices[len(indices) - (len(indices) % (self.batch_size * self.nranks)):]
        per = len(tail) // self.nranks
        sub.extend(tail[self.local_rank * per:(self.local_rank + 1) * per])
        batch = []
        for idx in sub:
            batch.append(idx)
            if len(batch) == self.batch_size:
                yield batch
                batch = []
        if batch and not self.drop_last:
            yield batch

    def __len__(self):
        return self.num_samples // self.batch_size if self.drop_last else (self.num_samples + self.batch_size - 1) // self.batch_size

    def set_epoch(self, epoch):
        self.epoch = epoch


def default_collate_fn(batch):
    sample = batch[0]
    if isinstance(sample, torch.Tensor):
        return as_tensor(torch.stack([b.as_subclass(torch.Tensor) if type(b) is not torch.Tensor else b for b in batch]))
    if isinstance(sample, np.ndarray):
        return to_tensor(np.stack(batch))
    if isinstance(sample, (int, np.integer)):
        return to_tensor(np.asarray(batch, dtype=np.int64))
    if isinstance(sample, (float, np.floating)):
        return to_tensor(np.asarray(batch, dtype=np.float32))
    if isinstance(sample, (str, bytes)):
        return list(batch)
    if isinstance(sample, dict):
        return {k: default_collate_fn([b[k] for b in batch]) for k in sample}
    if isinstance(sample, (tuple, list)):
        return [default_collate_fn(list(s)) for s in zip(*batch)]
    raise TypeError(f"cannot collate {type(sample)}")


class DataLoader:
    def __init__(self, dataset, feed_list=None, places=None, return_list=True, batch_sampler=None, batch_size=1,
                 shuffle=False, drop_last=False, collate_fn=None, num_workers=0, use_buffer_reader=True,
                 prefetch_factor=2, use_shared_memory=True, timeout=0, worker_init_fn=None, persistent_workers=False):
        self.dataset, self.batch_sampler = dataset, batch_sampler
        kw = dict(num_workers=num_workers, collate_fn=collate_fn or default_collate_fn, timeout=timeout,
                  worker_init_fn=worker_init_fn, pin_memory=use_buffer_reader and torch.cuda.is_available())
        if num_workers > 0:
            kw.update(prefetch_factor=prefetch_factor, persistent_workers=persistent_workers)
        if isinstance(dataset, tud.IterableDataset):
            self._loader = tud.DataLoader(dataset, batch_size=batch_size, drop_last=drop_last, **kw)
        elif batch_sampler is not None:
            self._loader = tud.DataLoader(dataset, batch_sampler=batch_sampler, **kw)
        elif batch_size is None:
            self._loader = tud.DataLoader(dataset, batch_size=None, shuffle=shuffle, **kw)
        else:
            self._loader = tud.DataLoader(dataset, batch_size=batch_size, shuffle=shuffle, drop_last=drop_last, **kw)

    def __iter__(self):
        from .._core.dtype import default_device
        from ..profiler.timer import benchmark
        from ..profiler.utils import RecordEvent, in_profiler_mode
        from ..profiler.profiler_statistic import TracerEventType
        dev = default_device()
        bench = benchmark()
        bench.check_if_need_record(self)
        it = iter(self._loader)
        while True:
            # reader cost of the throughput timer, and a Dataloader range in a running profile
            bench.before_reader()
            rng = RecordEvent("Dataloader#next", TracerEventType.Dataloader) if in_profiler_mode() else None
            if rng is not None:
                rng.begin()
            try:
                batch = next(it)
            except StopIteration:
                return
            finally:
                if rng is not None:
                    rng.end()
            batch = _move(batch, dev)
            bench.after_reader()
            yield batch

    def __len__(self):
        return len(self._loader)

    def __call__(self):
        return self.__iter__()


def _move(b, dev):
    if isinstance(b, torch.Tensor):
        return as_tensor(b.to(dev, non_blocking=True)) if dev.type == "cuda" else as_tensor(b)
    if isinstance(b, dict):
        return {k: _move(v, dev) for k, v in b.items()}
    if isinstance(b, (list, tuple)):
        return type(b)(_move(v, dev) for v in b)
    return b


class SubsetRandomSampler(Sampler):
    """Samples the given indices in random order, without replacement (io/dataloader/sampler.py)."""

    def __init__(self, indices):
        if len(indices) == 0:
            raise ValueError("The length of `indices` in SubsetRandomSampler should be greater than 0.")
        self.indices = list(indices)

    def __iter__(self):
        import torch
        for i in torch.randperm(len(self.indices)).tolist():
            yield self.indices[i]

    def __len__(self):
        return len(self.indices)
