"""Slot-file datasets (python/paddle/distributed/fleet/dataset/dataset.py ``InMemoryDataset`` / ``QueueDataset``).

Files hold one example per line in the multi-slot format ``<n> v1 .. vn <m> w1 .. wm ...`` (one group per variable
passed to ``init(use_var=...)``), optionally produced by piping each file through ``pipe_command``.  Iterating a
dataset yields feed dicts ``{var.name: ndarray [batch, n]}`` that ``static.Executor.train_from_dataset`` consumes."""
from __future__ import annotations

import random
import subprocess

import numpy as np


class DatasetBase:
    def __init__(self):
        self.batch_size, self.thread_num, self.use_var, self.pipe_command = 1, 1, [], "cat"
        self.filelist, self.input_type, self.fs_name, self.fs_ugi = [], 0, "", ""

    def init(self, batch_size=1, thread_num=1, use_var=None, pipe_command="cat", input_type=0, fs_name="", fs_ugi="",
             download_cmd="cat", **kwargs):
        self.batch_size, self.thread_num, self.use_var = batch_size, thread_num, list(use_var or [])
        self.pipe_command, self.input_type = pipe_command, input_type

    _init_distributed_settings = update_settings = lambda self, **kw: self.__dict__.update(kw)

    def set_filelist(self, filelist):
        self.filelist = list(filelist)

    def _lines(self, path):
        if self.pipe_command in ("cat", "", None):
            with open(path) as f:
                yield from f
        else:
            with open(path, "rb") as f:
                out = subprocess.run(self.pipe_command, shell=True, stdin=f, capture_output=True, check=True).stdout
            yield from out.decode().splitlines()

    def _parse(self, line):
        toks = line.split()
        rec, i = [], 0
        for var in self.use_var:
            n = int(toks[i])
            vals = toks[i + 1:i + 1 + n]
            i += 1 + n
            kind = str(getattr(var, "dtype", "int64"))
            rec.append(np.asarray(vals, dtype=np.float32 if "float" in kind else np.int64))
        return rec

    def _records(self):
        for path in self.filelist:
            for line in self._lines(path):
                if line.strip():
                    yield self._parse(line)

    def _batches(self, records):
        buf = []
        for r in records:
            buf.append(r)
            if len(buf) == self.batch_size:
                yield self._collate(buf)
                buf = []
        if buf:
            yield self._collate(buf)

    def _collate(self, recs):
        out = {}
        for j, var in enumerate(self.use_var):
            width = max(len(r[j]) for r in recs)
            arr = np.zeros((len(recs), width), dtype=recs[0][j].dtype)
            for i, r in enumerate(recs):
                arr[i, :len(r[j])] = r[j]
            out[var.name] = arr
        return out


class QueueDataset(DatasetBase):
    """Streams the files in order, nothing is held in memory."""

    def __iter__(self):
        return self._batches(self._records())


class InMemoryDataset(DatasetBase):
    def __init__(self):
        super().__init__()
        self._data = None

    def load_into_memory(self, is_shuffle=False):
        self._data = list(self._records())
        if is_shuffle:
            self.local_shuffle()

    def preload_into_memory(self, thread_num=None):
        self.load_into_memory()

    def wait_preload_done(self):
        pass

    def local_shuffle(self):
        random.shuffle(self._data)

    def global_shuffle(self, fleet=None, thread_num=12):
        """Every worker ends up with a random 1/n of all examples: examples are exchanged with an object
        all-gather and each worker keeps those whose shuffled position maps to its rank."""
        import torch.distributed as tdist
        if not (tdist.is_available() and tdist.is_initialized()) or tdist.get_world_size() == 1:
            return self.local_shuffle()
        parts = [None] * tdist.get_world_size()
        tdist.all_gather_object(parts, self._data)
        everything = [r for p in parts for r in p]
        random.Random(len(everything)).shuffle(everything)
        self._data = everything[tdist.get_rank()::tdist.get_world_size()]

    def release_memory(self):
        self._data = None

    def get_memory_data_size(self, fleet=None):
        return len(self._data or [])

    get_shuffle_data_size = get_memory_data_size

    def slots_shuffle(self, slots):
        names = [v.name for v in self.use_var]
        for s in slots:
            j = names.index(s)
            col = [r[j] for r in self._data]
            random.shuffle(col)
            for r, c in zip(self._data, col):
                r[j] = c

    def __iter__(self):
        if self._data is None:
            self.load_into_memory()
        return self._batches(iter(self._data))
