"""``paddle.distributed.save_state_dict`` (python/paddle/distributed/checkpoint/save_state_dict.py:135): every
rank writes ``{rank}_{unique_id}.distcp`` with its local shards (replicated copies are written once, by the lowest
holder, :107-132) and the coordinator writes ``{unique_id}.metadata`` describing every shard of every tensor."""
from __future__ import annotations

import multiprocessing as mp
import os

import torch

from ...framework.io import save as _save
from .. import collective as C
from .metadata import LocalTensorIndex, LocalTensorMetadata, Metadata
from .utils import describe, flatten_state_dict

_async_procs = []


def _dtype_name(dt):
    return str(dt).replace("torch.", "")


def _unique_id(path):
    ids = [int(f.split(".")[0]) for f in os.listdir(path) if f.endswith(".metadata") and f.split(".")[0].isdigit()]
    return max(ids) + 1 if ids else 0


def file_crc32(fn):
    import zlib
    crc, size = 0, 0
    with open(fn, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            crc = zlib.crc32(chunk, crc)
            size += len(chunk)
    return crc & 0xFFFFFFFF, size


def _write(obj, fn):
    """Writes the shard, then a ``<shard>.crc`` side file (``crc32 size``) that the loader checks: a truncated or
    bit-flipped shard is reported by name instead of surfacing as a wrong tensor or an unpickling error."""
    _save(obj, fn)
    crc, size = file_crc32(fn)
    with open(fn + ".crc", "w") as f:
        f.write(f"{crc:08x} {size}\n")


def save_state_dict(state_dict, path, process_group=None, coordinator_rank=0, unique_id=None, async_save=False):
    assert isinstance(state_dict, dict), "The state_dict should be a dictionary."
    os.makedirs(path, exist_ok=True)
    flat, mapping = flatten_state_dict(state_dict)
    rank = C.get_rank() if C.is_initialized() else 0
    world = C.get_world_size() if C.is_initialized() else 1
    if unique_id is None:
        uid = [_unique_id(path)] if rank == coordinator_rank else [None]
        if world > 1:
            C.broadcast_object_list(uid, coordinator_rank, process_group)
        unique_id = uid[0]
    file_name = f"{rank}_{unique_id}.distcp"
    local_meta, to_write = {}, {}
    for key, v in flat.items():
        d = describe(v)
        if d is None:
            if not isinstance(v, torch.Tensor) and rank == coordinator_rank:
                to_write[key] = v                      # plain python values (scheduler state ...) written once
                local_meta[key] = ("obj", (), (), "object", 0)
            continue
        local, gshape, lshape, off, replica = d
        local_meta[key] = ("tensor", off, lshape, _dtype_name(local.dtype), replica)
        to_write[key] = local
    gathered = [None] * world
    if world > 1:
        C.all_gather_object(gathered, local_meta, process_group)
    else:
        gathered = [local_meta]
    # dedup: for each (key, offset) the lowest rank among the holders with the smallest replica id writes
    owner = {}
    for r, metas in enumerate(gathered):
        for key, (kind, off, lshape, dt, replica) in metas.items():
            cur = owner.get((key, off))
            if cur is None or (replica, r) < (cur[0], cur[1]):
                owner[(key, off)] = (replica, r, lshape, dt, kind)
    mine = {key: v for key, v in to_write.items() if owner[(key, local_meta[key][1])][1] == rank}
    if rank == coordinator_rank:
        md = Metadata()
        for (key, off), (replica, r, lshape, dt, kind) in sorted(owner.items(), key=lambda kv: (kv[0][0], kv[0][1])):
            md.state_dict_metadata.setdefault(key, []).append(LocalTensorMetadata(off, lshape, dt))
            md.storage_metadata[LocalTensorIndex(key, off)] = f"{r}_{unique_id}.distcp"
        md.flat_mapping = mapping
        _write(md, os.path.join(path, f"{unique_id}.metadata"))
    payload = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in mine.items()}
    if async_save:
        ctx = mp.get_context("spawn")
        p = ctx.Process(target=_write, args=(payload, os.path.join(path, file_name)))
        p.start()
        _async_procs.append(p)
    else:
        _write(payload, os.path.join(path, file_name))
    if world > 1:
        C.barrier(process_group)


def wait_async_save():
    while _async_procs:
        _async_procs.pop().join()
