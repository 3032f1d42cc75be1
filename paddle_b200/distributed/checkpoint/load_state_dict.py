"""``paddle.distributed.load_state_dict`` (python/paddle/distributed/checkpoint/load_state_dict.py:526): read the
metadata files, intersect every wanted local shard with the saved chunks (``compute_overlap`` :394, ``ReadItem``
:43), copy the overlaps.  The target may live on a different mesh / placement than the one that saved.  Files
are on a shared directory here, so each rank reads the chunks it needs itself instead of receiving them from
the rank that wrote them."""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from ...framework.io import load as _load
from .. import collective as C
from .utils import describe, flatten_state_dict


@dataclass(frozen=True)
class ReadItem:
    tensor_key: str
    file_name: str
    src_global_offset: tuple
    cur_offset: tuple      # offset inside the target's local tensor
    storage_offset: tuple  # offset inside the saved chunk
    lengths: tuple


class CheckpointCorruptError(RuntimeError):
    """A checkpoint shard does not match the checksum written next to it, or cannot be decoded."""


def _load_verified(fn):
    side = fn + ".crc"
    if os.path.exists(side):
        from .save_state_dict import file_crc32
        want_crc, want_size = open(side).read().split()
        crc, size = file_crc32(fn)
        if size != int(want_size) or crc != int(want_crc, 16):
            raise CheckpointCorruptError(
                f"checkpoint shard {fn} is corrupt: size {size} / crc {crc:08x}, expected {want_size} / {want_crc}")
    try:
        return _load(fn)
    except CheckpointCorruptError:
        raise
    except Exception as e:  # noqa: BLE001 - any decoding failure of a shard is a corrupt checkpoint
        raise CheckpointCorruptError(f"checkpoint shard {fn} cannot be decoded: {type(e).__name__}: {e}") from e


def compute_overlap(cur_offset, cur_shape, src_offset, src_shape):
    cur_off, src_off, lengths = [], [], []
    for co, cs, so, ss in zip(cur_offset, cur_shape, src_offset, src_shape):
        lo, hi = max(co, so), min(co + cs, so + ss)
        if hi <= lo:
            return None
        cur_off.append(lo - co), src_off.append(lo - so), lengths.append(hi - lo)
    return tuple(cur_off), tuple(src_off), tuple(lengths)


def get_max_id(path):
    """Newest checkpoint version under ``path``: the largest numeric id among ``{id}.metadata`` /
    ``{rank}_{id}.distcp`` files (python/paddle/distributed/checkpoint/utils.py:124).  Ids are compared as
    integers: a lexicographic order would put version 9 after version 10."""
    ids = []
    for f in os.listdir(path):
        stem, dot, ext = f.rpartition(".")
        if ext == "metadata" and stem.isdigit():
            ids.append(int(stem))
        elif ext == "distcp":
            tail = stem.rpartition("_")[2]
            if tail.isdigit():
                ids.append(int(tail))
    return max(ids) if ids else None


def _agree_on_id(unique_id, process_group, coordinator_rank=0):
    """Every rank must read the same version: the coordinator's choice is broadcast (a periodic save that is running
    while a late rank lists the directory would otherwise let ranks pick different ids;
    python/paddle/distributed/checkpoint/utils.py:135 ``check_unique_id``)."""
    if C.is_initialized() and C.get_world_size() > 1:
        box = [unique_id]
        ranks = getattr(process_group, "ranks", None)
        src = ranks[coordinator_rank] if ranks else coordinator_rank
        C.broadcast_object_list(box, src=src, group=process_group)
        return box[0]
    return unique_id


def _metadata_files(path, unique_id=None):
    """The metadata of ONE checkpoint version: ``unique_id`` or, when it is None, the newest one under ``path``
    (load_state_dict.py:590,871 use ``get_max_id``).  Metadata files whose name is not a number (hand-made merges)
    are only read when no numbered version exists."""
    if unique_id is None:
        unique_id = get_max_id(path)
    if unique_id is not None:
        files = [f"{unique_id}.metadata"]
        assert os.path.exists(os.path.join(path, files[0])), f"no {files[0]} under {path}"
    else:
        files = sorted(f for f in os.listdir(path) if f.endswith(".metadata"))
    assert files, f"no .metadata file under {path}"
    return [_load_verified(os.path.join(path, f)) for f in files]


def get_read_items(path, flat, metas):
    items = []
    for key, v in flat.items():
        d = describe(v)
        if d is None:
            continue
        _, _, lshape, off, _ = d
        found = False
        for md in metas:
            for chunk in md.state_dict_metadata.get(key, []):
                from .metadata import LocalTensorIndex
                if chunk.dtype == "object":
                    continue
                ov = compute_overlap(off, lshape, chunk.global_offset, chunk.local_shape)
                if ov is None and len(lshape) > 0:
                    continue
                ov = ov or ((), (), ())
                fn = md.storage_metadata[LocalTensorIndex(key, tuple(chunk.global_offset))]
                items.append(ReadItem(key, fn, tuple(chunk.global_offset), ov[0], ov[1], ov[2]))
                found = True
        if not found:
            raise KeyError(f"'{key}' is not in the checkpoint under {path}")
    return items


def load_state_dict(state_dict, path, process_group=None, coordinator_rank=0, unique_id=None, offload=False):
    """Fills the tensors of ``state_dict`` in place."""
    assert isinstance(state_dict, dict)
    flat, _ = flatten_state_dict(state_dict)
    if unique_id is None:
        unique_id = _agree_on_id(get_max_id(path), process_group, coordinator_rank)
    metas = _metadata_files(path, unique_id)
    items = get_read_items(path, flat, metas)
    cache = {}
    with torch.no_grad():
        for it in items:
            if it.file_name not in cache:
                cache[it.file_name] = _load_verified(os.path.join(path, it.file_name))
            src = cache[it.file_name][it.tensor_key].as_subclass(torch.Tensor)
            dst = describe(flat[it.tensor_key])[0]
            s_idx = tuple(slice(o, o + n) for o, n in zip(it.storage_offset, it.lengths))
            d_idx = tuple(slice(o, o + n) for o, n in zip(it.cur_offset, it.lengths))
            dst[d_idx].copy_(src[s_idx].to(dst.dtype)) if d_idx else dst.copy_(src.to(dst.dtype))
    # plain python entries are returned through the dict itself
    for md in metas:
        for key, chunks in md.state_dict_metadata.items():
            if chunks and chunks[0].dtype == "object" and key in flat and not isinstance(flat[key], torch.Tensor):
                from .metadata import LocalTensorIndex
                fn = md.storage_metadata[LocalTensorIndex(key, ())]
                if fn not in cache:
                    cache[fn] = _load_verified(os.path.join(path, fn))
                _assign(state_dict, md.flat_mapping.get(key, (key,)), cache[fn][key])
    if C.is_initialized() and C.get_world_size() > 1:
        C.barrier(process_group)


def _assign(d, path, value):
    for p in path[:-1]:
        d = d[p]
    d[path[-1]] = value


def load_merged_state_dict(path, prefix=None, unique_id=None, offload=False):
    """Reassemble every tensor of the checkpoint in full on this rank (load_state_dict.py:830)."""
    metas = _metadata_files(path, unique_id)
    from .metadata import LocalTensorIndex
    out, cache = {}, {}
    for md in metas:
        for key, chunks in md.state_dict_metadata.items():
            if prefix is not None and not key.startswith(prefix):
                continue
            if chunks[0].dtype == "object":
                continue
            gshape = [max(c.global_offset[i] + c.local_shape[i] for c in chunks) for i in range(len(chunks[0].local_shape))]
            full = None
            for c in chunks:
                fn = md.storage_metadata[LocalTensorIndex(key, tuple(c.global_offset))]
                if fn not in cache:
                    cache[fn] = _load_verified(os.path.join(path, fn))
                src = cache[fn][key].as_subclass(torch.Tensor)
                if full is None:
                    full = torch.zeros(gshape, dtype=src.dtype)
                idx = tuple(slice(o, o + n) for o, n in zip(c.global_offset, c.local_shape))
                if idx:
                    full[idx] = src
                else:
                    full = src.clone()
            from ..._core.tensor import as_tensor
            out[key] = as_tensor(full)
    return out
