"""``paddle.save`` / ``paddle.load`` with the reference's on-disk layout (python/paddle/framework/io.py).

* A *state dict* (every value a Tensor, or a nested dict free of Tensors) is pickled as
  ``{structured_name: numpy.ndarray, ..., "StructuredToParameterName@@": {structured_name: param.name}}``
  (``_build_saved_state_dict``, io.py:163-183).  bf16 is stored as a ``uint16`` array.  With pickle
  protocol 2/3 arrays above ``(2**30-1)/itemsize`` elements are split into ``key@@.i`` slices listed
  under ``"UnpackBigParamInfor@@"`` (io_utils.py:234-273); the default protocol 4 never splits.
* Any other object (e.g. an optimizer state dict whose ``master_weights`` holds Tensors) goes through
  a pickler whose dispatch table reduces each Tensor to the tuple ``(name, ndarray)`` (``_pickle_save``,
  io.py:413-492); ``load`` turns such tuples back into Tensors carrying that name.
"""
from __future__ import annotations

import collections
import copyreg
import io as _io
import math
import os
import pickle
import threading

import numpy as np
import torch

from .._core.tensor import EagerParamBase, Tensor, as_tensor, to_tensor

_NAME_TABLE = "StructuredToParameterName@@"
_UNPACK_INFO = "UnpackBigParamInfor@@"


def _to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()
    return t.contiguous().numpy().copy() if t.is_contiguous() else np.ascontiguousarray(t.numpy())


def _contain_tensor(obj) -> bool:
    if isinstance(obj, torch.Tensor):
        return True
    if isinstance(obj, dict):
        return any(_contain_tensor(v) for v in obj.values())
    if isinstance(obj, (list, tuple)):
        return any(_contain_tensor(v) for v in obj)
    return False


def _is_state_dict(obj) -> bool:
    if not isinstance(obj, dict):
        return False
    for value in obj.values():
        if isinstance(value, dict):
            if any(_contain_tensor(v) for v in value.values()):
                return False
        elif not isinstance(value, torch.Tensor):
            return False
    return True


def _build_saved_state_dict(state_dict):
    save_dict, name_table = {}, {}
    for key, value in state_dict.items():
        if isinstance(value, torch.Tensor):
            if value.numel() == 0 and value.dim() == 1 and isinstance(value, EagerParamBase):
                raise ValueError("The saved tensor is not initialized. If you used group sharded, please use "
                                 "save_group_sharded_model.")
            save_dict[key] = _to_numpy(value)
            name_table[key] = as_tensor(value).name
        else:
            save_dict[key] = value
    save_dict[_NAME_TABLE] = name_table
    return save_dict


def _unpack_saved_dict(saved_obj, protocol):
    if not (1 < protocol < 4) or not isinstance(saved_obj, dict):
        return saved_obj
    unpack_info, parts = {}, {}
    for key, value in saved_obj.items():
        if isinstance(value, np.ndarray):
            limit = int((2 ** 30 - 1) / value.dtype.itemsize)
            n = int(np.prod(value.shape))
            if n > limit:
                unpack_info[key] = {"OriginShape": value.shape, "slices": []}
                flat = value.flatten()
                for i in range(int(math.ceil(n / limit))):
                    part = f"{key}@@.{i}"
                    unpack_info[key]["slices"].append(part)
                    parts[part] = flat[i * limit:(i + 1) * limit]
    if unpack_info:
        for key, info in unpack_info.items():
            saved_obj.pop(key)
            for part in info["slices"]:
                saved_obj[part] = parts[part]
        saved_obj[_UNPACK_INFO] = unpack_info
    return saved_obj


def _pack_loaded_dict(load_obj):
    if isinstance(load_obj, dict) and _UNPACK_INFO in load_obj:
        removes = []
        for key, info in load_obj[_UNPACK_INFO].items():
            slices = [load_obj[p] for p in info["slices"]]
            load_obj[key] = np.concatenate(slices).reshape(info["OriginShape"])
            removes += info["slices"]
        for k in removes:
            load_obj.pop(k)
        load_obj.pop(_UNPACK_INFO)
    return load_obj


def _reduce_tensor(t):
    return (tuple, ((as_tensor(t).name, _to_numpy(t)),))


def _pickle_save(obj, f, protocol):
    pickler = pickle.Pickler(f, protocol)
    table = copyreg.dispatch_table.copy()
    table[Tensor] = _reduce_tensor
    table[EagerParamBase] = _reduce_tensor
    table[torch.Tensor] = _reduce_tensor
    pickler.dispatch_table = table
    pickler.dump(obj)


def save(obj, path, protocol=4, **configs):
    """Save a state dict / Tensor / nested container to ``path`` (``.pdparams``, ``.pdopt``, ...)."""
    if not isinstance(protocol, int) or protocol < 2 or protocol > 4:
        raise ValueError(f"Expected 1<'protocol'<5, but received protocol={protocol}")
    if isinstance(path, (str, os.PathLike)):
        path = os.fspath(path)
        if os.path.basename(path) == "":
            raise ValueError("The input path MUST be format of dirname/filename, but received empty filename.")
        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)
        fobj = open(path, "wb")
        close = True
    else:
        fobj, close = path, False
    try:
        if _is_state_dict(obj):
            saved = _unpack_saved_dict(_build_saved_state_dict(obj), protocol)
            pickle.dump(saved, fobj, protocol=protocol)
        else:
            _pickle_save(obj, fobj, protocol)
    finally:
        if close:
            fobj.close()


_async_threads = []


def async_save(obj, path, protocol=4, sync_other_task=False, **configs):
    """Copy tensors to host first, then pickle on a background thread."""
    def to_cpu(o):
        if isinstance(o, dict):
            return {k: to_cpu(v) for k, v in o.items()}
        if isinstance(o, torch.Tensor):
            c = as_tensor(o.detach().cpu())
            c.name = as_tensor(o).name
            return c
        return o
    if sync_other_task:
        clear_async_save_task_queue()
    snap = to_cpu(obj)
    t = threading.Thread(target=save, args=(snap, path, protocol))
    t.start()
    _async_threads.append(t)


def clear_async_save_task_queue():
    while _async_threads:
        _async_threads.pop().join()


def _is_name_array_tuple(o):
    return isinstance(o, tuple) and len(o) == 2 and isinstance(o[0], str) and isinstance(o[1], np.ndarray)


def _restore(obj, return_numpy):
    if _is_name_array_tuple(obj):
        if return_numpy:
            return obj[1]
        t = to_tensor(obj[1])
        t.name = obj[0]
        return t
    if isinstance(obj, np.ndarray):
        return obj if return_numpy else to_tensor(obj)
    if isinstance(obj, (dict, collections.OrderedDict)):
        return type(obj)((k, _restore(v, return_numpy)) for k, v in obj.items())
    if isinstance(obj, list):
        return [_restore(v, return_numpy) for v in obj]
    if isinstance(obj, tuple):
        return tuple(_restore(v, return_numpy) for v in obj)
    return obj


def load(path, **configs):
    """Inverse of :func:`save`.  ``return_numpy=True`` keeps ndarrays; ``keep_name_table=True`` keeps the
    ``StructuredToParameterName@@`` entry."""
    return_numpy = configs.get("return_numpy", False)
    keep_name_table = configs.get("keep_name_table", False)
    if isinstance(path, (str, os.PathLike)):
        path = os.fspath(path)
        if not os.path.exists(path):
            raise ValueError(f"The path `{path}` does not exist")
        with open(path, "rb") as f:
            obj = pickle.load(f, encoding="latin1")
    else:
        obj = pickle.load(path, encoding="latin1")
    if isinstance(obj, dict) and _NAME_TABLE in obj:
        obj = _pack_loaded_dict(obj)
        names = obj[_NAME_TABLE]
        if not keep_name_table:
            obj.pop(_NAME_TABLE)
        out = {}
        for k, v in obj.items():
            if k == _NAME_TABLE:
                out[k] = v
            elif isinstance(v, np.ndarray) and not return_numpy:
                t = to_tensor(v)
                if k in names:
                    t.name = names[k]
                out[k] = t
            else:
                out[k] = _restore(v, return_numpy)
        return out
    obj = _pack_loaded_dict(obj) if isinstance(obj, dict) else obj
    return _restore(obj, return_numpy)
