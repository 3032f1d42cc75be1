"""dtype / place helpers.  Paddle dtypes are represented by the torch dtype objects themselves
(``paddle.float32 is torch.float32``); strings such as ``'float32'`` are accepted everywhere."""
from __future__ import annotations

import numpy as np
import torch

_NAME2T = {
    "float32": torch.float32, "float": torch.float32, "fp32": torch.float32,
    "float64": torch.float64, "double": torch.float64,
    "float16": torch.float16, "half": torch.float16, "fp16": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "uint16": torch.bfloat16,
    "int8": torch.int8, "uint8": torch.uint8, "int16": torch.int16, "int32": torch.int32,
    "int": torch.int32, "int64": torch.int64, "long": torch.int64, "bool": torch.bool,
    "complex64": torch.complex64, "complex128": torch.complex128,
    "float8_e4m3fn": torch.float8_e4m3fn, "float8_e5m2": torch.float8_e5m2,
}
_T2NAME = {
    torch.float32: "float32", torch.float64: "float64", torch.float16: "float16",
    torch.bfloat16: "bfloat16", torch.int8: "int8", torch.uint8: "uint8", torch.int16: "int16",
    torch.int32: "int32", torch.int64: "int64", torch.bool: "bool", torch.complex64: "complex64",
    torch.complex128: "complex128", torch.float8_e4m3fn: "float8_e4m3fn", torch.float8_e5m2: "float8_e5m2",
}
_default_dtype = torch.float32
_device = None


def to_torch(dtype):
    if dtype is None:
        return None
    if isinstance(dtype, torch.dtype):
        return dtype
    if isinstance(dtype, str):
        key = dtype.replace("paddle.", "")
        if key in _NAME2T:
            return _NAME2T[key]
        raise TypeError(f"unknown dtype {dtype!r}")
    if isinstance(dtype, np.dtype) or (isinstance(dtype, type) and issubclass(dtype, np.generic)):
        return _NAME2T[np.dtype(dtype).name]
    if dtype is float:
        return _default_dtype
    if dtype is int:
        return torch.int64
    if dtype is bool:
        return torch.bool
    raise TypeError(f"unknown dtype {dtype!r}")


def to_name(dtype) -> str:
    return _T2NAME.get(to_torch(dtype), str(dtype))


def set_default_dtype(d):
    global _default_dtype
    _default_dtype = to_torch(d)
    torch.set_default_dtype(_default_dtype)


def get_default_dtype():
    return _default_dtype


def default_device() -> torch.device:
    global _device
    if _device is None:
        if torch.cuda.is_available():
            _device = torch.device("cuda", torch.cuda.current_device())
        else:
            _device = torch.device("cpu")
    return _device


def set_device(device):
    """``paddle.set_device('gpu:0' | 'cpu' | 'gpu')``."""
    global _device
    d = to_device(device)
    if d.type == "cuda":
        torch.cuda.set_device(d)
    _device = d
    return d


def get_device() -> str:
    d = default_device()
    return "cpu" if d.type == "cpu" else f"gpu:{d.index if d.index is not None else 0}"


class CPUPlace:
    def __init__(self):
        self.device = torch.device("cpu")

    def __repr__(self):
        return "Place(cpu)"


class CUDAPlace:
    def __init__(self, idx=0):
        self.device = torch.device("cuda", idx)

    def get_device_id(self):
        return self.device.index

    def __repr__(self):
        return f"Place(gpu:{self.device.index})"


class CUDAPinnedPlace(CPUPlace):
    pass


def to_device(place):
    if place is None:
        return None
    if isinstance(place, torch.device):
        return place
    if isinstance(place, (CPUPlace, CUDAPlace)):
        return place.device
    if isinstance(place, str):
        s = place.lower()
        if s.startswith("gpu") or s.startswith("cuda"):
            idx = int(s.split(":")[1]) if ":" in s else (torch.cuda.current_device() if torch.cuda.is_available() else 0)
            return torch.device("cuda", idx)
        if s.startswith("cpu"):
            return torch.device("cpu")
    raise ValueError(f"unknown place {place!r}")
