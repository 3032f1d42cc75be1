"""Small helpers of the pipeline point-to-point layer
(python/paddle/distributed/fleet/meta_parallel/pp_utils/utils.py): the integer codes under which tensor dtypes travel
in the shape/dtype handshake, byte sizes, float checks."""
from __future__ import annotations

import torch

from ....._core import dtype as _dt

FLOAT_TYPE_DICT = {torch.float16: "float16", torch.float32: "float32", torch.float64: "float64", torch.bfloat16: "bfloat16"}
PADDLE_TO_NUMBER = {torch.float16: 0, torch.float32: 1, torch.float64: 2, torch.int32: 3, torch.int64: 4,
                    torch.bfloat16: 5, torch.bool: 6, torch.uint8: 7, torch.int8: 8}
NUMBER_TO_DTYPE = {v: k for k, v in PADDLE_TO_NUMBER.items()}


def is_float_tensor(tensor):
    return tensor.dtype in FLOAT_TYPE_DICT


def get_tensor_dtype(dtype):
    assert dtype in FLOAT_TYPE_DICT, f"{dtype} is not a floating dtype"
    return FLOAT_TYPE_DICT[dtype]


def paddle_2_number(dtype):
    return PADDLE_TO_NUMBER[_dt.to_torch(dtype) or dtype]


def number_2_dtype(number):
    return NUMBER_TO_DTYPE[int(number)]


def get_tensor_bytes(tensor):
    """Bytes of ``tensor``'s elements (``numel * element size``)."""
    return tensor.numel() * tensor.element_size()
