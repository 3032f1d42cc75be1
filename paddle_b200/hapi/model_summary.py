"""``paddle.summary`` (python/paddle/hapi/model_summary.py:40-600): one forward pass with hooks on every leaf layer
records input / output shapes and parameter counts; the table ends with the totals and size estimates in MB."""
from __future__ import annotations

import numbers
from collections import OrderedDict

import numpy as np
import torch


def _shape_of(x):
    if isinstance(x, torch.Tensor):
        return list(x.shape)
    if isinstance(x, (list, tuple)):
        return [_shape_of(v) for v in x]
    if isinstance(x, dict):
        return {k: _shape_of(v) for k, v in x.items()}
    return []


def _numel_of(shape):
    if isinstance(shape, dict):
        return sum(_numel_of(v) for v in shape.values())
    if shape and isinstance(shape[0], (list, dict)):
        return sum(_numel_of(s) for s in shape)
    return int(np.prod(shape)) if shape else 0


def _normalize_sizes(input_size):
    """``(3, 224, 224)`` / ``[(1, 28), (1, 10)]`` / InputSpec-like objects -> list of shapes; a leading ``None`` or
    ``-1`` batch dimension becomes 1."""
    def one(s):
        if hasattr(s, "shape") and not isinstance(s, (list, tuple)):
            s = s.shape
        return [1 if (d is None or d == -1) else int(d) for d in s]
    if hasattr(input_size, "shape") and not isinstance(input_size, (list, tuple)):
        return [one(input_size)]
    if isinstance(input_size, (list, tuple)) and input_size and all(isinstance(d, numbers.Number) or d is None for d in input_size):
        return [one(input_size)]
    return [one(s) for s in input_size]


def summary_string(model, input_size=None, dtypes=None, input=None):
    """-> (table text, {"total_params": .., "trainable_params": ..})."""
    import paddle_b200 as paddle
    if input is None:
        if input_size is None:
            raise ValueError("input_size and input cannot both be None")
        sizes = _normalize_sizes(input_size)
        if dtypes is None:
            dtypes = ["float32"] * len(sizes)
        elif isinstance(dtypes, str):
            dtypes = [dtypes] * len(sizes)
        args = [paddle.zeros(s, dtype=d) if "float" in str(d) else paddle.zeros(s, dtype=d) for s, d in zip(sizes, dtypes)]
    else:
        args = [input]               # a given input is passed as ONE argument, whatever its type (tensor, list, dict)
    rows = OrderedDict()
    hooks = []

    def hook(layer, inp, out):
        key = f"{type(layer).__name__}-{len(rows) + 1}"
        own = list(layer.parameters(include_sublayers=False))
        rows[key] = dict(input_shape=_shape_of(inp[0] if isinstance(inp, tuple) and len(inp) == 1 else inp), output_shape=_shape_of(out),
                         nb_params=sum(int(torch.Tensor.numel(p)) for p in own),
                         trainable=sum(int(torch.Tensor.numel(p)) for p in own if not p.stop_gradient))
    for layer in model.sublayers(include_self=True):
        if not list(layer.children()) or layer is model and not list(model.children()):
            hooks.append(layer.register_forward_post_hook(hook))
    was_training = model.training
    model.eval()
    try:
        with torch.no_grad():
            model(*args)
    finally:
        for h in hooks:
            h.remove()
        if was_training:
            model.train()
    total = sum(int(torch.Tensor.numel(p)) for p in model.parameters())
    trainable = sum(int(torch.Tensor.numel(p)) for p in model.parameters() if not p.stop_gradient)
    w = [max(20, *(len(k) for k in rows)) + 2, 26, 26, 14]
    line = "-" * sum(w)
    out = [line, f"{'Layer (type)':<{w[0]}}{'Input Shape':<{w[1]}}{'Output Shape':<{w[2]}}{'Param #':>{w[3]}}", "=" * sum(w)]
    total_out = 0
    for k, r in rows.items():
        out.append(f"{k:<{w[0]}}{str(r['input_shape'])[:w[1] - 1]:<{w[1]}}{str(r['output_shape'])[:w[2] - 1]:<{w[2]}}{r['nb_params']:>{w[3]},d}")
        total_out += _numel_of(r["output_shape"])
    def _leaves(o):
        if isinstance(o, torch.Tensor):
            yield o
        elif isinstance(o, (list, tuple)):
            for v in o:
                yield from _leaves(v)
        elif isinstance(o, dict):
            for v in o.values():
                yield from _leaves(v)
    in_numel = sum(int(torch.Tensor.numel(a)) for a in _leaves(args))
    mb = lambda n: n * 4 / 1024 ** 2
    out += ["=" * sum(w), f"Total params: {total:,d}", f"Trainable params: {trainable:,d}", f"Non-trainable params: {total - trainable:,d}", line,
            f"Input size (MB): {mb(in_numel):.2f}", f"Forward/backward pass size (MB): {mb(2 * total_out):.2f}", f"Params size (MB): {mb(total):.2f}",
            f"Estimated Total Size (MB): {mb(in_numel + 2 * total_out + total):.2f}", line]
    return "\n".join(out) + "\n", {"total_params": total, "trainable_params": trainable}


def summary(net, input_size=None, dtypes=None, input=None):
    text, info = summary_string(net, input_size, dtypes, input)
    print(text)
    return info
