"""``paddle.flops`` for dynamic-graph layers (python/paddle/hapi/dynamic_flops.py:40-330): forward hooks on leaf
layers count multiply-accumulates per layer type; ``custom_ops`` maps a layer class to a counter
``fn(layer, inputs, output) -> operations``."""
from __future__ import annotations

import numpy as np
import torch


def _numel(t):
    return int(np.prod(t.shape)) if hasattr(t, "shape") else 0


def count_convNd(m, x, y):
    kernel_ops = int(np.prod(m.weight.shape[2:])) * (m.weight.shape[1])          # per output element: k * (Cin / groups)
    bias_ops = 1 if getattr(m, "bias", None) is not None else 0
    return _numel(y) * (kernel_ops + bias_ops)


def count_linear(m, x, y):
    return _numel(y) * m.weight.shape[0]


def count_bn(m, x, y):
    return 2 * _numel(x[0]) if getattr(m, "weight", None) is not None else _numel(x[0])


def count_leaky_relu(m, x, y):
    return _numel(x[0])


def count_avgpool(m, x, y):
    return _numel(y)


def count_adap_avgpool(m, x, y):
    kernel = np.array(x[0].shape[2:]) // np.maximum(np.array(y.shape[2:]), 1)
    return _numel(y) * (int(np.prod(kernel)) + 1)


def count_zero_ops(m, x, y):
    return 0


def count_parameters(m):
    return sum(int(torch.Tensor.numel(p)) for p in m.parameters(include_sublayers=False))


def _register():
    from .. import nn
    table = {}
    for name, fn in (("Conv1D", count_convNd), ("Conv2D", count_convNd), ("Conv3D", count_convNd), ("Conv1DTranspose", count_convNd),
                     ("Conv2DTranspose", count_convNd), ("Conv3DTranspose", count_convNd), ("Linear", count_linear),
                     ("BatchNorm", count_bn), ("BatchNorm1D", count_bn), ("BatchNorm2D", count_bn), ("BatchNorm3D", count_bn),
                     ("LayerNorm", count_bn), ("GroupNorm", count_bn), ("SyncBatchNorm", count_bn),
                     ("ReLU", count_zero_ops), ("ReLU6", count_zero_ops), ("LeakyReLU", count_leaky_relu), ("Dropout", count_zero_ops),
                     ("MaxPool1D", count_zero_ops), ("MaxPool2D", count_zero_ops), ("MaxPool3D", count_zero_ops),
                     ("AdaptiveMaxPool1D", count_zero_ops), ("AdaptiveMaxPool2D", count_zero_ops), ("AdaptiveMaxPool3D", count_zero_ops),
                     ("AvgPool1D", count_avgpool), ("AvgPool2D", count_avgpool), ("AvgPool3D", count_avgpool),
                     ("AdaptiveAvgPool1D", count_adap_avgpool), ("AdaptiveAvgPool2D", count_adap_avgpool), ("AdaptiveAvgPool3D", count_adap_avgpool)):
        cls = getattr(nn, name, None)
        if isinstance(cls, type):
            table[cls] = fn
    return table


def dynamic_flops(model, inputs, custom_ops=None, print_detail=False):
    """Total operations of one forward pass of ``model(*inputs)``."""
    table = _register()
    table.update(custom_ops or {})
    rows, hooks = [], []

    def make(fn, layer):
        def hook(l, x, y):
            out = y[0] if isinstance(y, (list, tuple)) else y
            ops = int(fn(l, x, out))
            rows.append((type(l).__name__, list(x[0].shape) if x and hasattr(x[0], "shape") else [], list(out.shape) if hasattr(out, "shape") else [],
                         count_parameters(l), ops))
        return hook
    unknown = set()
    for layer in model.sublayers(include_self=True):
        if list(layer.children()):
            continue
        fn = next((f for c, f in table.items() if type(layer) is c), None) or next((f for c, f in table.items() if isinstance(layer, c)), None)
        if fn is None:
            unknown.add(type(layer).__name__)
            continue
        hooks.append(layer.register_forward_post_hook(make(fn, layer)))
    was_training = model.training
    model.eval()
    try:
        with torch.no_grad():
            model(*inputs)
    finally:
        for h in hooks:
            h.remove()
        if was_training:
            model.train()
    total = sum(r[4] for r in rows)
    if print_detail:
        w = (22, 24, 24, 14, 16)
        line = "+" + "+".join("-" * x for x in w) + "+"
        fmt = lambda cells: "|" + "|".join(f"{str(c)[:x - 2]:^{x}}" for c, x in zip(cells, w)) + "|"
        print("\n".join([line, fmt(("Layer Name", "Input Shape", "Output Shape", "Params", "Flops")), line] +
                        [fmt((f"{n}_{i}", a, b, p, f)) for i, (n, a, b, p, f) in enumerate(rows)] + [line]))
        if unknown:
            print("Layers without a counter (treated as zero): " + ", ".join(sorted(unknown)))
    print(f"Total Flops: {total}     Total Params: {sum(int(torch.Tensor.numel(p)) for p in model.parameters())}")
    return total


def flops(net, input_size, custom_ops=None, print_detail=False):
    """``input_size`` is the full shape of one input including the batch dimension, e.g. ``[1, 3, 224, 224]``."""
    import paddle_b200 as paddle
    x = paddle.randn(list(input_size))
    return dynamic_flops(net, [x], custom_ops, print_detail)
