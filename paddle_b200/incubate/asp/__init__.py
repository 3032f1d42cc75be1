"""Automatic sparsity (python/paddle/incubate/asp/): prune supported layers' weights to the n:m pattern the sparse
tensor cores accept (2:4 by default) and keep the pattern through training by re-applying the masks after every
optimizer step."""
from __future__ import annotations

import itertools

import numpy as np
import torch

__all__ = ["calculate_density", "decorate", "prune_model", "set_excluded_layers", "reset_excluded_layers",
           "add_supported_layer"]

_excluded = set()
_supported = {"Linear", "Conv2D", "Conv1D", "Conv3D", "ColumnParallelLinear", "RowParallelLinear"}
_custom_prune = {}
_masks = {}            # id(param) -> (param, mask tensor)


def calculate_density(x):
    a = np.asarray(x.numpy() if hasattr(x, "numpy") else x).flatten()
    return float(np.nonzero(a)[0].size) / a.size


def set_excluded_layers(param_names, main_program=None):
    _excluded.update(param_names)


def reset_excluded_layers(main_program=None):
    _excluded.clear()


def add_supported_layer(layer, pruning_func=None):
    name = layer if isinstance(layer, str) else layer.__name__
    _supported.add(name)
    if pruning_func is not None:
        _custom_prune[name] = pruning_func


def _mask_1d(mat, n, m):
    """Keep the ``n`` largest magnitudes in every group of ``m`` consecutive elements of each row."""
    rows, cols = mat.shape
    pad = (-cols) % m
    a = torch.nn.functional.pad(mat.abs(), (0, pad)).reshape(rows, -1, m)
    idx = a.topk(n, -1).indices
    mask = torch.zeros_like(a).scatter_(-1, idx, 1.0).reshape(rows, -1)[:, :cols]
    return mask


def _mask_2d_best(mat, n, m):
    """m x m blocks with exactly n non-zeros in every row and column, chosen to keep the most magnitude."""
    rows, cols = mat.shape
    pr, pc = (-rows) % m, (-cols) % m
    a = torch.nn.functional.pad(mat.abs(), (0, pc, 0, pr))
    R, C = a.shape
    blocks = a.reshape(R // m, m, C // m, m).permute(0, 2, 1, 3).reshape(-1, m * m)
    row_patterns = [p for p in itertools.product([0, 1], repeat=m) if sum(p) == n]
    pats = [np.array(c) for c in itertools.product(row_patterns, repeat=m) if (np.array(c).sum(0) == n).all()]
    P = torch.tensor(np.stack(pats).reshape(len(pats), -1), dtype=a.dtype)
    best = (blocks @ P.t()).argmax(1)
    mask = P[best].reshape(R // m, C // m, m, m).permute(0, 2, 1, 3).reshape(R, C)
    return mask[:rows, :cols]


def create_mask(tensor, func_name="mask_1d", n=2, m=4):
    t = tensor.as_subclass(torch.Tensor).detach().float()
    shape = t.shape
    mat = t.reshape(shape[0], -1) if t.dim() != 2 else t
    if t.dim() == 4:                               # conv: prune along input channels
        mat = t.permute(0, 2, 3, 1).reshape(-1, shape[1])
    mask = _mask_2d_best(mat, n, m) if func_name in ("mask_2d_best", "mask_2d_greedy") else _mask_1d(mat, n, m)
    if t.dim() == 4:
        mask = mask.reshape(shape[0], shape[2], shape[3], shape[1]).permute(0, 3, 1, 2)
    return mask.reshape(shape).to(tensor.dtype)


def check_sparsity(tensor, n=2, m=4, func_name="check_1d"):
    t = tensor.as_subclass(torch.Tensor).detach() if isinstance(tensor, torch.Tensor) else torch.as_tensor(np.asarray(tensor))
    mat = t.reshape(t.shape[0], -1)
    pad = (-mat.shape[1]) % m
    g = torch.nn.functional.pad(mat, (0, pad)).reshape(mat.shape[0], -1, m)
    return bool(((g != 0).sum(-1) <= n).all())


def prune_model(model, n=2, m=4, mask_algo="mask_1d", with_mask=True):
    """Prunes the weights of every supported sub-layer of ``model``; returns ``{param name: mask}``."""
    out = {}
    for layer in model.sublayers(include_self=True):
        kind = type(layer).__name__
        if kind not in _supported:
            continue
        w = getattr(layer, "weight", None)
        if w is None or w.name in _excluded or w.dim() < 2:
            continue
        if kind in _custom_prune:
            pruned, mask = _custom_prune[kind](w.numpy(), m, n, mask_algo, w.name)
            mask = torch.as_tensor(mask, dtype=w.dtype)
            with torch.no_grad():
                w.as_subclass(torch.Tensor).copy_(torch.as_tensor(pruned, dtype=w.dtype))
        else:
            # Linear weights are [in, out]: the n:m groups run along the reduction (input) dimension
            src = w.as_subclass(torch.Tensor).t() if w.dim() == 2 else w
            mask = create_mask(src, mask_algo, n, m)
            mask = mask.t() if w.dim() == 2 else mask
            with torch.no_grad():
                w.as_subclass(torch.Tensor).mul_(mask.to(w.device))
        if with_mask:
            _masks[id(w)] = (w, mask.to(w.device))
        out[w.name] = mask
    return out


class OptimizerWithSparsityGuarantee:
    """Wraps an optimizer: after every step the stored masks are applied again."""

    def __init__(self, optimizer):
        self._optimizer = optimizer

    def __getattr__(self, name):
        return getattr(self._optimizer, name)

    def step(self):
        self._optimizer.step()
        with torch.no_grad():
            for w, mask in _masks.values():
                w.as_subclass(torch.Tensor).mul_(mask)

    def minimize(self, loss, startup_program=None, parameters=None, no_grad_set=None):
        loss.backward()
        self.step()
        return None, None


def decorate(optimizer):
    return OptimizerWithSparsityGuarantee(optimizer)
