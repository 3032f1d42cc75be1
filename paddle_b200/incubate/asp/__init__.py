"""Automatic sparsity (python/paddle/incubate/asp/): prune supported layers' weights to the n:m pattern the sparse
tensor cores accept (2:4 by default) and keep the pattern through training by re-applying the masks after every
optimizer step."""
from __future__ import annotations

import enum
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


class MaskAlgo(enum.Enum):
    """Mask generating algorithms (python/paddle/incubate/asp/utils.py:36)."""
    MASK_1D = "get_mask_1d"
    MASK_2D_GREEDY = "get_mask_2d_greedy"
    MASK_2D_BEST = "get_mask_2d_best"


class CheckMethod(enum.Enum):
    CHECK_1D = "check_mask_1d"
    CHECK_2D = "check_mask_2d"

    @staticmethod
    def get_checking_method(mask_algo):
        assert isinstance(mask_algo, MaskAlgo), "mask_algo should be MaskAlgo type"
        return CheckMethod.CHECK_1D if mask_algo == MaskAlgo.MASK_1D else CheckMethod.CHECK_2D


def _np(mat):
    if isinstance(mat, torch.Tensor):
        return mat.detach().as_subclass(torch.Tensor).cpu().numpy()
    return np.asarray(mat)


def _groups_1d(mat, m):
    """Rows padded with zeros to a multiple of ``m`` and cut into groups of ``m`` -> ([groups, m], padded shape)."""
    mat = _np(mat)
    mat = mat.reshape(1, -1) if mat.ndim == 1 else mat
    pad = (-mat.shape[1]) % m
    padded = np.pad(mat, ((0, 0), (0, pad)))
    return padded.reshape(-1, m), padded.shape


def check_mask_1d(mat, n, m):
    """n:m pattern along rows: at least ``n`` zeros in every group of ``m`` consecutive elements."""
    g, _ = _groups_1d(mat, m)
    return bool(((g != 0).sum(1) <= m - n).all())


def get_mask_1d(mat, n, m):
    """0 / 1 mask that zeroes the ``n`` smallest magnitudes of every group of ``m`` consecutive row elements."""
    src = _np(mat)
    g, padded_shape = _groups_1d(src, m)
    mask = np.ones_like(g)
    order = np.argsort(np.abs(g), axis=1, kind="stable")[:, :n]
    np.put_along_axis(mask, order, 0, axis=1)
    src2 = src.reshape(1, -1) if src.ndim == 1 else src
    return mask.reshape(padded_shape)[:, :src2.shape[1]].reshape(src.shape)


def _blocks_2d(mat, m):
    """Zero-padded to multiples of ``m`` both ways and cut into m x m blocks -> ([blocks, m * m], padded shape)."""
    mat = _np(mat)
    pr, pc = (-mat.shape[0]) % m, (-mat.shape[1]) % m
    padded = np.pad(mat, ((0, pr), (0, pc)))
    R, C = padded.shape
    return padded.reshape(R // m, m, C // m, m).transpose(0, 2, 1, 3).reshape(-1, m * m), padded.shape


def _unblock_2d(blocks, padded_shape, m, shape):
    R, C = padded_shape
    return blocks.reshape(R // m, C // m, m, m).transpose(0, 2, 1, 3).reshape(R, C)[:shape[0], :shape[1]]


def check_mask_2d(mat, n, m):
    """2-D n:m pattern per m x m block: at least ``n`` zeros in each row and each column.  As in the reference's check
    a block is rejected only when some row AND some column both break the rule."""
    blocks, _ = _blocks_2d(mat, m)
    b = blocks.reshape(-1, m, m) != 0
    row_bad = (b.sum(2) > m - n).any(1)
    col_bad = (b.sum(1) > m - n).any(1)
    return not bool((row_bad & col_bad).any())


def get_mask_2d_greedy(mat, n, m):
    """Per m x m block, keep elements in order of decreasing magnitude while no row or column exceeds ``m - n``."""
    src = _np(mat)
    blocks, padded_shape = _blocks_2d(src, m)
    out = np.zeros(blocks.shape, dtype=np.float64)
    keep = m - n
    for bi, blk in enumerate(np.abs(blocks)):
        rows, cols = np.zeros(m, int), np.zeros(m, int)
        for flat in np.argsort(blk)[::-1]:                 # largest first; equal values in reverse index order
            r, c = divmod(int(flat), m)
            if rows[r] < keep and cols[c] < keep:
                out[bi, flat] = 1
                rows[r] += 1
                cols[c] += 1
    return _unblock_2d(out, padded_shape, m, src.shape)


_PATTERNS = {}


def _valid_2d_patterns(n, m):
    key = (n, m)
    if key not in _PATTERNS:
        row = [p for p in itertools.product([0, 1], repeat=m) if sum(p) == m - n]
        pats = [np.array(c) for c in itertools.product(row, repeat=m) if (np.array(c).sum(0) <= m - n).all()]
        _PATTERNS[key] = np.stack(pats).reshape(len(pats), -1).astype(np.float64)
    return _PATTERNS[key]


def get_mask_2d_best(mat, n, m):
    """Per m x m block, the valid pattern (``m - n`` kept per row, at most ``m - n`` per column) with the largest kept
    magnitude - exhaustive over the patterns."""
    src = _np(mat)
    blocks, padded_shape = _blocks_2d(src, m)
    P = _valid_2d_patterns(n, m)
    best = (np.abs(blocks).astype(np.float64) @ P.T).argmax(1)
    return _unblock_2d(P[best].astype(src.dtype if src.dtype.kind == "f" else np.float64), padded_shape, m, src.shape)


def _mask_1d(mat, n, m):
    return torch.as_tensor(get_mask_1d(mat.cpu().numpy(), n, m), dtype=mat.dtype)


def _mask_2d_best(mat, n, m):
    return torch.as_tensor(get_mask_2d_best(mat.cpu().numpy(), n, m), dtype=mat.dtype)


def _algo_name(func_name):
    if isinstance(func_name, (MaskAlgo, CheckMethod)):
        return func_name.value
    return {"mask_1d": "get_mask_1d", "mask_2d_greedy": "get_mask_2d_greedy", "mask_2d_best": "get_mask_2d_best",
            "check_1d": "check_mask_1d", "check_2d": "check_mask_2d"}.get(func_name, func_name)


def create_mask(tensor, func_name=MaskAlgo.MASK_1D, n=2, m=4):
    """Mask of the same shape as ``tensor`` (numpy array or Tensor): 1-D and 2-D inputs are pruned as matrices, 3-D as
    [d0 * d1, d2], 4-D (convolution weights, [out, in, h, w]) along the input channels."""
    is_tensor = isinstance(tensor, torch.Tensor)
    t = _np(tensor)
    shape, dtype = t.shape, t.dtype
    fn = globals()[_algo_name(func_name)]
    if t.ndim == 1:
        mat = t.reshape(1, -1)
    elif t.ndim == 2:
        mat = t
    elif t.ndim == 3:
        mat = t.reshape(shape[0] * shape[1], shape[2])
    elif t.ndim == 4:
        mat = t.transpose(0, 2, 3, 1).reshape(-1, shape[1])
    else:
        raise ValueError(f"The dimension of input tensor is not supported in create_mask, only dimension < 4 is supported but got {t.ndim}")
    mask = fn(mat, n=n, m=m)
    if t.ndim == 4:
        mask = mask.reshape(shape[0], shape[2], shape[3], shape[1]).transpose(0, 3, 1, 2)
    mask = mask.reshape(shape).astype(dtype)
    return torch.as_tensor(mask).to(tensor.dtype) if is_tensor else mask


def check_sparsity(tensor, func_name=CheckMethod.CHECK_1D, n=2, m=4):
    t = _np(tensor)
    shape = t.shape
    fn = globals()[_algo_name(func_name)]
    if t.ndim == 1:
        mat = t.reshape(1, -1)
    elif t.ndim == 2:
        mat = t
    elif t.ndim == 3:
        mat = t.reshape(shape[0] * shape[1], shape[2])
    elif t.ndim == 4:
        mat = t.transpose(0, 2, 3, 1).reshape(-1, shape[1])
    else:
        raise ValueError(f"The dimension of input tensor is not supported in check_sparsity, only dimension < 4 is supported but got {t.ndim}")
    return fn(mat, n=n, m=m)


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
