"""Text form of a Tensor as the reference prints it (python/paddle/tensor/to_string.py:24-330):

    Tensor(shape=[2, 3], dtype=float32, place=Place(cpu), stop_gradient=True,
           [[1.        , 2.50000000, 3.        ],
            [4.        , 5.        , 6.        ]])

Floats with an integral value print as ``4.``, others with ``precision`` digits; every element is padded to the widest
one (and to a sign column when any element is negative); rows wrap at ``linewidth``; tensors above ``threshold``
elements show ``edgeitems`` at each end of every dimension around ``...``."""
from __future__ import annotations

import numpy as np


class PrintOptions:
    precision = 8
    threshold = 1000
    edgeitems = 3
    linewidth = 80
    sci_mode = False


DEFAULT_PRINT_OPTIONS = PrintOptions()


def set_printoptions(precision=None, threshold=None, edgeitems=None, sci_mode=None, linewidth=None):
    for name, val, typ in (("precision", precision, int), ("threshold", threshold, int), ("edgeitems", edgeitems, int),
                           ("linewidth", linewidth, int), ("sci_mode", sci_mode, bool)):
        if val is None:
            continue
        if not isinstance(val, typ) or (typ is int and isinstance(val, bool)):
            raise TypeError(f"The type of '{name}' in set_printoptions must be {typ.__name__}, but received {type(val).__name__}.")
        setattr(DEFAULT_PRINT_OPTIONS, name, val)


def _item_text(v):
    opt = DEFAULT_PRINT_OPTIONS
    if isinstance(v, (np.floating, float)):
        if opt.sci_mode:
            return f"{v:.{opt.precision}e}"
        if np.isfinite(v) and np.ceil(v) == v:
            return f"{v:.0f}."
        return f"{v:.{opt.precision}f}"
    return str(v)


def _pad(text, width, signed, negative):
    if width <= len(text):
        return text
    if signed and not negative:
        return " " + text.ljust(width - 1)
    return text.ljust(width)


def _edges(a, k):
    """The elements a summarised print shows (used to size the columns)."""
    if a.size == 0 or a.ndim == 0:
        return a
    if a.shape[0] > 2 * k:
        a = np.concatenate([a[:k], a[-k:]])
    if a.ndim == 1:
        return a
    return np.stack([_edges(x, k) for x in a])


def _fmt(a, summary, indent, width, signed):
    opt = DEFAULT_PRINT_OPTIONS
    k = opt.edgeitems

    def cell(v):
        neg = bool(np.isreal(v) and not isinstance(v, (np.bool_, bool)) and v < 0) if not np.iscomplexobj(v) else False
        return _pad(_item_text(v), width, signed, neg)
    if a.ndim == 0:
        return cell(a[()])
    if a.ndim == 1:
        per_line = max(1, (opt.linewidth - indent) // (width + 2))
        if summary and a.shape[0] > 2 * k:
            items = [cell(v) for v in a[:k]] + ["..."] + [cell(v) for v in a[-k:]]
        else:
            items = [cell(v) for v in a]
        lines = [", ".join(items[i:i + per_line]) for i in range(0, len(items), per_line)]
        return "[" + (",\n" + " " * (indent + 1)).join(lines) + "]"
    if summary and a.shape[0] > 2 * k:
        rows = [_fmt(x, summary, indent + 1, width, signed) for x in a[:k]] + ["..."] + \
               [_fmt(x, summary, indent + 1, width, signed) for x in a[-k:]]
    else:
        rows = [_fmt(x, summary, indent + 1, width, signed) for x in a]
    return "[" + ("," + "\n" * (a.ndim - 1) + " " * (indent + 1)).join(rows) + "]"


def format_array(a, indent):
    a = np.asarray(a)
    size = 0 if a.ndim == 0 else a.size
    summary = size > DEFAULT_PRINT_OPTIONS.threshold
    shown = _edges(a, DEFAULT_PRINT_OPTIONS.edgeitems) if summary else a
    width, signed = 0, False
    for v in np.asarray(shown).reshape(-1):
        if not signed and not np.iscomplexobj(v) and not isinstance(v, (np.bool_, bool)) and v < 0:
            signed = True
        width = max(width, len(_item_text(v)))
    if a.ndim and a.shape[0] == 0:
        return "[]"
    return _fmt(a, summary, indent, width, signed)


def place_str(device):
    if device.type == "cuda":
        return f"Place(gpu:{device.index or 0})"
    return f"Place({device.type})"


def to_string(t, prefix="Tensor"):
    import torch

    from .._core import dtype as _dt
    indent = len(prefix) + 1
    plain = t.detach().as_subclass(torch.Tensor)
    if plain.dtype in (torch.bfloat16,) or str(plain.dtype).startswith("torch.float8"):
        plain = plain.float()
    try:
        arr = plain.cpu().resolve_conj().resolve_neg().numpy()
        data = format_array(arr, indent)
    except Exception:  # noqa: BLE001 - meta tensors, tensors on a lost device ...
        data = "<unprintable>"
    return (f"{prefix}(shape={list(t.shape)}, dtype={_dt.to_name(t.dtype)}, place={place_str(t.device)}, "
            f"stop_gradient={t.stop_gradient},\n{' ' * indent}{data})")
