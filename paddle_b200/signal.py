"""``paddle.signal`` (python/paddle/signal.py): ``stft`` / ``istft`` with Paddle's layout
(input ``[..., seq]``, output ``[..., n_fft//2+1, frames]``)."""
from __future__ import annotations

import torch

from ._core.tensor import as_tensor

__all__ = ["stft", "istft"]       # the reference exports these two; frame / overlap_add are importable as well


def _p(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


def stft(x, n_fft, hop_length=None, win_length=None, window=None, center=True, pad_mode="reflect", normalized=False,
         onesided=True, name=None):
    x, window = _p(x), _p(window)
    return as_tensor(torch.stft(x, n_fft, hop_length, win_length, window, center, pad_mode, normalized, onesided,
                                return_complex=True))


def istft(x, n_fft, hop_length=None, win_length=None, window=None, center=True, normalized=False, onesided=True,
          length=None, return_complex=False, name=None):
    x, window = _p(x), _p(window)
    return as_tensor(torch.istft(x, n_fft, hop_length, win_length, window, center, normalized, onesided, length,
                                 return_complex))


def frame(x, frame_length, hop_length, axis=-1, name=None):
    """Overlapping frames of length ``frame_length`` every ``hop_length`` samples: ``axis=-1`` -> [..., frame_length,
    num_frames]; ``axis=0`` -> [num_frames, frame_length, ...] (python/paddle/signal.py ``frame``)."""
    from ._op_table import frame as _frame
    if axis not in (0, -1):
        raise ValueError(f"Unexpected axis: {axis}. It should be 0 or -1.")
    if frame_length > x.shape[axis]:
        raise ValueError(f"frame_length ({frame_length}) should be less or equal than the size of axis {axis} ({x.shape[axis]})")
    if hop_length <= 0:
        raise ValueError(f"hop_length should be > 0, but got {hop_length}")
    return _frame(x, frame_length, hop_length, axis)


def overlap_add(x, hop_length, axis=-1, name=None):
    """Inverse layout of ``frame``: frames are summed back at their offsets."""
    from ._op_table import overlap_add as _ola
    if axis not in (0, -1):
        raise ValueError(f"Unexpected axis: {axis}. It should be 0 or -1.")
    return _ola(x, hop_length, axis)
