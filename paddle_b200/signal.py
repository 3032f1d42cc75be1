"""``paddle.signal`` (python/paddle/signal.py): ``stft`` / ``istft`` with Paddle's layout
(input ``[..., seq]``, output ``[..., n_fft//2+1, frames]``)."""
from __future__ import annotations

import torch

from ._core.tensor import as_tensor

__all__ = ["stft", "istft"]


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
