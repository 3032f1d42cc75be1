"""``paddle.fft`` (python/paddle/fft.py): discrete Fourier transforms with Paddle's argument names
(``n``/``s``, ``axis``/``axes``, ``norm`` in {"backward", "ortho", "forward"})."""
from __future__ import annotations

import torch

from ._core.tensor import as_tensor

__all__ = ["fft", "ifft", "rfft", "irfft", "hfft", "ihfft", "fft2", "ifft2", "rfft2", "irfft2", "hfft2", "ihfft2", "fftn",
           "ifftn", "rfftn", "irfftn", "hfftn", "ihfftn", "fftfreq", "rfftfreq", "fftshift", "ifftshift"]


def _one(fn):
    def f(x, n=None, axis=-1, norm="backward", name=None):
        return as_tensor(fn(x, n=n, dim=axis, norm=norm))
    return f


def _many(fn, default_axes=None):
    def f(x, s=None, axes=default_axes, norm="backward", name=None):
        return as_tensor(fn(x, s=s, dim=axes, norm=norm))
    return f


fft, ifft, rfft, irfft, hfft, ihfft = (_one(getattr(torch.fft, n)) for n in ("fft", "ifft", "rfft", "irfft", "hfft", "ihfft"))
fft2, ifft2, rfft2, irfft2 = (_many(getattr(torch.fft, n), (-2, -1)) for n in ("fft2", "ifft2", "rfft2", "irfft2"))
hfft2, ihfft2 = (_many(getattr(torch.fft, n), (-2, -1)) for n in ("hfft2", "ihfft2"))
fftn, ifftn, rfftn, irfftn, hfftn, ihfftn = (_many(getattr(torch.fft, n)) for n in
                                             ("fftn", "ifftn", "rfftn", "irfftn", "hfftn", "ihfftn"))


def fftfreq(n, d=1.0, dtype=None, name=None):
    return as_tensor(torch.fft.fftfreq(n, d))


def rfftfreq(n, d=1.0, dtype=None, name=None):
    return as_tensor(torch.fft.rfftfreq(n, d))


def fftshift(x, axes=None, name=None):
    return as_tensor(torch.fft.fftshift(x, dim=axes))


def ifftshift(x, axes=None, name=None):
    return as_tensor(torch.fft.ifftshift(x, dim=axes))
