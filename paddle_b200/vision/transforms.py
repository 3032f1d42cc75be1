"""``paddle.vision.transforms`` (python/paddle/vision/transforms/): image transforms on CHW tensors / HWC arrays /
PIL images."""
from __future__ import annotations

import numbers
import random

import numpy as np
import torch

from .._core.tensor import as_tensor

__all__ = ["Compose", "ToTensor", "Normalize", "Resize", "CenterCrop", "RandomCrop", "RandomHorizontalFlip",
           "RandomVerticalFlip", "Transpose", "Pad", "RandomResizedCrop", "BrightnessTransform", "ContrastTransform",
           "Grayscale", "RandomRotation", "to_tensor", "normalize", "resize", "center_crop", "crop", "hflip", "vflip", "pad",
           "to_grayscale", "BaseTransform"]


def _to_chw_float(img):
    """-> float tensor [C, H, W] in the input's value range, plus a function restoring the input kind."""
    if isinstance(img, torch.Tensor):
        return img.as_subclass(torch.Tensor).float(), lambda t: as_tensor(t.to(img.dtype))
    arr = np.asarray(img)
    pil = not isinstance(img, np.ndarray)
    a = arr[..., None] if arr.ndim == 2 else arr
    t = torch.from_numpy(a.copy()).permute(2, 0, 1).float()

    def back(t):
        out = t.permute(1, 2, 0).round().clamp(0, 255).to(torch.uint8).numpy() if arr.dtype == np.uint8 else \
            t.permute(1, 2, 0).numpy().astype(arr.dtype)
        out = out[..., 0] if arr.ndim == 2 else out
        if pil:
            from PIL import Image
            return Image.fromarray(out)
        return out
    return t, back


def to_tensor(pic, data_format="CHW"):
    t, _ = _to_chw_float(pic)
    if not isinstance(pic, torch.Tensor) and np.asarray(pic).dtype == np.uint8:
        t = t / 255.0
    return as_tensor(t if data_format == "CHW" else t.permute(1, 2, 0))


def normalize(img, mean, std, data_format="CHW", to_rgb=False):
    t = img.as_subclass(torch.Tensor).float() if isinstance(img, torch.Tensor) else torch.as_tensor(np.asarray(img)).float()
    shape = (-1, 1, 1) if data_format == "CHW" else (1, 1, -1)
    m, s = torch.as_tensor(mean, dtype=torch.float32).reshape(shape), torch.as_tensor(std, dtype=torch.float32).reshape(shape)
    out = (t - m) / s
    return as_tensor(out) if isinstance(img, torch.Tensor) else out.numpy()


def resize(img, size, interpolation="bilinear"):
    t, back = _to_chw_float(img)
    H, W = t.shape[-2:]
    if isinstance(size, int):
        size = (size, int(size * W / H)) if H <= W else (int(size * H / W), size)
    mode = {"nearest": "nearest", "bilinear": "bilinear", "bicubic": "bicubic", "area": "area"}.get(interpolation, "bilinear")
    kw = {"align_corners": False} if mode in ("bilinear", "bicubic") else {}
    return back(torch.nn.functional.interpolate(t[None], size=tuple(size), mode=mode, **kw)[0])


def crop(img, top, left, height, width):
    t, back = _to_chw_float(img)
    return back(t[:, top:top + height, left:left + width])


def center_crop(img, output_size):
    t, back = _to_chw_float(img)
    oh, ow = (output_size, output_size) if isinstance(output_size, numbers.Number) else output_size
    H, W = t.shape[-2:]
    top, left = int(round((H - oh) / 2.0)), int(round((W - ow) / 2.0))
    return back(t[:, top:top + oh, left:left + ow])


def hflip(img):
    t, back = _to_chw_float(img)
    return back(t.flip(-1))


def vflip(img):
    t, back = _to_chw_float(img)
    return back(t.flip(-2))


def pad(img, padding, fill=0, padding_mode="constant"):
    t, back = _to_chw_float(img)
    if isinstance(padding, int):
        padding = (padding,) * 4
    elif len(padding) == 2:
        padding = (padding[0], padding[1], padding[0], padding[1])
    l, tp, r, b = padding
    mode = {"constant": "constant", "edge": "replicate", "reflect": "reflect", "symmetric": "reflect"}[padding_mode]
    kw = {"value": float(fill)} if mode == "constant" else {}
    return back(torch.nn.functional.pad(t[None], (l, r, tp, b), mode=mode, **kw)[0])


def to_grayscale(img, num_output_channels=1):
    t, back = _to_chw_float(img)
    g = (0.299 * t[0] + 0.587 * t[1] + 0.114 * t[2])[None]
    return back(g.expand(num_output_channels, -1, -1) if num_output_channels > 1 else g) if isinstance(img, torch.Tensor) \
        else back(g.expand(3, -1, -1)) if num_output_channels == 3 else np.asarray(g[0].round().clamp(0, 255).to(torch.uint8))


class BaseTransform:
    def __init__(self, keys=None):
        self.keys = keys

    def __call__(self, inputs):
        if isinstance(inputs, tuple) and self.keys:
            return tuple(self._apply_image(x) if k == "image" else x for x, k in zip(inputs, self.keys))
        return self._apply_image(inputs)

    def _apply_image(self, img):
        raise NotImplementedError


class Compose:
    def __init__(self, transforms):
        self.transforms = list(transforms)

    def __call__(self, data):
        for t in self.transforms:
            data = t(data)
        return data


class ToTensor(BaseTransform):
    def __init__(self, data_format="CHW", keys=None):
        super().__init__(keys)
        self.data_format = data_format

    def _apply_image(self, img):
        return to_tensor(img, self.data_format)


class Normalize(BaseTransform):
    def __init__(self, mean=0.0, std=1.0, data_format="CHW", to_rgb=False, keys=None):
        super().__init__(keys)
        self.mean = [mean] * 3 if isinstance(mean, numbers.Number) else mean
        self.std = [std] * 3 if isinstance(std, numbers.Number) else std
        self.data_format = data_format

    def _apply_image(self, img):
        return normalize(img, self.mean, self.std, self.data_format)


class Resize(BaseTransform):
    def __init__(self, size, interpolation="bilinear", keys=None):
        super().__init__(keys)
        self.size, self.interpolation = size, interpolation

    def _apply_image(self, img):
        return resize(img, self.size, self.interpolation)


class CenterCrop(BaseTransform):
    def __init__(self, size, keys=None):
        super().__init__(keys)
        self.size = size

    def _apply_image(self, img):
        return center_crop(img, self.size)


class RandomCrop(BaseTransform):
    def __init__(self, size, padding=None, pad_if_needed=False, fill=0, padding_mode="constant", keys=None):
        super().__init__(keys)
        self.size = (size, size) if isinstance(size, numbers.Number) else tuple(size)
        self.padding, self.fill, self.padding_mode = padding, fill, padding_mode

    def _apply_image(self, img):
        if self.padding is not None:
            img = pad(img, self.padding, self.fill, self.padding_mode)
        t, _ = _to_chw_float(img)
        H, W = t.shape[-2:]
        top, left = random.randint(0, H - self.size[0]), random.randint(0, W - self.size[1])
        return crop(img, top, left, *self.size)


class RandomHorizontalFlip(BaseTransform):
    def __init__(self, prob=0.5, keys=None):
        super().__init__(keys)
        self.prob = prob

    def _apply_image(self, img):
        return hflip(img) if random.random() < self.prob else img


class RandomVerticalFlip(RandomHorizontalFlip):
    def _apply_image(self, img):
        return vflip(img) if random.random() < self.prob else img


class Transpose(BaseTransform):
    def __init__(self, order=(2, 0, 1), keys=None):
        super().__init__(keys)
        self.order = order

    def _apply_image(self, img):
        a = np.asarray(img)
        a = a[..., None] if a.ndim == 2 else a
        return a.transpose(self.order)


class Pad(BaseTransform):
    def __init__(self, padding, fill=0, padding_mode="constant", keys=None):
        super().__init__(keys)
        self.padding, self.fill, self.padding_mode = padding, fill, padding_mode

    def _apply_image(self, img):
        return pad(img, self.padding, self.fill, self.padding_mode)


class RandomResizedCrop(BaseTransform):
    def __init__(self, size, scale=(0.08, 1.0), ratio=(3 / 4, 4 / 3), interpolation="bilinear", keys=None):
        super().__init__(keys)
        self.size = (size, size) if isinstance(size, int) else tuple(size)
        self.scale, self.ratio, self.interpolation = scale, ratio, interpolation

    def _apply_image(self, img):
        t, _ = _to_chw_float(img)
        H, W = t.shape[-2:]
        for _ in range(10):
            area = H * W * random.uniform(*self.scale)
            ar = np.exp(random.uniform(np.log(self.ratio[0]), np.log(self.ratio[1])))
            w, h = int(round(np.sqrt(area * ar))), int(round(np.sqrt(area / ar)))
            if 0 < w <= W and 0 < h <= H:
                top, left = random.randint(0, H - h), random.randint(0, W - w)
                return resize(crop(img, top, left, h, w), self.size, self.interpolation)
        return resize(center_crop(img, min(H, W)), self.size, self.interpolation)


class BrightnessTransform(BaseTransform):
    def __init__(self, value, keys=None):
        super().__init__(keys)
        self.value = value

    def _apply_image(self, img):
        t, back = _to_chw_float(img)
        return back(t * random.uniform(max(0, 1 - self.value), 1 + self.value))


class ContrastTransform(BrightnessTransform):
    def _apply_image(self, img):
        t, back = _to_chw_float(img)
        f = random.uniform(max(0, 1 - self.value), 1 + self.value)
        m = t.mean()
        return back((t - m) * f + m)


class Grayscale(BaseTransform):
    def __init__(self, num_output_channels=1, keys=None):
        super().__init__(keys)
        self.n = num_output_channels

    def _apply_image(self, img):
        return to_grayscale(img, self.n)


class RandomRotation(BaseTransform):
    def __init__(self, degrees, interpolation="nearest", expand=False, center=None, fill=0, keys=None):
        super().__init__(keys)
        self.degrees = (-degrees, degrees) if isinstance(degrees, numbers.Number) else degrees
        self.interpolation = interpolation

    def _apply_image(self, img):
        t, back = _to_chw_float(img)
        ang = np.deg2rad(random.uniform(*self.degrees))
        theta = torch.tensor([[np.cos(ang), -np.sin(ang), 0.0], [np.sin(ang), np.cos(ang), 0.0]], dtype=torch.float32)[None]
        grid = torch.nn.functional.affine_grid(theta, (1, *t.shape), align_corners=False)
        mode = "nearest" if self.interpolation == "nearest" else "bilinear"
        return back(torch.nn.functional.grid_sample(t[None], grid, mode=mode, align_corners=False)[0])
