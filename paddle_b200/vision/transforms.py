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


def _is_pil_image(img):
    try:
        from PIL import Image
    except ImportError:
        return False
    return isinstance(img, Image.Image)


def _is_numpy_image(img):
    return isinstance(img, np.ndarray) and img.ndim in (2, 3)


def _is_tensor_image(img):
    return isinstance(img, torch.Tensor)


class BaseTransform:
    """Base of the transforms (python/paddle/vision/transforms/transforms.py ``BaseTransform``).  ``keys`` names what each
    element of a tuple input is (``"image"``, ``"coords"``, ``"boxes"``, ``"mask"``; ``None`` entries pass through) and
    every element goes to ``_apply_<key>``.  ``_get_params(inputs)`` is evaluated once per call into ``self.params`` so
    that random decisions are shared by all elements."""

    def __init__(self, keys=None):
        if keys is None:
            keys = ("image",)
        elif not isinstance(keys, (list, tuple)):
            raise ValueError(f"keys should be a list or tuple, but got {type(keys)}")
        for k in keys:
            if k is not None and not hasattr(self, f"_apply_{k}") and k not in ("image", "coords", "boxes", "mask"):
                raise NotImplementedError(f"{k} is unsupported data structure")
        self.keys = tuple(keys)
        self.params = None

    def _get_params(self, inputs):
        return None

    def __call__(self, inputs):
        is_seq = isinstance(inputs, (tuple, list))
        seq = tuple(inputs) if is_seq else (inputs,)
        self.params = self._get_params(seq)
        out = []
        for i, x in enumerate(seq):
            key = self.keys[i] if i < len(self.keys) else None
            fn = getattr(self, f"_apply_{key}", None) if key is not None else None
            out.append(fn(x) if fn is not None else x)
        if not is_seq:
            return out[0]
        return tuple(out) if isinstance(inputs, tuple) else out

    def _apply_image(self, img):
        raise NotImplementedError

    def _apply_boxes(self, boxes):
        raise NotImplementedError

    def _apply_mask(self, mask):
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


# ----------------------------------------------------------------------------- colour and geometric extras
__all__ += ["SaturationTransform", "HueTransform", "ColorJitter", "RandomAffine", "RandomPerspective", "RandomErasing",
            "affine", "rotate", "perspective", "adjust_brightness", "adjust_contrast", "adjust_hue", "erase"]


def _scale_of(img):
    return 255.0 if not isinstance(img, torch.Tensor) or img.dtype == torch.uint8 else 1.0


def adjust_brightness(img, brightness_factor):
    t, back = _to_chw_float(img)
    return back((t * brightness_factor).clamp(0, _scale_of(img)))


def adjust_contrast(img, contrast_factor):
    t, back = _to_chw_float(img)
    g = (0.299 * t[0] + 0.587 * t[1] + 0.114 * t[2]).mean() if t.shape[0] == 3 else t.mean()
    return back(((t - g) * contrast_factor + g).clamp(0, _scale_of(img)))


def adjust_saturation(img, saturation_factor):
    t, back = _to_chw_float(img)
    g = (0.299 * t[0] + 0.587 * t[1] + 0.114 * t[2])[None]
    return back(((t - g) * saturation_factor + g).clamp(0, _scale_of(img)))


def _rgb_to_hsv(t):
    r, g, b = t
    mx, mn = torch.max(t, 0).values, torch.min(t, 0).values
    d = mx - mn
    s = torch.where(mx > 0, d / mx.clamp_min(1e-12), torch.zeros_like(mx))
    dz = d.clamp_min(1e-12)
    h = torch.where(mx == r, ((g - b) / dz) % 6, torch.where(mx == g, (b - r) / dz + 2, (r - g) / dz + 4)) / 6.0
    h = torch.where(d == 0, torch.zeros_like(h), h)
    return torch.stack([h, s, mx])


def _hsv_to_rgb(t):
    h, s, v = t
    i = torch.floor(h * 6)
    f = h * 6 - i
    p, q, u = v * (1 - s), v * (1 - f * s), v * (1 - (1 - f) * s)
    i = i.long() % 6
    r = torch.stack([v, q, p, p, u, v]).gather(0, i[None])[0]
    g = torch.stack([u, v, v, q, p, p]).gather(0, i[None])[0]
    b = torch.stack([p, p, u, v, v, q]).gather(0, i[None])[0]
    return torch.stack([r, g, b])


def adjust_hue(img, hue_factor):
    if not -0.5 <= hue_factor <= 0.5:
        raise ValueError("hue_factor is not in [-0.5, 0.5].")
    t, back = _to_chw_float(img)
    if t.shape[0] != 3:
        return img
    sc = _scale_of(img)
    hsv = _rgb_to_hsv(t / sc)
    hsv[0] = (hsv[0] + hue_factor) % 1.0
    return back(_hsv_to_rgb(hsv) * sc)


def erase(img, i, j, h, w, v, inplace=False):
    if isinstance(img, torch.Tensor):
        out = img if inplace else img.clone()
        out.as_subclass(torch.Tensor)[..., i:i + h, j:j + w] = torch.as_tensor(v, dtype=out.dtype)
        return out
    arr = np.asarray(img).copy()
    arr[i:i + h, j:j + w] = np.asarray(v.numpy() if isinstance(v, torch.Tensor) else v).reshape(-1)[0] if np.ndim(v) == 0 \
        else np.asarray(v)
    if not isinstance(img, np.ndarray):
        from PIL import Image
        return Image.fromarray(arr)
    return arr


def _warp(img, theta_or_grid, interpolation, fill, homography=None):
    """Samples the image on an output grid; ``theta`` is the 2x3 output->input map in normalised coordinates."""
    t, back = _to_chw_float(img)
    C, H, W = t.shape
    if homography is None:
        grid = torch.nn.functional.affine_grid(theta_or_grid[None], (1, C, H, W), align_corners=False)
    else:
        ys, xs = torch.meshgrid(torch.arange(H, dtype=torch.float32) + 0.5, torch.arange(W, dtype=torch.float32) + 0.5,
                                indexing="ij")
        ones = torch.ones_like(xs)
        src = torch.einsum("ij,jhw->ihw", homography, torch.stack([xs, ys, ones]))
        gx, gy = src[0] / src[2] / W * 2 - 1, src[1] / src[2] / H * 2 - 1
        grid = torch.stack([gx, gy], -1)[None]
    mode = "nearest" if interpolation == "nearest" else "bilinear"
    out = torch.nn.functional.grid_sample(t[None], grid, mode=mode, padding_mode="zeros", align_corners=False)[0]
    if fill:
        mask = torch.nn.functional.grid_sample(torch.ones(1, 1, H, W), grid, mode=mode, padding_mode="zeros",
                                               align_corners=False)[0]
        fv = torch.as_tensor(fill, dtype=torch.float32).reshape(-1, 1, 1)
        out = out * mask + fv * (1 - mask)
    return back(out)


def _affine_theta(angle, translate, scale, shear, H, W, center=None):
    """Inverse affine (output -> input) in normalised [-1, 1] coordinates for rotation by ``angle`` degrees
    counter-clockwise about ``center``, then shear, scale and translation in pixels."""
    rot = np.deg2rad(angle)
    sx, sy = [np.deg2rad(s) for s in (shear if isinstance(shear, (list, tuple)) else (shear, 0.0))]
    cx, cy = ((W * 0.5, H * 0.5) if center is None else center)
    # forward matrix M = T(center) * T(translate) * R S Sh * T(-center) in pixel coordinates (y down)
    a = np.cos(rot - sy) / np.cos(sy)
    b = -np.cos(rot - sy) * np.tan(sx) / np.cos(sy) - np.sin(rot)
    c = np.sin(rot - sy) / np.cos(sy)
    d = -np.sin(rot - sy) * np.tan(sx) / np.cos(sy) + np.cos(rot)
    M = np.array([[a * scale, b * scale, 0.0], [c * scale, d * scale, 0.0], [0, 0, 1.0]])
    T1 = np.array([[1, 0, cx + translate[0]], [0, 1, cy + translate[1]], [0, 0, 1.0]])
    T2 = np.array([[1, 0, -cx], [0, 1, -cy], [0, 0, 1.0]])
    fwd = T1 @ M @ T2
    inv = np.linalg.inv(fwd)
    # pixel -> normalised: x_n = 2 x / W - 1
    N = np.array([[2.0 / W, 0, -1], [0, 2.0 / H, -1], [0, 0, 1]])
    th = N @ inv @ np.linalg.inv(N)
    return torch.tensor(th[:2], dtype=torch.float32)


def affine(img, angle, translate, scale, shear, interpolation="nearest", fill=0, center=None):
    t, _ = _to_chw_float(img)
    H, W = t.shape[-2:]
    return _warp(img, _affine_theta(angle, translate, scale, shear, H, W, center), interpolation, fill)


def rotate(img, angle, interpolation="nearest", expand=False, center=None, fill=0):
    t, _ = _to_chw_float(img)
    H, W = t.shape[-2:]
    return _warp(img, _affine_theta(-angle, (0, 0), 1.0, (0.0, 0.0), H, W, center), interpolation, fill)


def _homography(startpoints, endpoints):
    """3x3 matrix mapping ``endpoints`` (output corners) to ``startpoints`` (input corners)."""
    A, bvec = [], []
    for (x, y), (u, v) in zip(endpoints, startpoints):
        A.append([x, y, 1, 0, 0, 0, -u * x, -u * y])
        A.append([0, 0, 0, x, y, 1, -v * x, -v * y])
        bvec += [u, v]
    h = np.linalg.lstsq(np.asarray(A, dtype=np.float64), np.asarray(bvec, dtype=np.float64), rcond=None)[0]
    return torch.tensor(np.append(h, 1.0).reshape(3, 3), dtype=torch.float32)


def perspective(img, startpoints, endpoints, interpolation="nearest", fill=0):
    return _warp(img, None, interpolation, fill, homography=_homography(startpoints, endpoints))


class SaturationTransform(BrightnessTransform):
    def _apply_image(self, img):
        if self.value == 0:
            return img
        return adjust_saturation(img, random.uniform(max(0, 1 - self.value), 1 + self.value))


class HueTransform(BaseTransform):
    def __init__(self, value, keys=None):
        super().__init__(keys)
        if not 0 <= value <= 0.5:
            raise ValueError("hue value should be in [0.0, 0.5]")
        self.value = value

    def _apply_image(self, img):
        if self.value == 0:
            return img
        return adjust_hue(img, random.uniform(-self.value, self.value))


class ColorJitter(BaseTransform):
    def __init__(self, brightness=0, contrast=0, saturation=0, hue=0, keys=None):
        super().__init__(keys)
        self.ts = [BrightnessTransform(brightness), ContrastTransform(contrast), SaturationTransform(saturation),
                   HueTransform(hue)]

    def _apply_image(self, img):
        order = list(range(4))
        random.shuffle(order)
        for i in order:
            if self.ts[i].value:
                img = self.ts[i]._apply_image(img)
        return img


class RandomAffine(BaseTransform):
    def __init__(self, degrees, translate=None, scale=None, shear=None, interpolation="nearest", fill=0, center=None,
                 keys=None):
        super().__init__(keys)
        self.degrees = (-degrees, degrees) if isinstance(degrees, numbers.Number) else tuple(degrees)
        self.translate, self.scale = translate, scale
        if isinstance(shear, numbers.Number):
            shear = (-shear, shear)
        self.shear, self.interpolation, self.fill, self.center = shear, interpolation, fill, center

    def _apply_image(self, img):
        t, _ = _to_chw_float(img)
        H, W = t.shape[-2:]
        angle = random.uniform(*self.degrees)
        tr = (0, 0)
        if self.translate is not None:
            tr = (round(random.uniform(-self.translate[0] * W, self.translate[0] * W)),
                  round(random.uniform(-self.translate[1] * H, self.translate[1] * H)))
        sc = random.uniform(*self.scale) if self.scale is not None else 1.0
        sh = (0.0, 0.0)
        if self.shear is not None:
            sh = (random.uniform(self.shear[0], self.shear[1]),
                  random.uniform(self.shear[2], self.shear[3]) if len(self.shear) == 4 else 0.0)
        return affine(img, angle, tr, sc, sh, self.interpolation, self.fill, self.center)


class RandomPerspective(BaseTransform):
    def __init__(self, prob=0.5, distortion_scale=0.5, interpolation="nearest", fill=0, keys=None):
        super().__init__(keys)
        self.prob, self.d, self.interpolation, self.fill = prob, distortion_scale, interpolation, fill

    def _apply_image(self, img):
        if random.random() >= self.prob:
            return img
        t, _ = _to_chw_float(img)
        H, W = t.shape[-2:]
        hw, hh = int(self.d * W / 2), int(self.d * H / 2)
        r = random.randint
        end = [(r(0, hw), r(0, hh)), (W - 1 - r(0, hw), r(0, hh)), (W - 1 - r(0, hw), H - 1 - r(0, hh)),
               (r(0, hw), H - 1 - r(0, hh))]
        start = [(0, 0), (W - 1, 0), (W - 1, H - 1), (0, H - 1)]
        return perspective(img, start, end, self.interpolation, self.fill)


class RandomErasing(BaseTransform):
    def __init__(self, prob=0.5, scale=(0.02, 0.33), ratio=(0.3, 3.3), value=0, inplace=False, keys=None):
        super().__init__(keys)
        self.prob, self.scale, self.ratio, self.value, self.inplace = prob, scale, ratio, value, inplace

    def _apply_image(self, img):
        if random.random() >= self.prob:
            return img
        t, _ = _to_chw_float(img)
        C, H, W = t.shape
        area = H * W
        for _ in range(10):
            a = area * random.uniform(*self.scale)
            ar = np.exp(random.uniform(np.log(self.ratio[0]), np.log(self.ratio[1])))
            h, w = int(round(np.sqrt(a * ar))), int(round(np.sqrt(a / ar)))
            if 0 < h < H and 0 < w < W:
                i, j = random.randint(0, H - h), random.randint(0, W - w)
                v = torch.randn(C, h, w) if self.value == "random" else self.value
                if isinstance(img, torch.Tensor):
                    return erase(img, i, j, h, w, v, self.inplace)
                return erase(img, i, j, h, w, 0 if self.value == "random" else v, self.inplace)
        return img


# ``paddle.vision.transforms.functional`` is a module of its own in the reference
from .._core.submodule_alias import alias_submodules as _alias  # noqa: E402
_alias(__name__, ("functional", "transforms"))
