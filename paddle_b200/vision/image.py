"""Image backend selection and loading (python/paddle/vision/image.py)."""
_backend = "pil"

__all__ = []


def set_image_backend(backend):
    global _backend
    if backend not in ("pil", "cv2", "tensor"):
        raise ValueError(f"Expected backend are one of ['pil', 'cv2', 'tensor'], but got {backend}")
    _backend = backend


def get_image_backend():
    return _backend


def image_load(path, backend=None):
    backend = backend or _backend
    if backend not in ("pil", "cv2", "tensor"):
        raise ValueError(f"Expected backend are one of ['pil', 'cv2', 'tensor'], but got {backend}")
    from PIL import Image
    img = Image.open(path)
    if backend == "pil":
        return img
    import numpy as np
    arr = np.array(img.convert("RGB"))[..., ::-1] if backend == "cv2" else np.array(img)
    if backend == "tensor":
        from .transforms import to_tensor
        return to_tensor(img)
    return arr
