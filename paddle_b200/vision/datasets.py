"""``paddle.vision.datasets``: dataset classes that read LOCAL files (this build has no network: ``download=True``
without the files raises)."""
from __future__ import annotations

import gzip
import os
import pickle
import struct
import tarfile

import numpy as np

from ..io import Dataset


class MNIST(Dataset):
    NAME = "mnist"

    def __init__(self, image_path=None, label_path=None, mode="train", transform=None, download=True, backend=None):
        if image_path is None or label_path is None or not (os.path.exists(image_path) and os.path.exists(label_path)):
            raise RuntimeError(f"{self.NAME}: pass image_path/label_path of the idx .gz files (no network to download them)")
        with gzip.open(image_path, "rb") as f:
            _, n, r, c = struct.unpack(">IIII", f.read(16))
            self.images = np.frombuffer(f.read(), dtype=np.uint8).reshape(n, r, c)
        with gzip.open(label_path, "rb") as f:
            f.read(8)
            self.labels = np.frombuffer(f.read(), dtype=np.uint8).astype(np.int64)
        self.transform = transform

    def __getitem__(self, i):
        img = self.images[i]
        if self.transform is not None:
            img = self.transform(img)
        return img, np.array([self.labels[i]])

    def __len__(self):
        return len(self.labels)


class FashionMNIST(MNIST):
    NAME = "fashion-mnist"


class Cifar10(Dataset):
    def __init__(self, data_file=None, mode="train", transform=None, download=True, backend=None):
        if data_file is None or not os.path.exists(data_file):
            raise RuntimeError("Cifar: pass data_file (the python-version tar.gz); there is no network to download it")
        want = "data_batch" if mode == "train" else "test_batch"
        xs, ys = [], []
        with tarfile.open(data_file) as tar:
            for m in tar.getmembers():
                if want in m.name or (self._fine and ("train" in m.name if mode == "train" else "test" in m.name)):
                    d = pickle.load(tar.extractfile(m), encoding="bytes")
                    xs.append(d[b"data"])
                    ys += d.get(b"labels", d.get(b"fine_labels", []))
        self.data = np.concatenate(xs).reshape(-1, 3, 32, 32).transpose(0, 2, 3, 1)
        self.labels = np.asarray(ys, dtype=np.int64)
        self.transform = transform

    _fine = False

    def __getitem__(self, i):
        img = self.data[i]
        if self.transform is not None:
            img = self.transform(img)
        return img, np.array(self.labels[i])

    def __len__(self):
        return len(self.labels)


class Cifar100(Cifar10):
    _fine = True


class DatasetFolder(Dataset):
    def __init__(self, root, loader=None, extensions=None, transform=None, is_valid_file=None):
        exts = tuple(extensions or (".jpg", ".jpeg", ".png", ".ppm", ".bmp", ".pgm", ".tif", ".tiff", ".webp"))
        self.classes = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
        self.class_to_idx = {c: i for i, c in enumerate(self.classes)}
        self.samples = [(os.path.join(root, c, f), self.class_to_idx[c]) for c in self.classes
                        for f in sorted(os.listdir(os.path.join(root, c)))
                        if (is_valid_file(os.path.join(root, c, f)) if is_valid_file else f.lower().endswith(exts))]
        self.loader = loader or self._pil
        self.transform = transform

    @staticmethod
    def _pil(path):
        from PIL import Image
        with open(path, "rb") as f:
            return Image.open(f).convert("RGB")

    def __getitem__(self, i):
        path, y = self.samples[i]
        img = self.loader(path)
        if self.transform is not None:
            img = self.transform(img)
        return img, y

    def __len__(self):
        return len(self.samples)


class ImageFolder(DatasetFolder):
    def __init__(self, root, loader=None, extensions=None, transform=None, is_valid_file=None):
        exts = tuple(extensions or (".jpg", ".jpeg", ".png", ".bmp"))
        self.samples = [(os.path.join(dp, f), 0) for dp, _, fs in sorted(os.walk(root)) for f in sorted(fs)
                        if f.lower().endswith(exts)]
        self.loader = loader or self._pil
        self.transform = transform

    def __getitem__(self, i):
        img = self.loader(self.samples[i][0])
        return [self.transform(img) if self.transform is not None else img]


class Flowers(Dataset):
    """Oxford 102 flowers (python/paddle/vision/datasets/flowers.py): ``data_file`` is ``102flowers.tgz``,
    ``label_file`` ``imagelabels.mat`` and ``setid_file`` ``setid.mat``.  As in the reference, ``train`` uses the
    (larger) ``tstid`` split, ``test`` uses ``trnid`` and ``valid`` uses ``valid``."""
    _FLAG = {"train": "tstid", "test": "trnid", "valid": "valid"}

    def __init__(self, data_file=None, label_file=None, setid_file=None, mode="train", transform=None, download=True,
                 backend=None):
        assert mode.lower() in ("train", "valid", "test"), f"mode should be 'train', 'valid' or 'test', but got {mode}"
        root = os.path.expanduser("~/.cache/paddle/dataset/flowers")
        data_file = data_file or os.path.join(root, "102flowers.tgz")
        label_file = label_file or os.path.join(root, "imagelabels.mat")
        setid_file = setid_file or os.path.join(root, "setid.mat")
        for f in (data_file, label_file, setid_file):
            if not os.path.exists(f):
                raise RuntimeError(f"Flowers needs {f}; this build cannot download it")
        import scipy.io as scio
        self.backend = backend or "pil"
        self.transform = transform
        self.labels = scio.loadmat(label_file)["labels"][0]
        self.indexes = scio.loadmat(setid_file)[self._FLAG[mode.lower()]][0]
        self._tar = tarfile.open(data_file)
        self._members = {m.name: m for m in self._tar.getmembers()}

    def __getitem__(self, idx):
        import io

        from PIL import Image
        index = int(self.indexes[idx])
        raw = self._tar.extractfile(self._members["jpg/image_%05d.jpg" % index]).read()
        image = Image.open(io.BytesIO(raw))
        if self.backend == "cv2":
            image = np.array(image)
        if self.transform is not None:
            image = self.transform(image)
        return image, np.array([self.labels[index - 1]]).astype("int64")

    def __len__(self):
        return len(self.indexes)


class VOC2012(Dataset):
    """Pascal VOC 2012 segmentation pairs read straight from ``VOCtrainval_11-May-2012.tar``
    (python/paddle/vision/datasets/voc2012.py); the mode -> image-set mapping is the reference's."""
    _SET = "VOCdevkit/VOC2012/ImageSets/Segmentation/{}.txt"
    _DATA = "VOCdevkit/VOC2012/JPEGImages/{}.jpg"
    _LABEL = "VOCdevkit/VOC2012/SegmentationClass/{}.png"
    _FLAG = {"train": "trainval", "test": "train", "valid": "val"}

    def __init__(self, data_file=None, mode="train", transform=None, download=True, backend=None):
        assert mode.lower() in ("train", "valid", "test"), f"mode should be 'train', 'valid' or 'test', but got {mode}"
        data_file = data_file or os.path.expanduser("~/.cache/paddle/dataset/voc2012/VOCtrainval_11-May-2012.tar")
        if not os.path.exists(data_file):
            raise RuntimeError(f"VOC2012 needs {data_file}; this build cannot download it")
        self.backend = backend or "pil"
        self.transform = transform
        self._tar = tarfile.open(data_file)
        self._members = {m.name: m for m in self._tar.getmembers()}
        names = self._tar.extractfile(self._members[self._SET.format(self._FLAG[mode.lower()])]).read().decode().split()
        self.data = [self._DATA.format(n) for n in names]
        self.labels = [self._LABEL.format(n) for n in names]

    def __getitem__(self, idx):
        import io

        from PIL import Image
        data = Image.open(io.BytesIO(self._tar.extractfile(self._members[self.data[idx]]).read()))
        label = Image.open(io.BytesIO(self._tar.extractfile(self._members[self.labels[idx]]).read()))
        if self.backend == "cv2":
            data, label = np.array(data), np.array(label)
        if self.transform is not None:
            data = self.transform(data)
        return data, (label if self.backend == "pil" else label.astype("int64"))

    def __len__(self):
        return len(self.data)
