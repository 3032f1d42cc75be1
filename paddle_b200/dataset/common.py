"""Helpers of the legacy dataset package (python/paddle/dataset/common.py)."""
import glob
import hashlib
import os
import pickle

DATA_HOME = os.path.expanduser("~/.cache/paddle/dataset")


def md5file(fname):
    h = hashlib.md5()
    with open(fname, "rb") as f:
        for chunk in iter(lambda: f.read(4096), b""):
            h.update(chunk)
    return h.hexdigest()


def download(url, module_name, md5sum, save_name=None):
    path = os.path.join(DATA_HOME, module_name, save_name or url.split("/")[-1])
    if os.path.exists(path) and (md5sum is None or md5file(path) == md5sum):
        return path
    raise RuntimeError(f"Cannot download {url}: no network access; place the file at {path}")


def split(reader, line_count, suffix="%05d.pickle", dumper=pickle.dump):
    lines, idx = [], 0
    for d in reader():
        lines.append(d)
        if len(lines) >= line_count:
            with open(suffix % idx, "wb") as f:
                dumper(lines, f)
            lines, idx = [], idx + 1
    if lines:
        with open(suffix % idx, "wb") as f:
            dumper(lines, f)


def cluster_files_reader(files_pattern, trainer_count, trainer_id, loader=pickle.load):
    def reader():
        files = sorted(glob.glob(files_pattern))
        for fn in files[trainer_id::trainer_count]:
            with open(fn, "rb") as f:
                yield from loader(f)
    return reader
