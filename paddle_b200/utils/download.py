"""``paddle.utils.download`` (python/paddle/utils/download.py): weight files are resolved from the local cache
``~/.cache/paddle/hapi/weights`` or a ``file://`` URL; this build has no network access."""
import hashlib
import os
import shutil

WEIGHTS_HOME = os.path.expanduser("~/.cache/paddle/hapi/weights")


def _md5(path):
    h = hashlib.md5()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def get_path_from_url(url, root_dir, md5sum=None, check_exist=True, decompress=True, method="get"):
    name = url.split("/")[-1]
    target = os.path.join(root_dir, name)
    if not (check_exist and os.path.exists(target)):
        src = url[len("file://"):] if url.startswith("file://") else None
        if src is None or not os.path.exists(src):
            raise RuntimeError(f"cannot download {url}: no network access; place the file at {target}")
        os.makedirs(root_dir, exist_ok=True)
        shutil.copyfile(src, target)
    if md5sum is not None and _md5(target) != md5sum:
        raise RuntimeError(f"md5 mismatch for {target}")
    return target


def get_weights_path_from_url(url, md5sum=None):
    return get_path_from_url(url, WEIGHTS_HOME, md5sum)
