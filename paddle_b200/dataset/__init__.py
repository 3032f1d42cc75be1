"""``paddle.dataset``: the legacy reader-style dataset package.  Its loaders download public corpora; offline they
resolve files from ``~/.cache/paddle/dataset`` and raise when a file is absent.  ``common`` carries the helpers
(md5file, download, cluster file splitting) the readers are built from."""
from . import common  # noqa: F401

__all__ = []


def __getattr__(name):
    if name in ("mnist", "cifar", "uci_housing", "imdb", "imikolov", "movielens", "conll05", "wmt14", "wmt16", "flowers",
                "voc2012", "image"):
        raise ImportError(f"paddle.dataset.{name} downloads its corpus on first use, which an offline build cannot do; "
                          f"use paddle.vision.datasets / paddle.text with local files")
    raise AttributeError(name)
