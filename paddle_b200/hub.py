"""``paddle.hub`` (python/paddle/hapi/hub.py): ``list`` / ``help`` / ``load`` entry points from a ``hubconf.py``.
Only ``source="local"`` works here (github / gitee sources need a network)."""
from __future__ import annotations

import importlib.util
import os
import sys

__all__ = ["list", "help", "load"]


def _import(repo_dir, source):
    if source != "local":
        raise RuntimeError(f"hub source '{source}' needs network access; clone the repository and use source='local'")
    path = os.path.join(repo_dir, "hubconf.py")
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    sys.path.insert(0, repo_dir)
    try:
        spec = importlib.util.spec_from_file_location("hubconf", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        sys.path.remove(repo_dir)
    return mod


def list(repo_dir, source="github", force_reload=False):  # noqa: A001
    mod = _import(repo_dir, source)
    return [n for n in dir(mod) if callable(getattr(mod, n)) and not n.startswith("_")]


def help(repo_dir, model, source="github", force_reload=False):  # noqa: A001
    return getattr(_import(repo_dir, source), model).__doc__


def load(repo_dir, model, source="github", force_reload=False, **kwargs):
    return getattr(_import(repo_dir, source), model)(**kwargs)


def load_state_dict_from_url(url, model_dir=None, check_hash=False, file_name=None, map_location=None):
    """Loads a state dict from a ``file://`` URL or a local path (there is no network access in this build)."""
    import os
    from .framework.io import load as _load
    path = url[len("file://"):] if url.startswith("file://") else url
    if not os.path.exists(path):
        raise RuntimeError(f"cannot fetch {url!r}: only local files are reachable")
    return _load(path)
