"""``paddle.distributed.io`` (python/paddle/distributed/io.py): persistables of static programs."""
import os

from ..static import load as _load, load_inference_model, save as _save  # noqa: F401


def is_persistable(var):
    return bool(getattr(var, "persistable", False))


def save_persistables(executor, dirname, main_program=None, filename=None):
    from ..static import default_main_program
    os.makedirs(dirname, exist_ok=True)
    _save(main_program or default_main_program(), os.path.join(dirname, filename or "persistables"))


def load_persistables(executor, dirname, main_program=None, filename=None):
    from ..static import default_main_program
    _load(main_program or default_main_program(), os.path.join(dirname, filename or "persistables"), executor)


def load_inference_model_distributed(dirname, executor, model_filename=None, params_filename=None, pserver_endpoints=None):
    return load_inference_model(os.path.join(dirname, model_filename or "model"), executor)
