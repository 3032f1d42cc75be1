"""Fleet logger (python/paddle/distributed/fleet/utils/log_util.py): ``logger``, ``set_log_level``,
``get_log_level_code/name``, ``layer_to_str``."""
import logging

logger = logging.getLogger("FleetLog")
if not logger.handlers:
    _h = logging.StreamHandler()
    _h.setFormatter(logging.Formatter("%(levelname)s %(asctime)s %(filename)s:%(lineno)d] %(message)s"))
    logger.addHandler(_h)
    logger.setLevel(logging.INFO)
    logger.propagate = False


def set_log_level(level):
    logger.setLevel(level if isinstance(level, int) else getattr(logging, str(level).upper()))


def get_log_level_code():
    return logger.getEffectiveLevel()


def get_log_level_name():
    return logging.getLevelName(get_log_level_code())


def layer_to_str(base, *args, **kwargs):
    parts = [str(a) for a in args] + [f"{k}={v}" for k, v in kwargs.items()]
    return f"{base}({', '.join(parts)})"
