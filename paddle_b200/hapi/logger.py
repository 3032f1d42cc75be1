"""Logger of the high-level API (python/paddle/hapi/logger.py:23-70): one stream handler on rank 0, optional file."""
from __future__ import annotations

import logging
import os
import sys


def setup_logger(output=None, name="paddle_b200.hapi", log_level=logging.INFO):
    logger = logging.getLogger(name)
    logger.propagate = False
    logger.setLevel(log_level)
    fmt = logging.Formatter("%(asctime)s - %(levelname)s - %(message)s", datefmt="%Y-%m-%d %H:%M:%S")
    rank = int(os.environ.get("PADDLE_TRAINER_ID", os.environ.get("RANK", 0)))
    if rank == 0 and not any(isinstance(h, logging.StreamHandler) and not isinstance(h, logging.FileHandler) for h in logger.handlers):
        h = logging.StreamHandler(sys.stdout)
        h.setFormatter(fmt)
        logger.addHandler(h)
    if output is not None:
        path = output if output.endswith((".txt", ".log")) else os.path.join(output, "log.txt")
        if rank > 0:
            path += f".rank{rank}"
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        fh = logging.FileHandler(path)
        fh.setFormatter(fmt)
        logger.addHandler(fh)
    return logger
