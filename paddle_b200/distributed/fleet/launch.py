"""Legacy entry point ``python -m paddle.distributed.fleet.launch`` (python/paddle/distributed/fleet/launch.py:771):
same job as ``python -m paddle.distributed.launch``; the old flag spellings are mapped to the current ones."""
from __future__ import annotations

import sys

_RENAMES = {"--gpus": "--devices", "--selected_gpus": "--devices", "--ips": "--ips", "--nproc_per_node": "--nproc_per_node",
            "--log_dir": "--log_dir", "--servers": "--servers", "--workers": "--trainers", "--worker_num": "--trainer_num",
            "--server_num": "--server_num"}


def _translate(argv):
    out = []
    for a in argv:
        key, eq, val = a.partition("=")
        out.append(_RENAMES.get(key, key) + (eq + val if eq else ""))
    return out


def launch(argv=None):
    from ..launch.main import launch as _launch
    return _launch(_translate(list(sys.argv[1:] if argv is None else argv)))


if __name__ == "__main__":
    launch()
