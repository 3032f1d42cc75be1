"""GPU utilisation watcher of the launcher (python/paddle/distributed/launch/controllers/watcher.py,
launch/utils/nvsmi.py): a background thread that samples ``nvidia-smi`` (read-only query) every ``interval`` seconds
and appends one line per GPU to ``<log_dir>/gpu.log``.  Nothing is sampled when ``nvidia-smi`` is absent."""
from __future__ import annotations

import os
import shutil
import subprocess
import threading
import time

FIELDS = ("index", "utilization.gpu", "memory.used", "memory.total", "power.draw", "clocks.sm")


def query_nvidia_smi(fields=FIELDS):
    """One sample: list of dicts, one per GPU ([] when the tool is missing or fails)."""
    exe = shutil.which("nvidia-smi")
    if exe is None:
        return []
    try:
        out = subprocess.run([exe, f"--query-gpu={','.join(fields)}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=10).stdout
    except (OSError, subprocess.SubprocessError):
        return []
    rows = []
    for line in out.strip().splitlines():
        vals = [v.strip() for v in line.split(",")]
        if len(vals) == len(fields):
            rows.append(dict(zip(fields, vals)))
    return rows


class Watcher:
    def __init__(self, log_dir, interval=30.0, sampler=query_nvidia_smi, devices=None):
        self.path = os.path.join(log_dir, "gpu.log")
        self.interval, self.sampler = float(interval), sampler
        self.devices = None if devices is None else {str(d) for d in devices}
        self._stop = threading.Event()
        self._thread = None
        self.samples = 0

    def _loop(self):
        os.makedirs(os.path.dirname(self.path) or ".", exist_ok=True)
        while not self._stop.is_set():
            rows = self.sampler()
            if rows:
                stamp = time.strftime("%Y-%m-%d %H:%M:%S")
                with open(self.path, "a") as f:
                    for r in rows:
                        if self.devices is None or str(r.get("index")) in self.devices:
                            f.write(stamp + " " + " ".join(f"{k}={v}" for k, v in r.items()) + "\n")
                self.samples += 1
            self._stop.wait(self.interval)

    def start(self):
        if self._thread is None:
            self._thread = threading.Thread(target=self._loop, name="pd-launch-gpu-watcher", daemon=True)
            self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(5)
            self._thread = None
