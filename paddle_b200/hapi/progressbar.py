"""Console progress line of ``Model.fit`` / ``evaluate`` / ``predict`` (python/paddle/hapi/progressbar.py:26-240)."""
from __future__ import annotations

import sys
import time


class ProgressBar:
    """``update(step, values)`` rewrites one line (``verbose=1``, on a terminal) or prints one line per call
    (``verbose=2`` / ``3``); values are ``(name, number or list)`` pairs.  ``verbose=3`` adds the reader and batch
    cost averages kept by the caller in ``values``."""

    def __init__(self, num=None, width=30, verbose=1, start=True, file=None, name="step"):
        self._num = None if (num is not None and num <= 0) else num
        self._width = width
        self._verbose = verbose
        self.file = file if file is not None else sys.stdout
        self.name = name
        self._last_len = 0
        self._dynamic = hasattr(self.file, "isatty") and self.file.isatty()
        self._start = time.time()
        self._last_update = self._start
        if start:
            self.start()

    def start(self):
        self._start = self._last_update = time.time()

    @staticmethod
    def _fmt(v):
        if isinstance(v, (list, tuple)):
            return " ".join(ProgressBar._fmt(x) for x in v)
        try:
            v = float(v)
        except (TypeError, ValueError):
            return str(v)
        if v == int(v) and abs(v) < 1e6:
            return f"{v:.4f}"
        return f"{v:.4f}" if abs(v) > 1e-3 else f"{v:.4e}"

    def _eta(self, current, now):
        per = (now - self._start) / current if current else 0.0
        if self._num is None:
            return per, None
        return per, per * (self._num - current)

    def update(self, current_num, values=()):
        now = time.time()
        per, eta = self._eta(current_num, now)
        metrics = " - ".join(f"{k}: {self._fmt(v)}" for k, v in values)
        unit = f"{per:.0f}s" if per >= 1 else (f"{per * 1e3:.0f}ms" if per >= 1e-3 else f"{per * 1e6:.0f}us")
        if self._verbose == 1:
            if self._num is not None:
                done = int(self._width * current_num / self._num)
                bar = "[" + "=" * max(done - 1, 0) + (">" if current_num < self._num else "=") + "." * (self._width - done) + "]"
                head = f"{self.name} {current_num:>{len(str(self._num))}}/{self._num} {bar}"
            else:
                head = f"{self.name} {current_num:3d}"
            line = f"{head} - {metrics} - {unit}/{self.name}"
            if eta is not None and current_num < self._num:
                line += f" - ETA: {int(eta) // 3600:d}:{int(eta) % 3600 // 60:02d}:{int(eta) % 60:02d}"
            if self._dynamic:
                self.file.write("\r" + line + " " * max(self._last_len - len(line), 0))
                if self._num is not None and current_num >= self._num:
                    self.file.write("\n")
            else:
                self.file.write(line + "\n")
            self._last_len = len(line)
        elif self._verbose in (2, 3):
            head = f"{self.name} {current_num}/{self._num}" if self._num else f"{self.name} {current_num}"
            self.file.write(f"{head} - {metrics} - {unit}/{self.name}\n")
        self.file.flush()
        self._last_update = now
