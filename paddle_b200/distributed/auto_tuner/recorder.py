"""History of the configurations that were run (python/paddle/distributed/auto_tuner/recorder.py:23-180)."""
from __future__ import annotations

import csv
import os


class HistoryRecorder:
    def __init__(self, tuner_cfg=None, metric=None, direction=None):
        tuner_cfg = tuner_cfg if isinstance(tuner_cfg, dict) else {}
        mc = tuner_cfg.get("metric_cfg", {})
        self.tuner_cfg = tuner_cfg
        self.metric = metric or mc.get("name", "tokens_per_second")
        d = (direction or mc.get("OptimizationDirection", "max")).lower()
        self.direction = "max" if d.startswith("max") else "min"
        self.search_algo = tuner_cfg.get("search_algo", {}).get("name", "grid")
        self.history = []
        self.store_path = None
        self.additional_metric_key = None

    def add_cfg(self, **cfg):
        cur = dict(cfg)
        cur.setdefault("job_id", len(self.history) + 1)
        self.history.append(cur)

    def sort_metric(self, direction=None, metric_name=None):
        direction = direction or self.direction
        metric_name = metric_name or self.metric
        ok = [h for h in self.history if isinstance(h.get(metric_name), (int, float)) and not h.get("error_info")]
        bad = [h for h in self.history if h not in ok]
        ok.sort(key=lambda h: h[metric_name], reverse=direction.lower().startswith("max"))
        self.history = ok + bad
        return ok

    def get_best(self, metric=None, direction=None, buffer=None, max_mem_usage=None):
        """``(best configuration, True when there is none)``.  With ``buffer`` (GB) configurations whose measured
        ``max_mem_usage`` comes within that margin of the limit are passed over."""
        ranked = self.sort_metric(direction, metric)
        for h in ranked:
            if buffer is not None and max_mem_usage is not None and isinstance(h.get("max_mem_usage"), (int, float)):
                if h["max_mem_usage"] > max_mem_usage - buffer:
                    continue
            return h, False
        return None, True

    def _store_history_impl(self, data, path="./history.csv"):
        keys = []
        for h in data:
            for k in h:
                if k not in keys:
                    keys.append(k)
        with open(path, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=keys)
            w.writeheader()
            for h in data:
                w.writerow({k: ("" if v is None else v) for k, v in h.items()})

    def store_history(self, path="./history.csv"):
        self.store_path = path
        self._store_history_impl(self.history, path)

    def load_history(self, path="./history.csv"):
        """``(history, True when the file does not exist)``; numbers and booleans are converted back."""
        if not os.path.exists(path):
            return [], True
        out = []
        with open(path) as f:
            for row in csv.DictReader(f):
                conv = {}
                for k, v in row.items():
                    if v == "":
                        conv[k] = None
                    elif v in ("True", "False"):
                        conv[k] = v == "True"
                    else:
                        try:
                            conv[k] = int(v)
                        except ValueError:
                            try:
                                conv[k] = float(v)
                            except ValueError:
                                conv[k] = v
                out.append(conv)
        self.history = out
        return out, False

    def clean_history(self):
        self.history = []
