from .hapi import Callback, EarlyStopping, LRScheduler, ModelCheckpoint, ProgBarLogger  # noqa: F401


import json as _json
import os as _os

from .hapi import Callback as _Callback


class ReduceLROnPlateau(_Callback):
    """Multiplies the learning rate by ``factor`` when ``monitor`` stops improving for ``patience`` evaluations
    (python/paddle/hapi/callbacks.py ``ReduceLROnPlateau``)."""

    def __init__(self, monitor="loss", factor=0.1, patience=10, verbose=1, mode="auto", min_delta=1e-4, cooldown=0,
                 min_lr=0):
        if factor >= 1.0:
            raise ValueError("ReduceLROnPlateau does not support a factor >= 1.0.")
        self.monitor, self.factor, self.patience, self.verbose = monitor, factor, patience, verbose
        self.min_delta, self.cooldown, self.min_lr = min_delta, cooldown, min_lr
        self.less = mode == "min" or (mode == "auto" and "acc" not in monitor)
        self.best, self.wait, self.cooldown_counter = None, 0, 0

    def on_train_begin(self, logs=None):
        self.best, self.wait, self.cooldown_counter = None, 0, 0

    def on_eval_end(self, logs=None):
        v = (logs or {}).get(self.monitor)
        if v is None:
            return
        v = float(v[0] if isinstance(v, (list, tuple)) else v)
        if self.cooldown_counter > 0:
            self.cooldown_counter -= 1
            self.wait = 0
        better = self.best is None or (v < self.best - self.min_delta if self.less else v > self.best + self.min_delta)
        if better:
            self.best, self.wait = v, 0
        elif self.cooldown_counter <= 0:
            self.wait += 1
            if self.wait >= self.patience:
                opt = self.model._optimizer
                old = opt.get_lr()
                if old > self.min_lr and not hasattr(opt._learning_rate, "step"):
                    new = max(old * self.factor, self.min_lr)
                    opt.set_lr(new)
                    if self.verbose:
                        print(f"ReduceLROnPlateau reducing learning rate to {new}.")
                    self.cooldown_counter, self.wait = self.cooldown, 0


class VisualDL(_Callback):
    """Scalar logger with the reference's constructor.  The VisualDL package is not a dependency: scalars are appended
    as JSON lines to ``<log_dir>/scalars.jsonl``."""

    def __init__(self, log_dir):
        self.log_dir, self.epochs, self.steps, self.epoch = log_dir, None, None, 0
        self._step = {"train": 0, "eval": 0}

    def _write(self, mode, logs):
        _os.makedirs(self.log_dir, exist_ok=True)
        rec = {"mode": mode, "step": self._step[mode]}
        for k, v in (logs or {}).items():
            if isinstance(v, (list, tuple)) and v:
                v = v[0]
            if isinstance(v, (int, float)):
                rec[k] = float(v)
        with open(_os.path.join(self.log_dir, "scalars.jsonl"), "a") as f:
            f.write(_json.dumps(rec) + "\n")

    def on_train_batch_end(self, step, logs=None):
        self._step["train"] += 1
        self._write("train", logs)

    def on_eval_end(self, logs=None):
        self._step["eval"] += 1
        self._write("eval", logs)


class WandbCallback(VisualDL):
    """Same local scalar log as :class:`VisualDL`; the wandb service is not reachable from an offline build."""

    def __init__(self, project=None, entity=None, name=None, dir=None, mode=None, job_type=None, **kwargs):
        super().__init__(dir or "./wandb")
        self.project, self.entity, self.run_name = project, entity, name
