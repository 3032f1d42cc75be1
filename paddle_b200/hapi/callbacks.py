"""Callbacks of ``paddle.Model`` (python/paddle/hapi/callbacks.py:33-1400): the hook protocol, ``CallbackList`` /
``config_callbacks`` that assemble the default set, progress logging, checkpoints, learning-rate stepping, early
stopping, plateau-based decay and scalar logging."""
from __future__ import annotations

import json
import numbers
import os
import time

from .progressbar import ProgressBar


class Callback:
    """Hooks called by ``Model.fit`` / ``evaluate`` / ``predict``.  ``self.model`` is the ``paddle.Model``;
    ``self.params`` holds ``batch_size, epochs, steps, verbose, metrics, save_dir, save_freq, log_freq``."""

    def __init__(self):
        self.model = None
        self.params = {}

    def set_params(self, params):
        self.params = params

    def set_model(self, model):
        self.model = model

    def on_train_begin(self, logs=None): ...
    def on_train_end(self, logs=None): ...
    def on_eval_begin(self, logs=None): ...
    def on_eval_end(self, logs=None): ...
    def on_predict_begin(self, logs=None): ...
    def on_predict_end(self, logs=None): ...
    def on_epoch_begin(self, epoch, logs=None): ...
    def on_epoch_end(self, epoch, logs=None): ...
    def on_train_batch_begin(self, step, logs=None): ...
    def on_train_batch_end(self, step, logs=None): ...
    def on_eval_batch_begin(self, step, logs=None): ...
    def on_eval_batch_end(self, step, logs=None): ...
    def on_predict_batch_begin(self, step, logs=None): ...
    def on_predict_batch_end(self, step, logs=None): ...


class CallbackList:
    def __init__(self, callbacks=None):
        self.callbacks = list(callbacks or [])
        self.params = {}
        self.model = None

    def append(self, callback):
        self.callbacks.append(callback)

    def __iter__(self):
        return iter(self.callbacks)

    def set_params(self, params):
        self.params = params
        for c in self.callbacks:
            c.set_params(params)

    def set_model(self, model):
        self.model = model
        for c in self.callbacks:
            c.set_model(model)

    def _call(self, name, *args):
        for c in self.callbacks:
            getattr(c, name)(*args)

    def on_begin(self, mode, logs=None):
        self._call(f"on_{mode}_begin", logs)

    def on_end(self, mode, logs=None):
        self._call(f"on_{mode}_end", logs)

    def on_epoch_begin(self, epoch=None, logs=None):
        self._call("on_epoch_begin", epoch, logs)

    def on_epoch_end(self, epoch=None, logs=None):
        self._call("on_epoch_end", epoch, logs)

    def on_batch_begin(self, mode, step=None, logs=None):
        self._call(f"on_{mode}_batch_begin", step, logs)

    def on_batch_end(self, mode, step=None, logs=None):
        self._call(f"on_{mode}_batch_end", step, logs)


def config_callbacks(callbacks=None, model=None, batch_size=None, epochs=None, steps=None, log_freq=2, verbose=2, save_freq=1,
                     save_dir=None, metrics=None, mode="train"):
    """User callbacks plus the defaults that are not already among them: a progress logger, a checkpoint writer
    (training with ``save_dir``) and a learning-rate stepper (training)."""
    cbks = list(callbacks) if isinstance(callbacks, (list, tuple)) else ([callbacks] if callbacks is not None else [])
    if not any(isinstance(c, ProgBarLogger) for c in cbks) and verbose:
        cbks = [ProgBarLogger(log_freq, verbose=verbose)] + cbks
    if not any(isinstance(c, ModelCheckpoint) for c in cbks) and mode == "train" and save_dir:
        cbks.append(ModelCheckpoint(save_freq, save_dir))
    if not any(isinstance(c, LRScheduler) for c in cbks) and mode == "train":
        cbks.append(LRScheduler())
    lst = CallbackList(cbks)
    lst.set_model(model)
    lst.set_params({"batch_size": batch_size, "epochs": epochs, "steps": steps, "verbose": verbose, "log_freq": log_freq,
                    "save_freq": save_freq, "save_dir": save_dir, "metrics": list(metrics or ["loss"])})
    return lst


def _scalar(v):
    if isinstance(v, (list, tuple)) and v:
        v = v[0]
    try:
        return float(v)
    except (TypeError, ValueError):
        return None


class ProgBarLogger(Callback):
    """Prints the loss and metrics every ``log_freq`` steps: ``verbose`` 0 silent, 1 one rewritten bar per epoch,
    2 one line per report, 3 also the average reader / batch cost and samples per second."""

    def __init__(self, log_freq=1, verbose=2):
        super().__init__()
        self.log_freq, self.verbose = log_freq, verbose
        self.epochs = self.steps = None
        self.epoch = 0
        self.progbar = None

    def _is_print(self):
        return self.verbose and int(os.environ.get("PADDLE_TRAINER_ID", os.environ.get("RANK", 0))) == 0

    def _values(self, logs, timing):
        vals = [(k, (logs or {})[k]) for k in self.params.get("metrics", []) if k in (logs or {})]
        if not vals:
            vals = [(k, v) for k, v in (logs or {}).items() if _scalar(v) is not None and k not in ("batch_size", "step")]
        if self.verbose == 3 and timing["count"]:
            n = timing["count"]
            vals += [("avg_reader_cost", timing["data"] / n), ("avg_batch_cost", timing["batch"] / n)]
            if timing["batch"] > 0:
                vals.append(("avg_samples", timing["samples"] / n))
                vals.append(("ips", timing["samples"] / timing["batch"]))
        return vals

    def _begin(self, steps, name):
        self.progbar = ProgressBar(num=steps, verbose=self.verbose, name=name)
        self._timing = {"data": 0.0, "batch": 0.0, "count": 0, "samples": 0, "t": time.time()}

    def _batch_begin(self):
        now = time.time()
        self._timing["data"] += now - self._timing["t"]
        self._timing["t0"] = self._timing["t"]

    def _batch_end(self, step, logs):
        now = time.time()
        t = self._timing
        t["batch"] += now - t.get("t0", t["t"])
        t["count"] += 1
        t["samples"] += (logs or {}).get("batch_size", 0) or 0
        t["t"] = now
        if self._is_print() and ((step + 1) % self.log_freq == 0 or (self.progbar._num and step + 1 == self.progbar._num)):
            self.progbar.update(step + 1, self._values(logs, t))
            t.update(data=0.0, batch=0.0, count=0, samples=0)

    # train
    def on_train_begin(self, logs=None):
        self.epochs, self.steps = self.params.get("epochs"), self.params.get("steps")

    def on_epoch_begin(self, epoch=None, logs=None):
        self.epoch = epoch or 0
        if self._is_print() and self.epochs:
            print(f"Epoch {self.epoch + 1}/{self.epochs}")
        self._begin(self.steps, "step")

    def on_train_batch_begin(self, step, logs=None):
        self._batch_begin()

    def on_train_batch_end(self, step, logs=None):
        self._batch_end(step, logs)

    # eval
    def on_eval_begin(self, logs=None):
        self.eval_steps = (logs or {}).get("steps")
        self._begin(self.eval_steps, "step")
        if self._is_print():
            print("Eval begin...")

    def on_eval_batch_begin(self, step, logs=None):
        self._batch_begin()

    def on_eval_batch_end(self, step, logs=None):
        self._batch_end(step, logs)

    def on_eval_end(self, logs=None):
        if self._is_print():
            vals = " - ".join(f"{k}: {ProgressBar._fmt(v)}" for k, v in (logs or {}).items() if _scalar(v) is not None and k != "samples")
            print(f"Eval samples: {(logs or {}).get('samples', '?')}" + (f" - {vals}" if vals else ""))

    # predict
    def on_predict_begin(self, logs=None):
        self._begin((logs or {}).get("steps"), "step")
        if self._is_print():
            print("Predict begin...")

    def on_predict_batch_begin(self, step, logs=None):
        self._batch_begin()

    def on_predict_batch_end(self, step, logs=None):
        self._batch_end(step, logs)

    def on_predict_end(self, logs=None):
        if self._is_print():
            print(f"Predict samples: {(logs or {}).get('samples', '?')}")


class ModelCheckpoint(Callback):
    """Saves ``<save_dir>/<epoch>`` every ``save_freq`` epochs and ``<save_dir>/final`` at the end (rank 0 only)."""

    def __init__(self, save_freq=1, save_dir=None):
        super().__init__()
        self.save_freq, self.save_dir = save_freq, save_dir
        self.epoch = 0

    def _is_save(self):
        return self.model is not None and self.save_dir and int(os.environ.get("PADDLE_TRAINER_ID", os.environ.get("RANK", 0))) == 0

    def on_epoch_begin(self, epoch=None, logs=None):
        self.epoch = epoch or 0

    def on_epoch_end(self, epoch, logs=None):
        if self._is_save() and (self.epoch + 1) % self.save_freq == 0:
            self.model.save(os.path.join(self.save_dir, str(epoch)))

    def on_train_end(self, logs=None):
        if self._is_save():
            self.model.save(os.path.join(self.save_dir, "final"))


class LRScheduler(Callback):
    """Steps the optimizer's learning-rate scheduler after every optimizer update (``by_step``) or every epoch."""

    def __init__(self, by_step=True, by_epoch=False):
        super().__init__()
        if by_step and by_epoch:
            raise ValueError("by_step option is mutually exclusive with by_epoch")
        self.by_step, self.by_epoch = by_step, by_epoch

    def _step(self):
        opt = getattr(self.model, "_optimizer", None)
        lr = getattr(opt, "_learning_rate", None)
        if hasattr(lr, "step"):
            lr.step()

    def on_train_batch_end(self, step, logs=None):
        if self.by_step and (logs or {}).get("updated", True):
            self._step()

    def on_epoch_end(self, epoch, logs=None):
        if self.by_epoch:
            self._step()


class _Monitor(Callback):
    def _init_monitor(self, monitor, mode, min_delta):
        self.monitor = monitor
        if mode not in ("auto", "min", "max"):
            mode = "auto"
        self.less = mode == "min" or (mode == "auto" and "acc" not in monitor)
        self.min_delta = abs(min_delta)

    def _better(self, v, best):
        return best is None or (v < best - self.min_delta if self.less else v > best + self.min_delta)


class EarlyStopping(_Monitor):
    """Stops training when ``monitor`` (an evaluation result) has not improved for more than ``patience``
    evaluations; keeps the best weights in ``<save_dir>/best_model`` when ``save_best_model``."""

    def __init__(self, monitor="loss", mode="auto", patience=0, verbose=1, min_delta=0, baseline=None, save_best_model=True):
        super().__init__()
        self._init_monitor(monitor, mode, min_delta)
        self.patience, self.verbose, self.baseline, self.save_best_model = patience, verbose, baseline, save_best_model
        self.best, self.wait, self.stopped_epoch = baseline, 0, 0

    def on_train_begin(self, logs=None):
        self.best, self.wait = self.baseline, 0

    def on_eval_end(self, logs=None):
        v = _scalar((logs or {}).get(self.monitor))
        if v is None:
            return
        if self._better(v, self.best):
            self.best, self.wait = v, 0
            save_dir = self.params.get("save_dir")
            if self.save_best_model and save_dir:
                self.model.save(os.path.join(save_dir, "best_model"))
        else:
            self.wait += 1
            if self.wait > self.patience:
                self.model.stop_training = True
                if self.verbose:
                    print(f"Early stopping: {self.monitor} has not improved on {self.best} for {self.wait} evaluations.")


class ReduceLROnPlateau(_Monitor):
    """Multiplies the learning rate by ``factor`` when ``monitor`` stops improving for ``patience`` evaluations."""

    def __init__(self, monitor="loss", factor=0.1, patience=10, verbose=1, mode="auto", min_delta=1e-4, cooldown=0, min_lr=0):
        super().__init__()
        if factor >= 1.0:
            raise ValueError("ReduceLROnPlateau does not support a factor >= 1.0.")
        self._init_monitor(monitor, mode, min_delta)
        self.factor, self.patience, self.verbose, self.cooldown, self.min_lr = factor, patience, verbose, cooldown, min_lr
        self.best, self.wait, self.cooldown_counter = None, 0, 0

    def on_train_begin(self, logs=None):
        self.best, self.wait, self.cooldown_counter = None, 0, 0

    def on_eval_end(self, logs=None):
        v = _scalar((logs or {}).get(self.monitor))
        if v is None:
            return
        if self.cooldown_counter > 0:
            self.cooldown_counter -= 1
            self.wait = 0
        if self._better(v, self.best):
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


class VisualDL(Callback):
    """Scalar logger with the reference's constructor.  The VisualDL package is not a dependency: scalars are appended
    as JSON lines to ``<log_dir>/scalars.jsonl``."""

    def __init__(self, log_dir):
        super().__init__()
        self.log_dir, self.epochs, self.steps, self.epoch = log_dir, None, None, 0
        self._step = {"train": 0, "eval": 0}

    def _write(self, mode, logs):
        os.makedirs(self.log_dir, exist_ok=True)
        rec = {"mode": mode, "step": self._step[mode]}
        for k, v in (logs or {}).items():
            s = _scalar(v)
            if s is not None and isinstance(s, numbers.Number):
                rec[k] = s
        with open(os.path.join(self.log_dir, "scalars.jsonl"), "a") as f:
            f.write(json.dumps(rec) + "\n")

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
