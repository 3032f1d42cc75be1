"""``paddle.Model`` (python/paddle/hapi/model.py:1050-2500): ``prepare`` / ``fit`` / ``evaluate`` / ``predict`` /
``train_batch`` / ``eval_batch`` / ``predict_batch`` / ``save`` / ``load`` / ``summary`` around a dynamic-graph
``Layer``.  Mixed precision through ``amp_configs`` (``auto_cast`` + ``GradScaler``), gradient accumulation, data
parallelism when the process group has more than one rank (``DataParallel`` + ``DistributedBatchSampler``; metrics
and evaluation losses are gathered over the ranks), callbacks through ``config_callbacks``."""
from __future__ import annotations

import contextlib
import os

import numpy as np
import torch

from ..io import DataLoader, Dataset, DistributedBatchSampler
from .callbacks import config_callbacks


def _to_list(v):
    if v is None:
        return []
    return list(v) if isinstance(v, (list, tuple)) else [v]


def _world():
    try:
        from .. import distributed as dist
        if dist.is_initialized():
            return dist.get_world_size(), dist.get_rank()
    except Exception:  # noqa: BLE001
        pass
    return 1, 0


class Model:
    def __init__(self, network, inputs=None, labels=None):
        self.network = network
        self._inputs, self._labels = _to_list(inputs) or None, _to_list(labels) or None
        self._optimizer = self._loss = None
        self._metrics = []
        self.stop_training = False
        self.mode = "train"
        self._amp_level = "O0"
        self._amp_kwargs = {}
        self._scaler = None
        self._ddp = None
        self._accumulate = 1
        self._prepared = False

    # ------------------------------------------------------------------------------------------------------ prepare
    def prepare(self, optimizer=None, loss=None, metrics=None, amp_configs=None):
        """``amp_configs``: ``"O1"`` / ``"O2"`` or a dict with ``level`` and any of ``dtype``, ``custom_white_list``,
        ``custom_black_list`` (for ``auto_cast``), ``init_loss_scaling``, ``incr_ratio``, ``decr_ratio``,
        ``incr_every_n_steps``, ``decr_every_n_nan_or_inf``, ``use_dynamic_loss_scaling`` (for ``GradScaler``)."""
        from ..metric import Metric
        self._optimizer = optimizer
        if loss is not None and not callable(loss):
            raise TypeError("'loss' must be a Layer or a callable")
        self._loss = loss
        self._metrics = _to_list(metrics)
        for m in self._metrics:
            if not isinstance(m, Metric):
                raise TypeError(f"{type(m).__name__} is not a paddle.metric.Metric")
        self._prepare_amp(amp_configs)
        world, _ = _world()
        if world > 1 and self._ddp is None:
            from ..distributed import DataParallel
            self._ddp = DataParallel(self.network)
        self._prepared = True

    def _prepare_amp(self, amp_configs):
        from .. import amp
        if amp_configs is None:
            self._amp_level, self._scaler = "O0", None
            return
        cfg = {"level": amp_configs} if isinstance(amp_configs, str) else dict(amp_configs)
        level = cfg.pop("level", "O1")
        if level not in ("O0", "O1", "O2"):
            raise ValueError("amp level must be 'O0', 'O1' or 'O2'")
        self._amp_level = level
        if level == "O0":
            self._scaler = None
            return
        scaler_keys = ("init_loss_scaling", "incr_ratio", "decr_ratio", "incr_every_n_steps", "decr_every_n_nan_or_inf", "use_dynamic_loss_scaling")
        scaler_kw = {k: cfg.pop(k) for k in scaler_keys if k in cfg}
        self._amp_kwargs = {k: cfg[k] for k in ("dtype", "custom_white_list", "custom_black_list") if k in cfg}
        unknown = set(cfg) - set(self._amp_kwargs) - {"use_fp16_guard"}
        if unknown:
            raise ValueError(f"unknown amp_configs keys: {sorted(unknown)}")
        dtype = self._amp_kwargs.get("dtype", "float16")
        if level == "O2":
            self.network, self._optimizer = amp.decorate(self.network, self._optimizer, level="O2", dtype=dtype)
        self._scaler = amp.GradScaler(**scaler_kw) if dtype == "float16" else None

    def _autocast(self):
        if self._amp_level == "O0":
            return contextlib.nullcontext()
        from .. import amp
        return amp.auto_cast(enable=True, level=self._amp_level, **self._amp_kwargs)

    # ------------------------------------------------------------------------------------------------------ batches
    def _split(self, batch):
        batch = list(batch) if isinstance(batch, (list, tuple)) else [batch]
        if self._inputs:
            n_in = len(self._inputs)
        elif self._labels:
            n_in = len(batch) - len(self._labels)
        else:
            n_in = max(len(batch) - 1, 1) if self._loss is not None or self._metrics else len(batch)
        return batch[:n_in], batch[n_in:]

    def _forward(self, ins):
        net = self._ddp if (self._ddp is not None and self.mode == "train") else self.network
        out = net(*ins)
        return list(out) if isinstance(out, (list, tuple)) else [out]

    def _update_metrics(self, outs, labs):
        res = []
        for m in self._metrics:
            r = m.compute(*outs, *labs)
            res.append(m.update(*r) if isinstance(r, (list, tuple)) else m.update(r))
        return res

    def train_batch(self, inputs, labels=None, update=True):
        """One forward + backward; the optimizer steps (and gradients are cleared) when ``update``.
        -> ([loss], metric results) or [loss] without metrics."""
        assert self._optimizer is not None and self._loss is not None, "call prepare(optimizer, loss) before training"
        self.network.train()
        self.mode = "train"
        ins, labs = _to_list(inputs), _to_list(labels)
        sync = contextlib.nullcontext()
        if self._ddp is not None and not update and hasattr(self._ddp, "no_sync"):
            sync = self._ddp.no_sync()                        # accumulate locally, all-reduce on the updating step
        with sync:
            with self._autocast():
                outs = self._forward(ins)
                loss = self._loss(*outs, *labs)
            losses = _to_list(loss)
            total = losses[0] if len(losses) == 1 else sum(losses[1:], losses[0])
            if self._accumulate > 1:
                total = total / self._accumulate
            if self._scaler is not None:
                self._scaler.scale(total).backward()
            else:
                total.backward()
        if update:
            if self._scaler is not None:
                self._scaler.step(self._optimizer)
                self._scaler.update()
            else:
                self._optimizer.step()
            self._optimizer.clear_grad()
        metrics = self._update_metrics(outs, labs)
        vals = [float(l) for l in losses]
        return (vals, metrics) if self._metrics else vals

    @torch.no_grad()
    def eval_batch(self, inputs, labels=None):
        self.network.eval()
        self.mode = "eval"
        ins, labs = _to_list(inputs), _to_list(labels)
        with self._autocast():
            outs = self._forward(ins)
            losses = [float(l) for l in _to_list(self._loss(*outs, *labs))] if self._loss is not None else []
        metrics = self._update_metrics(outs, labs)
        return (losses, metrics) if self._metrics else losses

    @torch.no_grad()
    def predict_batch(self, inputs):
        self.network.eval()
        self.mode = "test"
        with self._autocast():
            outs = self._forward(_to_list(inputs))
        return [o.float().numpy() if o.dtype in (torch.bfloat16, torch.float16) else o.numpy() for o in outs]

    # ------------------------------------------------------------------------------------------------------ loops
    def _loader(self, data, batch_size, shuffle, num_workers, drop_last=False):
        if data is None or isinstance(data, DataLoader) or not isinstance(data, Dataset):
            return data
        world, rank = _world()
        if world > 1:
            sampler = DistributedBatchSampler(data, batch_size, num_replicas=world, rank=rank, shuffle=shuffle, drop_last=drop_last)
            return DataLoader(data, batch_sampler=sampler, num_workers=num_workers)
        return DataLoader(data, batch_size=batch_size, shuffle=shuffle, num_workers=num_workers, drop_last=drop_last)

    @staticmethod
    def _len(loader):
        try:
            return len(loader)
        except TypeError:
            return None

    def _metric_names(self):
        names = ["loss"] if self._loss is not None else []
        for m in self._metrics:
            names += _to_list(m.name())
        return names

    def _metric_logs(self, logs):
        for m in self._metrics:
            for n, v in zip(_to_list(m.name()), _to_list(m.accumulate())):
                logs[n] = v
        return logs

    def fit(self, train_data=None, eval_data=None, batch_size=1, epochs=1, eval_freq=1, log_freq=10, save_dir=None, save_freq=1,
            verbose=2, drop_last=False, shuffle=True, num_workers=0, callbacks=None, accumulate_grad_batches=1, num_iters=None):
        assert train_data is not None, "train_data must be given"
        self._accumulate = max(1, int(accumulate_grad_batches))
        train = self._loader(train_data, batch_size, shuffle, num_workers, drop_last)
        evald = self._loader(eval_data, batch_size, False, num_workers)
        steps = self._len(train)
        if num_iters is not None and steps is not None:
            epochs = min(epochs, -(-num_iters // steps))
        cbks = config_callbacks(callbacks, model=self, epochs=epochs, steps=steps, log_freq=log_freq, save_freq=save_freq, save_dir=save_dir,
                                verbose=verbose, metrics=self._metric_names(), batch_size=batch_size)
        self.stop_training = False
        cbks.on_begin("train")
        it = 0
        logs = {}
        for epoch in range(epochs):
            if hasattr(getattr(train, "batch_sampler", None), "set_epoch"):
                train.batch_sampler.set_epoch(epoch)
            for m in self._metrics:
                m.reset()
            cbks.on_epoch_begin(epoch)
            logs = {}
            for step, batch in enumerate(train):
                cbks.on_batch_begin("train", step, logs)
                ins, labs = self._split(batch)
                last = steps is not None and step + 1 == steps
                update = (step + 1) % self._accumulate == 0 or last
                res = self.train_batch(ins, labs, update)
                loss = res[0] if self._metrics else res
                logs = {"loss": loss if len(loss) > 1 else loss[0], "step": step, "updated": update,
                        "batch_size": int(ins[0].shape[0]) if hasattr(ins[0], "shape") and len(ins[0].shape) else 1}
                self._metric_logs(logs)
                cbks.on_batch_end("train", step, logs)
                it += 1
                if num_iters is not None and it >= num_iters:
                    break
            cbks.on_epoch_end(epoch, logs)
            if evald is not None and (epoch + 1) % eval_freq == 0:
                eval_logs = self._run_eval(evald, cbks, None)
                cbks.on_end("eval", eval_logs)
            if self.stop_training or (num_iters is not None and it >= num_iters):
                break
        cbks.on_end("train", logs)
        self._accumulate = 1

    def _gather_mean(self, value, weight):
        world, _ = _world()
        if world == 1:
            return value
        from .. import distributed as dist
        t = torch.tensor([value * weight, weight], dtype=torch.float64)
        dev = next(iter(self.network.parameters())).device
        t = t.to(dev)
        dist.all_reduce(t)
        return float(t[0] / t[1]) if float(t[1]) else value

    def _run_eval(self, loader, cbks, num_iters):
        for m in self._metrics:
            m.reset()
        steps = self._len(loader)
        cbks.on_begin("eval", {"steps": steps if num_iters is None else min(steps or num_iters, num_iters), "metrics": self._metric_names()})
        losses, samples, logs = [], 0, {}
        for step, batch in enumerate(loader):
            cbks.on_batch_begin("eval", step, logs)
            ins, labs = self._split(batch)
            res = self.eval_batch(ins, labs)
            l = res[0] if self._metrics else res
            bs = int(ins[0].shape[0]) if hasattr(ins[0], "shape") and len(ins[0].shape) else 1
            samples += bs
            logs = {"step": step, "batch_size": bs}
            if l:
                losses.append((l[0], bs))
                logs["loss"] = l[0]
            self._metric_logs(logs)
            cbks.on_batch_end("eval", step, logs)
            if num_iters is not None and step + 1 >= num_iters:
                break
        out = {}
        if losses:
            mean = sum(v * w for v, w in losses) / max(sum(w for _, w in losses), 1)
            out["loss"] = [self._gather_mean(mean, sum(w for _, w in losses))]
        self._metric_logs(out)
        out["samples"] = samples
        return out

    def evaluate(self, eval_data, batch_size=1, log_freq=10, verbose=2, num_workers=0, callbacks=None, num_iters=None):
        loader = self._loader(eval_data, batch_size, False, num_workers)
        cbks = config_callbacks(callbacks, model=self, log_freq=log_freq, verbose=verbose, metrics=self._metric_names(), mode="eval",
                                steps=self._len(loader), batch_size=batch_size)
        logs = self._run_eval(loader, cbks, num_iters)
        cbks.on_end("eval", logs)
        logs.pop("samples", None)
        return logs

    def predict(self, test_data, batch_size=1, num_workers=0, stack_outputs=False, verbose=1, callbacks=None):
        loader = self._loader(test_data, batch_size, False, num_workers)
        cbks = config_callbacks(callbacks, model=self, verbose=verbose, metrics=[], mode="predict", steps=self._len(loader), batch_size=batch_size)
        cbks.on_begin("predict", {"steps": self._len(loader)})
        outs, samples, logs = [], 0, {}
        for step, batch in enumerate(loader):
            cbks.on_batch_begin("predict", step, logs)
            batch = list(batch) if isinstance(batch, (list, tuple)) else [batch]
            # without input specs a (inputs..., label) dataset of a model prepared with a loss drops the label
            n_in = len(self._inputs) if self._inputs else (len(batch) - len(self._labels) if self._labels else
                                                           (len(batch) - 1 if self._loss is not None and len(batch) > 1 else len(batch)))
            res = self.predict_batch(batch[:max(n_in, 1)])
            outs.append(res)
            samples += len(res[0])
            logs = {"step": step, "batch_size": len(res[0])}
            cbks.on_batch_end("predict", step, logs)
        cbks.on_end("predict", {"samples": samples})
        cols = list(zip(*outs))
        return [np.concatenate(c) if stack_outputs else list(c) for c in cols]

    # ------------------------------------------------------------------------------------------------------ persistence
    def save(self, path, training=True):
        """``training=True``: ``<path>.pdparams`` (+ ``.pdopt``) for resuming.  ``training=False``: an inference model
        through ``paddle.jit.save`` (needs ``inputs`` specs given to the constructor)."""
        _, rank = _world()
        if rank != 0:
            return
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        if not training:
            from .. import jit
            if not self._inputs:
                raise ValueError("saving an inference model needs the 'inputs' specification given to paddle.Model")
            jit.save(self.network, path, input_spec=self._inputs)
            return
        from ..framework.io import save
        save(self.network.state_dict(), path + ".pdparams")
        if self._optimizer is not None:
            save(self._optimizer.state_dict(), path + ".pdopt")

    def load(self, path, skip_mismatch=False, reset_optimizer=False):
        from ..framework.io import load
        path = path[:-len(".pdparams")] if path.endswith(".pdparams") else path
        state = load(path + ".pdparams")
        if skip_mismatch:
            own = self.network.state_dict()
            kept = {}
            for k, v in state.items():
                if k in own and tuple(np.shape(v)) == tuple(own[k].shape):
                    kept[k] = v
                else:
                    import warnings
                    warnings.warn(f"skip loading {k}: " + ("not in the model" if k not in own else f"shape {tuple(np.shape(v))} != {tuple(own[k].shape)}"))
            state = kept
        self.network.set_state_dict(state)
        if not reset_optimizer and self._optimizer is not None and os.path.exists(path + ".pdopt"):
            self._optimizer.set_state_dict(load(path + ".pdopt"))

    def parameters(self, *a, **k):
        return self.network.parameters(*a, **k)

    def summary(self, input_size=None, dtype=None):
        from .model_summary import summary
        if input_size is None and self._inputs:
            input_size = [tuple(s.shape) for s in self._inputs]
        return summary(self.network, input_size, dtype)
