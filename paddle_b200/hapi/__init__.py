"""``paddle.Model`` high-level API (python/paddle/hapi/model.py, callbacks.py): prepare / fit / evaluate /
predict / save / load, callbacks, ``summary`` and ``flops``."""
from __future__ import annotations

import os
import time

import numpy as np
import torch

from ..io import DataLoader, Dataset


class Callback:
    def set_params(self, params):
        self.params = params

    def set_model(self, model):
        self.model = model

    def on_train_begin(self, logs=None): pass
    def on_train_end(self, logs=None): pass
    def on_epoch_begin(self, epoch, logs=None): pass
    def on_epoch_end(self, epoch, logs=None): pass
    def on_train_batch_begin(self, step, logs=None): pass
    def on_train_batch_end(self, step, logs=None): pass
    def on_eval_begin(self, logs=None): pass
    def on_eval_end(self, logs=None): pass


class ProgBarLogger(Callback):
    def __init__(self, log_freq=1, verbose=2):
        self.log_freq, self.verbose = log_freq, verbose

    def on_epoch_begin(self, epoch, logs=None):
        self.epoch, self.t0 = epoch, time.time()

    def on_train_batch_end(self, step, logs=None):
        if self.verbose and step % self.log_freq == 0:
            items = " - ".join(f"{k}: {v:.4f}" if isinstance(v, float) else f"{k}: {v}" for k, v in (logs or {}).items())
            print(f"Epoch {self.epoch} step {step} - {items}")


class ModelCheckpoint(Callback):
    def __init__(self, save_freq=1, save_dir=None):
        self.save_freq, self.save_dir = save_freq, save_dir

    def on_epoch_end(self, epoch, logs=None):
        if self.save_dir and epoch % self.save_freq == 0:
            self.model.save(os.path.join(self.save_dir, str(epoch)))

    def on_train_end(self, logs=None):
        if self.save_dir:
            self.model.save(os.path.join(self.save_dir, "final"))


class LRScheduler(Callback):
    def __init__(self, by_step=True, by_epoch=False):
        self.by_step, self.by_epoch = by_step, by_epoch

    def _step(self):
        lr = getattr(self.model._optimizer, "_learning_rate", None)
        if hasattr(lr, "step"):
            lr.step()

    def on_train_batch_end(self, step, logs=None):
        if self.by_step:
            self._step()

    def on_epoch_end(self, epoch, logs=None):
        if self.by_epoch:
            self._step()


class EarlyStopping(Callback):
    def __init__(self, monitor="loss", mode="auto", patience=0, verbose=1, min_delta=0, baseline=None,
                 save_best_model=True):
        self.monitor, self.patience, self.min_delta = monitor, patience, min_delta
        self.less = mode == "min" or (mode == "auto" and "acc" not in monitor)
        self.best, self.wait = None, 0

    def on_eval_end(self, logs=None):
        v = (logs or {}).get(self.monitor)
        if v is None:
            return
        v = v[0] if isinstance(v, (list, tuple)) else v
        better = self.best is None or (v < self.best - self.min_delta if self.less else v > self.best + self.min_delta)
        if better:
            self.best, self.wait = v, 0
        else:
            self.wait += 1
            if self.wait > self.patience:
                self.model.stop_training = True


class Model:
    def __init__(self, network, inputs=None, labels=None):
        self.network = network
        self._inputs, self._labels = inputs, labels
        self._optimizer = self._loss = None
        self._metrics = []
        self.stop_training = False

    def prepare(self, optimizer=None, loss=None, metrics=None, amp_configs=None):
        self._optimizer, self._loss = optimizer, loss
        self._metrics = [] if metrics is None else (list(metrics) if isinstance(metrics, (list, tuple)) else [metrics])

    def _split(self, batch):
        batch = list(batch) if isinstance(batch, (list, tuple)) else [batch]
        n_in = len(self._inputs) if self._inputs else max(len(batch) - 1, 1)
        return batch[:n_in], batch[n_in:]

    def train_batch(self, inputs, labels=None, update=True):
        self.network.train()
        ins = inputs if isinstance(inputs, (list, tuple)) else [inputs]
        labs = [] if labels is None else (labels if isinstance(labels, (list, tuple)) else [labels])
        out = self.network(*ins)
        outs = out if isinstance(out, (list, tuple)) else [out]
        loss = self._loss(*outs, *labs)
        loss.backward()
        if update:
            self._optimizer.step()
            self._optimizer.clear_grad()
        metrics = [m.update(m.compute(*outs, *labs)) for m in self._metrics]
        return [float(loss)], metrics

    @torch.no_grad()
    def eval_batch(self, inputs, labels=None):
        self.network.eval()
        ins = inputs if isinstance(inputs, (list, tuple)) else [inputs]
        labs = [] if labels is None else (labels if isinstance(labels, (list, tuple)) else [labels])
        out = self.network(*ins)
        outs = out if isinstance(out, (list, tuple)) else [out]
        loss = [float(self._loss(*outs, *labs))] if self._loss else []
        metrics = [m.update(m.compute(*outs, *labs)) for m in self._metrics]
        return loss, metrics

    @torch.no_grad()
    def predict_batch(self, inputs):
        self.network.eval()
        ins = inputs if isinstance(inputs, (list, tuple)) else [inputs]
        out = self.network(*ins)
        return [o.numpy() for o in (out if isinstance(out, (list, tuple)) else [out])]

    def _loader(self, data, batch_size, shuffle, num_workers, drop_last=False):
        if data is None or isinstance(data, DataLoader):
            return data
        return DataLoader(data, batch_size=batch_size, shuffle=shuffle, num_workers=num_workers, drop_last=drop_last)

    def fit(self, train_data=None, eval_data=None, batch_size=1, epochs=1, eval_freq=1, log_freq=10, save_dir=None,
            save_freq=1, verbose=2, drop_last=False, shuffle=True, num_workers=0, callbacks=None,
            accumulate_grad_batches=1, num_iters=None):
        train = self._loader(train_data, batch_size, shuffle, num_workers, drop_last)
        evald = self._loader(eval_data, batch_size, False, num_workers)
        cbs = list(callbacks or []) + [ProgBarLogger(log_freq, verbose)]
        if save_dir:
            cbs.append(ModelCheckpoint(save_freq, save_dir))
        if not any(isinstance(c, LRScheduler) for c in cbs):
            cbs.append(LRScheduler())
        for c in cbs:
            c.set_model(self)
        [c.on_train_begin() for c in cbs]
        it = 0
        for epoch in range(epochs):
            [m.reset() for m in self._metrics]
            [c.on_epoch_begin(epoch) for c in cbs]
            logs = {}
            for step, batch in enumerate(train):
                ins, labs = self._split(batch)
                update = (step + 1) % accumulate_grad_batches == 0
                loss, _ = self.train_batch(ins, labs, update)
                logs = {"loss": loss[0]}
                for m in self._metrics:
                    names = m.name() if isinstance(m.name(), list) else [m.name()]
                    acc = m.accumulate()
                    for n, v in zip(names, acc if isinstance(acc, list) else [acc]):
                        logs[n] = v
                [c.on_train_batch_end(step, logs) for c in cbs]
                it += 1
                if num_iters and it >= num_iters:
                    break
            [c.on_epoch_end(epoch, logs) for c in cbs]
            if evald is not None and (epoch + 1) % eval_freq == 0:
                elogs = self.evaluate(evald, verbose=0)
                [c.on_eval_end(elogs) for c in cbs]
            if self.stop_training or (num_iters and it >= num_iters):
                break
        [c.on_train_end() for c in cbs]

    def evaluate(self, eval_data, batch_size=1, log_freq=10, verbose=2, num_workers=0, callbacks=None, num_iters=None):
        loader = self._loader(eval_data, batch_size, False, num_workers)
        [m.reset() for m in self._metrics]
        losses = []
        for i, batch in enumerate(loader):
            ins, labs = self._split(batch)
            l, _ = self.eval_batch(ins, labs)
            losses += l
            if num_iters and i + 1 >= num_iters:
                break
        logs = {"loss": [float(np.mean(losses))]} if losses else {}
        for m in self._metrics:
            names = m.name() if isinstance(m.name(), list) else [m.name()]
            acc = m.accumulate()
            for n, v in zip(names, acc if isinstance(acc, list) else [acc]):
                logs[n] = v
        return logs

    def predict(self, test_data, batch_size=1, num_workers=0, stack_outputs=False, verbose=1, callbacks=None):
        loader = self._loader(test_data, batch_size, False, num_workers)
        outs = []
        for batch in loader:
            ins, _ = self._split(batch) if isinstance(batch, (list, tuple)) and len(batch) > 1 else ([batch] if not isinstance(batch, (list, tuple)) else list(batch), [])
            outs.append(self.predict_batch(ins))
        res = list(zip(*outs))
        return [np.concatenate(r) if stack_outputs else list(r) for r in res]

    def save(self, path, training=True):
        from ..framework.io import save
        save(self.network.state_dict(), path + ".pdparams")
        if training and self._optimizer is not None:
            save(self._optimizer.state_dict(), path + ".pdopt")

    def load(self, path, skip_mismatch=False, reset_optimizer=False):
        from ..framework.io import load
        self.network.set_state_dict(load(path + ".pdparams"))
        if not reset_optimizer and self._optimizer is not None and os.path.exists(path + ".pdopt"):
            self._optimizer.set_state_dict(load(path + ".pdopt"))

    def parameters(self, *a, **k):
        return self.network.parameters(*a, **k)

    def summary(self, input_size=None, dtype=None):
        return summary(self.network, input_size, dtype)


def summary(net, input_size=None, dtypes=None, input=None):
    total = sum(int(torch.Tensor.numel(p)) for p in net.parameters())
    trainable = sum(int(torch.Tensor.numel(p)) for p in net.parameters() if p.requires_grad)
    lines = [f"{'Layer':40s} {'Params':>14s}"]
    for name, l in net.named_sublayers():
        n = sum(int(torch.Tensor.numel(p)) for p in l.parameters(include_sublayers=False))
        if n:
            lines.append(f"{name + ' (' + type(l).__name__ + ')':40s} {n:>14,d}")
    lines.append(f"Total params: {total:,d}\nTrainable params: {trainable:,d}\nNon-trainable params: {total - trainable:,d}")
    print("\n".join(lines))
    return {"total_params": total, "trainable_params": trainable}


def flops(net, input_size, custom_ops=None, print_detail=False):
    """Multiply-accumulate based FLOPs of Linear / Conv layers for one forward pass."""
    from ..nn.layer import common as L
    total = [0]
    hooks = []

    def lin(l, i, o):
        total[0] += 2 * int(np.prod(o.shape)) * l.weight.shape[0]

    def conv(l, i, o):
        total[0] += 2 * int(np.prod(o.shape)) * int(np.prod(l.weight.shape[1:]))
    for l in net.sublayers(include_self=True):
        if isinstance(l, L.Linear):
            hooks.append(l.register_forward_post_hook(lin))
        elif isinstance(l, L._ConvNd):
            hooks.append(l.register_forward_post_hook(conv))
    import paddle_b200 as paddle
    with torch.no_grad():
        net(paddle.zeros(list(input_size)))
    for h in hooks:
        h.remove()
    if print_detail:
        print(f"Total FLOPs: {total[0]:,d}")
    return total[0]
