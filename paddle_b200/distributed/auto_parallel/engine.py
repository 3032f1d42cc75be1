"""``Engine``: the high-level train / evaluate / predict driver of auto parallel
(python/paddle/distributed/auto_parallel/static/engine.py:80 ``Engine``; ``fit`` :1558, ``evaluate`` :1748,
``predict`` :1862, ``dataloader`` :1963, ``prepare`` :2011, ``run`` :2067, ``save`` :2349, ``load`` :2434, ``cost`` :2489).

The reference plans a serial program (completion, partitioning, reshard insertion, passes) and runs the rank-local
program on the static executor.  Here the model is a dynamic layer whose parameters may already be distributed
tensors (``shard_tensor`` / ``shard_layer`` / ``parallelize``); the engine feeds it the rank's share of every batch,
averages data-parallel gradients over the mesh dimension the data is split on, applies gradient merge, AMP and
recompute from ``Strategy``, and keeps the ``fit`` history / log dictionaries in the reference's shape
(``{"loss": [...], "<metric>": [...]}``)."""
from __future__ import annotations

import os
import time

import numpy as np
import torch

from ... import io as _io
from ..._core.tensor import as_tensor
from .. import collective as C
from .api import Strategy


def _as_list(x):
    if x is None:
        return []
    return list(x) if isinstance(x, (list, tuple)) else [x]


class Engine:
    def __init__(self, model=None, loss=None, optimizer=None, metrics=None, cluster=None, strategy=None):
        if model is not None and not callable(model):
            raise TypeError("'model' must be a paddle.nn.Layer or a callable")
        if loss is not None and not callable(loss):
            raise TypeError("'loss' must be a paddle.nn.Layer or a callable")
        if optimizer is not None and not hasattr(optimizer, "step"):
            raise TypeError("'optimizer' must be a paddle.optimizer.Optimizer")
        for m in _as_list(metrics):
            if not (hasattr(m, "compute") and hasattr(m, "update") and hasattr(m, "accumulate")):
                raise TypeError("every entry of 'metrics' must be a paddle.metric.Metric")
        if strategy is not None and not isinstance(strategy, Strategy):
            raise TypeError("'strategy' must be an auto.Strategy")
        self._model, self._loss, self._optimizer = model, loss, optimizer
        self._metrics = _as_list(metrics)
        self._cluster = cluster
        self._strategy = strategy or Strategy()
        self._mode = "train"
        self._inputs_spec = self._labels_spec = None
        self._prepared = False
        self._merge_k, self._merge_avg, self._merge_i = 1, True, 0
        self._scaler = None
        self.history = None
        self._plan = self._program = None
        self._rank = C.get_rank() if C.is_initialized() else 0
        self._world = C.get_world_size() if C.is_initialized() else 1

    # ------------------------------------------------------------------ preparation
    def prepare(self, inputs_spec=None, labels_spec=None, inputs=None, labels=None, main_program=None,
                startup_program=None, mode=None, init_parameters=True):
        """Fixes the mode and applies the strategy to the model (the reference builds and plans the program here)."""
        if mode is not None:
            self.to_mode(mode)
        self._inputs_spec, self._labels_spec = _as_list(inputs_spec), _as_list(labels_spec)
        st = self._strategy
        if st.gradient_merge.enable:
            self._merge_k = int(st.gradient_merge.get("k_steps", 1) or 1)
            self._merge_avg = bool(st.gradient_merge.get("avg", True))
        if st.amp.enable and self._scaler is None:
            from ... import amp
            self._amp_level = str(st.amp.get("level", "o1")).upper()
            self._amp_dtype = st.amp.get("dtype", "float16")
            if self._amp_dtype == "float16":
                self._scaler = amp.GradScaler(init_loss_scaling=float(st.amp.get("init_loss_scaling", 32768.0)))
        if st.recompute.enable and self._model is not None and not getattr(self._model, "_engine_recompute", False):
            from ..fleet.recompute import recompute
            fwd = self._model.forward

            def rec_forward(*a, **k):
                if torch.is_grad_enabled() and self._mode == "train":
                    return recompute(fwd, *a, **k)
                return fwd(*a, **k)
            self._model.forward = rec_forward
            self._model._engine_recompute = True
        self._prepared = True

    def to_mode(self, mode):
        if mode not in ("train", "eval", "predict"):
            raise ValueError("mode must be 'train', 'eval' or 'predict'")
        self._mode = mode
        if self._model is not None and hasattr(self._model, "train"):
            self._model.train() if mode == "train" else self._model.eval()

    # ------------------------------------------------------------------ data
    def dataloader(self, dataset, batch_size=1, shuffle=False, drop_last=False, collate_fn=None, num_workers=0,
                   use_buffer_reader=True, use_shared_memory=True, timeout=0, worker_init_fn=None, epochs=1,
                   steps_per_epoch=None, sample_split=1, mode=None, places=None):
        """Loader over this rank's share of ``dataset``: ``batch_size`` is the global batch; each data-parallel rank
        reads ``batch_size / world`` samples of every batch (engine.py:1963)."""
        if mode is not None:
            self.to_mode(mode)
        world = self._world
        if batch_size % world != 0:
            raise ValueError(f"batch_size {batch_size} must be divisible by the number of data-parallel ranks {world}")
        sampler = _io.DistributedBatchSampler(dataset, batch_size // world, num_replicas=world, rank=self._rank,
                                              shuffle=shuffle, drop_last=drop_last) if world > 1 else None
        if sampler is not None:
            return _io.DataLoader(dataset, batch_sampler=sampler, collate_fn=collate_fn, num_workers=num_workers)
        return _io.DataLoader(dataset, batch_size=batch_size, shuffle=shuffle, drop_last=drop_last,
                              collate_fn=collate_fn, num_workers=num_workers)

    def _split(self, batch, sample_split):
        batch = _as_list(batch)
        if sample_split is None:             # the input specs say how many leading fields are inputs; else all but the last
            sample_split = len(self._inputs_spec) if self._inputs_spec else (len(batch) - 1 if len(batch) > 1 else len(batch))
        return batch[:sample_split], batch[sample_split:]

    # ------------------------------------------------------------------ one step
    def _forward(self, inputs):
        if self._strategy.amp.enable:
            from ... import amp
            with amp.auto_cast(level=self._amp_level, dtype=self._amp_dtype):
                return self._model(*inputs)
        return self._model(*inputs)

    def _sync_grads(self):
        if self._world <= 1:
            return
        for p in self._optimizer._parameter_list if hasattr(self._optimizer, "_parameter_list") else self._model.parameters():
            g = getattr(p, "grad", None)
            if g is None or getattr(p, "is_distributed", False):
                continue
            C.all_reduce(g)
            g.div_(self._world)

    def _step(self, inputs, labels):
        """One batch in the current mode; returns (loss or None, outputs)."""
        if self._mode == "predict":
            with torch.no_grad():
                return None, self._forward(inputs)
        if self._mode == "eval":
            with torch.no_grad():
                out = self._forward(inputs)
                loss = self._loss(*_as_list(out), *labels) if self._loss is not None else None
            return loss, out
        out = self._forward(inputs)
        loss = self._loss(*_as_list(out), *labels)
        scaled = loss / self._merge_k if (self._merge_k > 1 and self._merge_avg) else loss
        (self._scaler.scale(scaled) if self._scaler is not None else scaled).backward()
        self._merge_i += 1
        if self._merge_i % self._merge_k == 0:
            self._sync_grads()
            if self._scaler is not None:
                self._scaler.step(self._optimizer)
                self._scaler.update()
            else:
                self._optimizer.step()
            self._optimizer.clear_grad()
            lr = getattr(self._optimizer, "_learning_rate", None)
            if hasattr(lr, "step") and getattr(self, "_lr_step_each_iter", True):
                lr.step()
        return loss.detach(), out

    def _update_metrics(self, out, labels, logs):
        for m in self._metrics:
            res = m.compute(*_as_list(out), *labels)
            m.update(*[np.asarray(r.detach().cpu() if hasattr(r, "detach") else r) for r in _as_list(res)])
            vals = _as_list(m.accumulate())
            for n, v in zip(_as_list(m.name()), vals):
                logs[n] = float(v)

    def _mean_over_ranks(self, value):
        if self._world <= 1 or value is None:
            return value
        t = torch.tensor([float(value)], dtype=torch.float32, device=C._device_for(None) if hasattr(C, "_device_for") else None)
        C.all_reduce(as_tensor(t))
        return float(t) / self._world

    # ------------------------------------------------------------------ fit / evaluate / predict
    def fit(self, train_data, train_sample_split=None, batch_size=1, epochs=1, steps_per_epoch=None, log_freq=10,
            save_dir=None, save_freq=1, valid_data=None, valid_sample_split=None, valid_freq=1, valid_steps=None,
            collate_fn=None, callbacks=None, verbose=2, nvprof_range=(-1, -1)):
        if self._loss is None or self._optimizer is None:
            raise ValueError("fit needs a loss and an optimizer")
        if not self._prepared:
            self.prepare(mode="train")
        loader = self.dataloader(train_data, batch_size, collate_fn=collate_fn, mode="train")
        history = {"loss": []}
        cbs = _as_list(callbacks)
        for cb in cbs:
            getattr(cb, "on_train_begin", lambda *a: None)({})
        for epoch in range(epochs):
            self.to_mode("train")
            for m in self._metrics:
                m.reset()
            logs, t0 = {}, time.time()
            for step, batch in enumerate(loader):
                if steps_per_epoch is not None and step >= steps_per_epoch:
                    break
                inputs, labels = self._split(batch, train_sample_split)
                loss, out = self._step(inputs, labels)
                logs = {"loss": float(loss), "epoch": epoch, "step": step}
                self._update_metrics(out, labels, logs)
                history["loss"].append(logs["loss"])
                for cb in cbs:
                    getattr(cb, "on_train_batch_end", lambda *a: None)(step, logs)
                if verbose and self._rank == 0 and log_freq and step % log_freq == 0:
                    print(f"[train] epoch {epoch} step {step} loss {logs['loss']:.6f} "
                          f"({(time.time() - t0) / (step + 1) * 1e3:.1f} ms/step)")
            for k, v in logs.items():
                if k not in ("loss", "epoch", "step"):
                    history.setdefault(k, []).append(v)
            if valid_data is not None and (epoch + 1) % valid_freq == 0:
                ev = self.evaluate(valid_data, valid_sample_split, batch_size, valid_steps, log_freq, collate_fn, None, 0)
                for k, v in ev.items():
                    history.setdefault("val_" + k, []).append(v)
            if save_dir is not None and (epoch + 1) % save_freq == 0:
                self.save(os.path.join(save_dir, f"epoch{epoch}"))
        for cb in cbs:
            getattr(cb, "on_train_end", lambda *a: None)(history)
        self.history = history
        return history

    def evaluate(self, valid_data, valid_sample_split=None, batch_size=1, steps=None, log_freq=10, collate_fn=None,
                 callbacks=None, verbose=2):
        if not self._prepared:
            self.prepare(mode="eval")
        loader = self.dataloader(valid_data, batch_size, collate_fn=collate_fn, mode="eval")
        for m in self._metrics:
            m.reset()
        logs, losses = {}, []
        for step, batch in enumerate(loader):
            if steps is not None and step >= steps:
                break
            inputs, labels = self._split(batch, valid_sample_split)
            loss, out = self._step(inputs, labels)
            if loss is not None:
                losses.append(float(loss))
            self._update_metrics(out, labels, logs)
        if losses:
            logs["loss"] = self._mean_over_ranks(float(np.mean(losses)))
        if verbose and self._rank == 0:
            print("[eval] " + " ".join(f"{k} {v:.6f}" for k, v in logs.items()))
        return logs

    def predict(self, test_data, test_sample_split=None, batch_size=1, steps=None, collate_fn=None, callbacks=None,
                verbose=2):
        if not self._prepared:
            self.prepare(mode="predict")
        loader = self.dataloader(test_data, batch_size, collate_fn=collate_fn, mode="predict")
        outputs = []
        for step, batch in enumerate(loader):
            if steps is not None and step >= steps:
                break
            inputs, _ = self._split(batch, test_sample_split)
            _, out = self._step(inputs, [])
            outputs.append([np.asarray(o.detach().cpu()) for o in _as_list(out)])
        return outputs

    def run(self, data=None, feed=None, fetch_list=None, mode=None):
        """One batch given as a list / tuple (inputs..., labels...) in the current mode; returns the log dictionary
        (``{"loss": ..., "outputs": [...]}``)."""
        if mode is not None:
            self.to_mode(mode)
        if not self._prepared:
            self.prepare(mode=self._mode)
        inputs, labels = self._split(list(feed.values()) if (data is None and feed) else data, None)
        inputs = [as_tensor(torch.as_tensor(np.asarray(x))) if not isinstance(x, torch.Tensor) else x for x in inputs]
        labels = [as_tensor(torch.as_tensor(np.asarray(x))) if not isinstance(x, torch.Tensor) else x for x in labels]
        loss, out = self._step(inputs, labels)
        logs = {"outputs": [np.asarray(o.detach().cpu()) for o in _as_list(out)]}
        if loss is not None:
            logs["loss"] = float(loss)
        return logs

    # ------------------------------------------------------------------ persistence / cost
    def save(self, path, training=True):
        """``training=True``: ``<path>.pdparams`` + ``<path>.pdopt`` of this rank (a ``_dist<rank>`` suffix is added when
        there are several ranks); otherwise an inference export through ``paddle.jit.save``."""
        from ...framework import io as framework_io
        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)
        if not training:
            from ... import jit
            jit.save(self._model, path, input_spec=self._inputs_spec or None)
            return
        suffix = f"_dist{self._rank}" if self._world > 1 else ""
        framework_io.save(self._model.state_dict(), path + suffix + ".pdparams")
        if self._optimizer is not None:
            framework_io.save(self._optimizer.state_dict(), path + suffix + ".pdopt")

    def load(self, path, strict=True, load_optimizer=True):
        from ...framework import io as framework_io
        suffix = f"_dist{self._rank}" if self._world > 1 else ""
        sd = framework_io.load(path + suffix + ".pdparams")
        missing = [k for k in self._model.state_dict() if k not in sd]
        if strict and missing:
            raise ValueError(f"checkpoint lacks parameters: {missing[:5]}")
        self._model.set_state_dict(sd)
        opt_path = path + suffix + ".pdopt"
        if load_optimizer and self._optimizer is not None and os.path.exists(opt_path):
            self._optimizer.set_state_dict(framework_io.load(opt_path))

    def plan(self, inputs_spec=None, labels_spec=None, n_devices=None, mode=None, cluster=None, memory_limit=None,
             batch_size=None):
        """Record the forward (and the loss) of the model on example tensors of the given specs, search the data / tensor
        parallel plans of the recorded program for ``n_devices`` devices (default: the cluster's, else the job's) and
        keep the best one: ``engine.main_program`` is the recorded program, ``plan.param_specs()`` the parameter
        layouts, ``plan.apply(model)`` shards the parameters accordingly.  Unknown (-1 / None) dims take
        ``batch_size`` (default 1)."""
        import paddle_b200 as paddle
        from ...static import graph as G
        from .static.cluster import Cluster, get_default_cluster
        from .static.planner import Planner
        mode = mode or self._mode
        ins = _as_list(inputs_spec) or self._inputs_spec or []
        labs = _as_list(labels_spec) or self._labels_spec or []
        if not ins:
            raise ValueError("plan() needs inputs_spec (shapes and dtypes of the model's inputs)")
        if cluster is None:
            cluster = self._cluster if isinstance(self._cluster, Cluster) else None
        if cluster is None:
            cluster = get_default_cluster(device_count=n_devices or (self._world if self._world > 1 else None))
        was_static = not paddle.in_dynamic_mode()
        paddle.enable_static()
        prog = paddle.static.Program()
        try:
            with paddle.static.program_guard(prog, paddle.static.Program()):
                def holder(sp, i, kind):
                    shape = [int(batch_size or 1) if d in (None, -1) else int(d) for d in sp.shape]
                    return paddle.static.data(sp.name or f"{kind}{i}", shape, sp.dtype)
                xs = [holder(sp, i, "input") for i, sp in enumerate(ins)]
                ys = [holder(sp, i, "label") for i, sp in enumerate(labs)]
                out = self._model(*xs)
                if self._loss is not None and ys and mode != "predict":
                    outs = out if isinstance(out, (list, tuple)) else [out]
                    self._loss(*outs, *ys)
        finally:
            if not was_static:
                paddle.disable_static()
        self._program = prog
        amp_dtype = None
        if self._strategy.amp.enable:
            amp_dtype = torch.float16 if str(self._strategy.amp.get("dtype", "float16")) == "float16" else torch.bfloat16
        planner = Planner(prog, cluster, n_devices=n_devices, mode="train" if mode == "train" else "predict",
                          memory_limit=memory_limit, assume_dtype=amp_dtype)
        self._plan = planner.plan()
        self._planner = planner
        return self._plan

    def cost(self, inputs_spec=None, labels_spec=None, mode=None):
        """(estimated step time in ms, estimated peak memory in bytes).  With input specs the model is recorded, planned
        and priced operator by operator (``plan``); without them only the memory of parameters and optimizer state is
        known and the time is ``None``."""
        mode = mode or self._mode
        specs = _as_list(inputs_spec) or self._inputs_spec or []
        if specs and self._model is not None:
            try:
                plan = self.plan(specs, _as_list(labels_spec) or self._labels_spec, mode=mode)
                return plan.cost.time * 1e3, plan.cost.memory
            except Exception as e:                                  # a model that cannot be recorded: fall back to the rough figure
                import warnings
                warnings.warn(f"Engine.cost: the model could not be planned ({type(e).__name__}: {e}); using the parameter-count estimate")
        n_param = sum(int(np.prod(p.shape)) for p in self._model.parameters())
        bytes_per = 2 if any(p.dtype in (torch.bfloat16, torch.float16) for p in self._model.parameters()) else 4
        state = n_param * (bytes_per + (12 if mode == "train" else 0))
        if not specs:
            return None, state
        tokens = int(np.prod([abs(int(s)) for s in specs[0].shape if s not in (None, -1)][:-1] or [1]))
        flops = 2.0 * n_param * tokens * (3 if mode == "train" else 1)
        peak = 1.3e15 if bytes_per == 2 else 7e13
        return flops / peak * 1e3, state

    # ------------------------------------------------------------------ introspection
    @property
    def main_program(self):
        return self._program

    startup_program = serial_main_program = serial_startup_program = main_program

    def get_dist_main_program(self, mode=None):
        """The partition of the planned program for this rank (a list of operators and collectives); ``None`` before
        ``plan``."""
        if self._plan is None:
            return None
        from .static.partitioner import Partitioner
        return Partitioner(self._plan.dist_context, self._rank).partition()

    get_dist_startup_program = get_serial_main_program = get_serial_startup_program = get_dist_main_program

    @property
    def optimizer(self):
        return self._optimizer

    @property
    def inputs(self):
        return self._inputs_spec

    @property
    def labels(self):
        return self._labels_spec

    @property
    def mode(self):
        return self._mode
