"""``paddle.amp``: auto_cast (O1 list-driven autocast, O2 pure low precision), decorate (cast model,
fp32 master weights in the optimizer), GradScaler with dynamic loss scaling
(python/paddle/amp/auto_cast.py:462,766; grad_scaler.py:62,657; amp_lists.py:20-108)."""
from __future__ import annotations

import contextlib

import torch

from .._core import dtype as _dt
from .._core.tensor import as_tensor
from . import debugging  # noqa: F401

# ops that stay in fp32 under O1 (subset of the reference black list that matters for torch.autocast,
# which already keeps reductions/softmax/losses in fp32)
WHITE_LIST = {"conv2d", "matmul", "linear", "einsum", "bmm", "flash_attn"}
BLACK_LIST = {"exp", "log", "softmax", "log_softmax", "cross_entropy", "layer_norm", "mean", "sum", "pow"}

_state = {"enable": False, "level": "O0", "dtype": torch.float32}


def amp_state():
    return dict(_state)


def is_float16_supported(device=None):
    return torch.cuda.is_available()


def is_bfloat16_supported(device=None):
    return True


@contextlib.contextmanager
def auto_cast(enable=True, custom_white_list=None, custom_black_list=None, level="O1", dtype="float16",
              use_promote=True):
    td = _dt.to_torch(dtype)
    prev = dict(_state)
    _state.update(enable=enable, level=level if enable else "O0", dtype=td if enable else torch.float32)
    try:
        if enable and level == "O1":
            dev = "cuda" if torch.cuda.is_available() else "cpu"
            with torch.autocast(dev, dtype=td):
                yield
        else:
            yield
    finally:
        _state.clear()
        _state.update(prev)


amp_guard = auto_cast


def decorate(models, optimizers=None, level="O1", dtype="float16", master_weight=None, save_dtype=None,
             master_grad=False, excluded_layers=None):
    """O2: cast the model's floating-point parameters to ``dtype`` (norm layers listed in
    ``excluded_layers`` keep fp32) and switch the optimizers to fp32 master weights.  With
    ``master_grad`` every parameter gets a persistent fp32 ``main_grad`` that backward accumulates into."""
    td = _dt.to_torch(dtype)
    single_model = not isinstance(models, (list, tuple))
    ms = [models] if single_model else list(models)
    if level == "O2":
        for m in ms:
            m._cast_excluding(td, excluded_layers)
            m.__dict__["_casted_by_pure_fp16"] = True
        opts = [] if optimizers is None else ([optimizers] if not isinstance(optimizers, (list, tuple)) else list(optimizers))
        for o in opts:
            if master_weight is not False:
                o._multi_precision = True
        if master_grad:
            from ..distributed.fleet.utils.mix_precision_utils import enable_main_grad
            for m in ms:
                enable_main_grad(m)
    if optimizers is None:
        return models
    return models, optimizers


amp_decorate = decorate


def _optimizer_chain(optimizer):
    """``optimizer`` and every optimizer it wraps (HybridParallelOptimizer -> sharding optimizer -> AdamW ...)."""
    chain, seen = [], set()
    o = optimizer
    while o is not None and id(o) not in seen:
        chain.append(o)
        seen.add(id(o))
        d = getattr(o, "__dict__", {})
        o = next((d[k] for k in ("_inner_opt", "_optim", "_inner_optimizer", "_optimizer", "_opt") if d.get(k) is not None),
                 None)
    return chain


class GradScaler:
    """Dynamic loss scaling: ``scale(loss)``, ``step(opt)`` (unscale + finite check + conditional
    update, all on device), ``update()``."""

    def __init__(self, enable=True, init_loss_scaling=2.0 ** 16, incr_ratio=2.0, decr_ratio=0.5,
                 incr_every_n_steps=2000, decr_every_n_nan_or_inf=1, use_dynamic_loss_scaling=True):
        self._enable = enable
        self._scale = float(init_loss_scaling)
        self._incr_ratio, self._decr_ratio = incr_ratio, decr_ratio
        self._incr_every_n_steps, self._decr_every_n = incr_every_n_steps, decr_every_n_nan_or_inf
        self._dynamic = use_dynamic_loss_scaling
        self._incr_count = self._decr_count = 0
        self._found_inf = None
        self._unscaled = False
        self._cache_founf_inf = False

    def is_enable(self):
        return self._enable

    def is_use_dynamic_loss_scaling(self):
        return self._dynamic

    def get_init_loss_scaling(self):
        return self._scale

    def set_init_loss_scaling(self, v):
        self._scale = float(v)

    def scale(self, var):
        return var * self._scale if self._enable else var

    def _grads(self, optimizer):
        out = []
        for p in optimizer._parameter_list:
            g = optimizer._grad_of(p)
            if g is not None:
                out.append(g)
        return out

    @torch.no_grad()
    def unscale_(self, optimizer):
        if not self._enable or self._unscaled:
            return
        # an optimizer facade may still hold reductions that produce gradients (sharding stage 3 finishes the
        # reduce-scatter of its last units here): they must land before anything is unscaled or checked
        pre = getattr(optimizer, "_before_unscale", None)
        if pre is not None:
            pre()
        grads = self._grads(optimizer)
        if not grads:
            # a rank without local gradients still takes part in the agreement on found_inf: the wrappers for
            # hybrid / sharded training all-reduce inside _sync_found_inf and every rank has to call it
            params = getattr(optimizer, "_parameter_list", None) or []
            dev = params[0].device if params else torch.device("cpu")
            self._found_inf = self._sync_found_inf(torch.zeros(1, dtype=torch.int32, device=dev))
            self._unscaled = True
            return
        dev = grads[0].device
        found = torch.zeros(1, dtype=torch.int32, device=dev)
        inv = torch.full((1,), 1.0 / self._scale, dtype=torch.float32, device=dev)
        if dev.type == "cuda" and all(g.is_contiguous() and g.dtype in (torch.float32, torch.bfloat16) for g in grads):
            from ..ops import native
            native.TensorTable(grads, grads).unscale_check(inv, found)
        else:
            bad = False
            for g in grads:
                g.mul_(inv.to(g.dtype))
                bad = bad or not bool(torch.isfinite(g).all())
            found.fill_(int(bad))
        self._found_inf = self._sync_found_inf(found)
        self._unscaled = True

    def _sync_found_inf(self, found):
        return found

    def step(self, optimizer):
        if not self._enable:
            return optimizer.step()
        self.unscale_(optimizer)
        # the flag has to reach the optimizer that applies the update: the hybrid / sharding wrappers delegate
        # attribute reads to the optimizer they wrap but keep what is assigned on themselves
        chain = _optimizer_chain(optimizer)
        for o in chain:
            o._skip_flag = self._found_inf
        counts = [(o, o.__dict__["_step_count"]) for o in chain if "_step_count" in getattr(o, "__dict__", {})]
        try:
            optimizer.step()
        finally:
            for o in chain:
                o._skip_flag = None
        self._cache_founf_inf = bool(self._found_inf.item()) if self._found_inf is not None else False
        if self._cache_founf_inf:
            # the update kernels left parameters and moments untouched (device-side flag); the host-side step counter
            # that feeds the bias correction must not advance either (the reference's adamw skips its beta-power
            # update under found_inf: paddle/phi/kernels/gpu/adamw_kernel.cu, skip_update)
            for o, c in counts:
                o._step_count = c

    def minimize(self, optimizer, *args, **kwargs):
        self.step(optimizer)
        self.update()

    def update(self):
        if not self._enable:
            return
        if self._dynamic:
            if self._cache_founf_inf:
                self._incr_count = 0
                self._decr_count += 1
                if self._decr_count >= self._decr_every_n:
                    self._scale = max(self._scale * self._decr_ratio, 1.0)
                    self._decr_count = 0
            else:
                self._decr_count = 0
                self._incr_count += 1
                if self._incr_count >= self._incr_every_n_steps:
                    self._scale *= self._incr_ratio
                    self._incr_count = 0
        self._unscaled = False
        self._found_inf = None

    def state_dict(self):
        return {"scale": self._scale, "incr_ratio": self._incr_ratio, "decr_ratio": self._decr_ratio,
                "incr_every_n_steps": self._incr_every_n_steps, "decr_every_n_nan_or_inf": self._decr_every_n,
                "incr_count": self._incr_count, "decr_count": self._decr_count,
                "use_dynamic_loss_scaling": self._dynamic} if self._enable else {}

    def load_state_dict(self, sd):
        if not sd:
            return
        self._scale = float(sd["scale"]) if not hasattr(sd["scale"], "item") else float(sd["scale"].item())
        self._incr_ratio, self._decr_ratio = sd["incr_ratio"], sd["decr_ratio"]
        self._incr_every_n_steps, self._decr_every_n = sd["incr_every_n_steps"], sd["decr_every_n_nan_or_inf"]
        self._incr_count, self._decr_count = sd.get("incr_count", 0), sd.get("decr_count", 0)
        self._dynamic = sd.get("use_dynamic_loss_scaling", True)


AmpScaler = GradScaler
