"""Sharding stage 1 (optimizer-state sharding) inside hybrid parallelism
(python/paddle/distributed/fleet/meta_optimizers/dygraph_optimizer/dygraph_sharding_optimizer.py).

V1 (``DygraphShardingOptimizer`` :54): parameters are assigned to ranks by a greedy size-balanced
partition (:256-290); gradients are ``reduce``d to their owner (:326-375); each rank updates only its own
parameters and then broadcasts them (:384-450).

V2 (``DygraphShardingOptimizerV2`` :592, ``split_param=True``): every parameter is laid out in a flat
buffer with 256-byte-aligned slots; rank r owns the contiguous slice ``[r*shard, (r+1)*shard)``; gradients
are reduce-scattered per buffer, the update runs on the slice with the flat AdamW kernel, and the updated
bf16/fp32 parameter buffer is all-gathered back.
"""
from __future__ import annotations

import math

import torch

from ....._core.tensor import as_tensor
from .... import collective as C
from .....framework.flags import flag


def _numel(p):
    return int(torch.Tensor.numel(p))


class DygraphShardingOptimizer:
    def __init__(self, optimizer, hcg):
        self._inner_opt = optimizer
        self._hcg = hcg
        self._sharding_world_size = hcg.get_sharding_parallel_world_size()
        self._sharding_rank = hcg.get_sharding_parallel_rank()
        self._group = hcg.get_sharding_parallel_group()
        self._parameter_list = list(optimizer._parameter_list)
        self._rank2params = self._partition_parameters()
        self._param2rank = {p.name: r for r, ps in self._rank2params.items() for p in ps}
        local = self._rank2params[self._sharding_rank]
        self._local_names = {p.name for p in local}
        # the inner optimizer only ever sees (and keeps state for) the local parameters
        self._origin_groups = optimizer._param_groups
        optimizer._param_groups = [{**g, "params": [p for p in g["params"] if p.name in self._local_names]}
                                   for g in optimizer._param_groups]
        optimizer._parameter_list = [p for g in optimizer._param_groups for p in g["params"]]

    def _partition_parameters(self):
        mapping = {r: [] for r in range(self._sharding_world_size)}
        sizes = [0] * self._sharding_world_size
        params = self._parameter_list
        if flag("sharding_sort_parameters"):
            params = sorted(params, key=_numel, reverse=True)
        for p in params:
            r = sizes.index(min(sizes))
            mapping[r].append(p)
            sizes[r] += _numel(p)
        return mapping

    @staticmethod
    def _grad(p):
        mg = getattr(p, "main_grad", None)
        return mg if mg is not None else torch.Tensor.grad.__get__(p)

    def reduce_gradients(self, parameter_list, hcg):
        for p in parameter_list:
            g = self._grad(p)
            if g is None:
                continue
            owner = self._group.ranks[self._param2rank[p.name]]
            C.reduce(g, dst=owner, op=C.ReduceOp.AVG, group=self._group)

    def _sharding_sync_parameters(self):
        with torch.no_grad():
            for r, ps in self._rank2params.items():
                src = self._group.ranks[r]
                for p in ps:
                    C.broadcast(p.data, src, self._group)

    def step(self):
        self._inner_opt.step()
        self._sharding_sync_parameters()

    def clear_grad(self, set_to_zero=True):
        for p in self._parameter_list:
            if set_to_zero:
                g = torch.Tensor.grad.__get__(p)
                if g is not None:
                    g.zero_()
                if getattr(p, "main_grad", None) is not None:
                    p.main_grad.zero_()
            else:
                p.grad = None

    def state_dict(self):
        return self._inner_opt.state_dict()

    def set_state_dict(self, sd):
        keep = {}
        for k, v in sd.items():
            if k in ("master_weights",):
                keep[k] = {n: t for n, t in v.items() if n in self._local_names}
            elif k == "LR_Scheduler" or any(str(k).startswith(n + "_") for n in self._local_names):
                keep[k] = v
        return self._inner_opt.set_state_dict(keep)

    def __getattr__(self, item):
        return getattr(self._inner_opt, item)


ALIGN_BYTES = 256


class DygraphShardingOptimizerV2:
    """Flat-buffer sharding: reduce-scatter grads -> slice update -> all-gather params."""

    def __init__(self, optimizer, hcg):
        self._inner_opt = optimizer
        self._hcg = hcg
        self._group = hcg.get_sharding_parallel_group()
        self._n = hcg.get_sharding_parallel_world_size()
        self._rank = hcg.get_sharding_parallel_rank()
        self._parameter_list = [p for p in optimizer._parameter_list if p.requires_grad]
        self._step_count = 0
        self._build_buffers()

    def _build_buffers(self):
        by_dtype = {}
        for p in self._parameter_list:
            by_dtype.setdefault(p.dtype, []).append(p)
        self._buffers = []
        for dtype, params in by_dtype.items():
            es = torch.empty(0, dtype=dtype).element_size()
            align = max(ALIGN_BYTES // es, 1) * self._n     # every slot is a multiple of 256 B x nranks
            offsets, total = [], 0
            for p in params:
                offsets.append(total)
                total += int(math.ceil(_numel(p) / align) * align)
            dev = params[0].device
            pbuf = torch.zeros(total, dtype=dtype, device=dev)
            gbuf = torch.zeros(total, dtype=torch.float32, device=dev)
            for p, off in zip(params, offsets):
                n = _numel(p)
                pbuf[off:off + n].copy_(p.data.reshape(-1))
                p.data = pbuf[off:off + n].view(p.shape)                # parameter storage now lives in the buffer
                p.main_grad = as_tensor(gbuf[off:off + n].view(p.shape))  # backward accumulates straight into it
                p._main_grad_persistent = True
                if not hasattr(p, "_main_grad_hook_handle"):
                    from ...utils.mix_precision_utils import _fold_grad_hook
                    p._main_grad_hook_handle = p.register_post_accumulate_grad_hook(_fold_grad_hook)
            shard = total // self._n
            lo = self._rank * shard
            b = {"dtype": dtype, "params": params, "offsets": offsets, "pbuf": pbuf, "gbuf": gbuf, "shard": shard,
                 "lo": lo, "gslice": torch.zeros(shard, dtype=torch.float32, device=dev),
                 "master": pbuf[lo:lo + shard].float().clone(),
                 "m": torch.zeros(shard, dtype=torch.float32, device=dev),
                 "v": torch.zeros(shard, dtype=torch.float32, device=dev)}
            self._buffers.append(b)

    def _fused_rs_adamw(self, b):
        """One-kernel reduce-scatter + AdamW (peer memory) is used when nothing has to look at the reduced gradient
        before the update: GPU, bf16 parameters, fused kernel policy, no global-norm clipping."""
        if "fused" in b:
            return b["fused"]
        b["fused"] = None
        clip = self._inner_opt._grad_clip
        if self._n > 1 and b["gbuf"].is_cuda and b["dtype"] == torch.bfloat16 and clip is None:
            from .....ops import functional as K
            from .....parallel import symm
            if K.get_kernel_policy() == "fused" and symm.supported() and self._n <= 8:
                from .....parallel.rs_adamw import FusedRSAdamW
                b["fused"] = FusedRSAdamW(self._group, b["shard"])
                b["inv_n"] = torch.tensor([1.0 / self._n], dtype=torch.float32, device=b["gbuf"].device)
        return b["fused"]

    def reduce_gradients(self, parameter_list, hcg):
        for b in self._buffers:
            if self._fused_rs_adamw(b) is not None:
                continue                       # the reduction happens inside the update kernel
            C.reduce_scatter(b["gslice"], b["gbuf"], op=C.ReduceOp.AVG, group=self._group)

    def _global_norm_sq(self):
        tot = None
        for b in self._buffers:
            s = b["gslice"].pow(2).sum().reshape(1)
            tot = s if tot is None else tot + s
        C.all_reduce(tot, group=self._group)
        mp = self._hcg.get_model_parallel_group()
        # tensor-parallel shards hold different parameters; replicated ones were counted once per mp rank
        return tot

    @torch.no_grad()
    def step(self):
        opt = self._inner_opt
        self._step_count += 1
        t = self._step_count
        lr = opt.get_lr()
        b1, b2, eps = opt._beta1, opt._beta2, opt._epsilon
        coeff = getattr(opt, "_coeff", 0.0)
        scale = None
        clip = opt._grad_clip
        if clip is not None and hasattr(clip, "clip_coef"):
            scale = clip.clip_coef(self._global_norm_sq())
        for b in self._buffers:
            lo, shard = b["lo"], b["shard"]
            pslice = b["pbuf"][lo:lo + shard]
            if b.get("fused") is not None:
                b["fused"].step(b["gbuf"], b["master"], b["m"], b["v"], pslice, lr, b1, b2, eps, coeff, b1 ** t, b2 ** t,
                                grad_scale=b["inv_n"], skip=opt._skip_flag)
            elif b["gslice"].is_cuda:
                from .....ops import native
                native.adamw_flat(pslice if b["dtype"] == torch.bfloat16 else None, b["master"], b["gslice"], b["m"],
                                  b["v"], lr, b1, b2, eps, coeff, b1 ** t, b2 ** t, scale, opt._skip_flag)
                if b["dtype"] != torch.bfloat16:
                    pslice.copy_(b["master"])
            else:
                g = b["gslice"] * (scale if scale is not None else 1.0)
                b["master"].mul_(1 - lr * coeff)
                b["m"].mul_(b1).add_(g, alpha=1 - b1)
                b["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
                denom = b["v"].sqrt() / math.sqrt(1 - b2 ** t) + eps
                b["master"].addcdiv_(b["m"], denom, value=-(lr / (1 - b1 ** t)))
                pslice.copy_(b["master"])
            C.all_gather(b["pbuf"], pslice.clone(), self._group)

    def clear_grad(self, set_to_zero=True):
        for b in self._buffers:
            b["gbuf"].zero_()
        for p in self._parameter_list:
            p.grad = None

    def state_dict(self):
        sd = {}
        for i, b in enumerate(self._buffers):
            sd[f"sharding_v2_buffer_{i}_moment1_0"] = as_tensor(b["m"])
            sd[f"sharding_v2_buffer_{i}_moment2_0"] = as_tensor(b["v"])
            sd[f"sharding_v2_buffer_{i}_fp32_master_0"] = as_tensor(b["master"])
        sd["sharding_v2_step"] = self._step_count
        return sd

    def set_state_dict(self, sd):
        for i, b in enumerate(self._buffers):
            for key, name in (("m", "moment1_0"), ("v", "moment2_0"), ("master", "fp32_master_0")):
                k = f"sharding_v2_buffer_{i}_{name}"
                if k in sd:
                    b[key].copy_(torch.as_tensor(sd[k]).to(b[key].device))
        self._step_count = int(sd.get("sharding_v2_step", self._step_count))

    def __getattr__(self, item):
        return getattr(self._inner_opt, item)
