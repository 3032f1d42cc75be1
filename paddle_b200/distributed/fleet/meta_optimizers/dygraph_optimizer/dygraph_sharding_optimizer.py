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
DEFAULT_COMM_BUFFER_MB = 256


class _Bucket:
    """One flat communication buffer: parameters of one dtype laid out class by class (see ``_class_key``) in
    256-byte x nranks aligned slots, fp32 gradients of the same layout, and this rank's slice of the optimizer state."""

    __slots__ = ("dtype", "params", "offsets", "total", "shard", "lo", "pbuf", "gbuf", "gslice", "master", "m", "v",
                 "segments", "hits", "need", "launched", "task", "fused", "inv_n", "event", "index")


class DygraphShardingOptimizerV2:
    """Sharding stage 1 with split parameters (``split_param=True``): reduce-scatter of flat gradient buckets, update of
    the owned slice, all-gather of the parameter buckets
    (python/paddle/distributed/fleet/meta_optimizers/dygraph_optimizer/dygraph_sharding_optimizer.py:592 and
    python/paddle/distributed/fleet/utils/tensor_fusion_helper.py:408 ``FusedCommBuffer``).

    * Buckets are filled in reverse parameter order (the order in which backward finishes gradients) up to
      ``comm_buffer_size_MB``; a gradient hook counts arrivals per bucket the way ``FusedCommBuffer.add_grad``
      does (:623-646: every parameter must have been accumulated ``accumulate_steps`` times) and starts the bucket's
      reduction as soon as it is complete, on a side stream, so it runs under the rest of backward.
    * The reduction is two-phase so that global-norm clipping works with the fused kernel: phase A reduces the owned
      slice (one kernel over peer memory, ``parallel/rs_adamw.py::FusedRSAdamW.reduce``, or NCCL reduce-scatter),
      then the squared norm of the reduced slices is summed - tensor-parallel (``is_distributed``) and replicated
      parameters separately, as ``HybridParallelClipGrad`` does (hybrid_parallel_optimizer.py:112-266) - and phase B
      applies AdamW with the clip coefficient folded in.
    * Inside a bucket parameters are ordered by (is_distributed, need_clip, learning-rate multiplier, decay
      coefficient), so each class is one contiguous range and the per-class learning rate / weight decay of the wrapped
      optimizer (``apply_decay_param_fun``, ``lr_ratio``, per-group ``learning_rate`` / ``weight_decay``,
      ``optimize_attr``) costs one update launch per class and bucket.
    * ``state_dict()`` emits the reference's per-parameter keys (``{param.name}_moment1_0`` ..., ``master_weights``,
      python/paddle/optimizer/optimizer.py:376,1030) with FULL tensors gathered over the sharding group, so a ``.pdopt``
      written under one sharding degree loads under another (or under none).
    """

    def __init__(self, optimizer, hcg, sharding_configs=None):
        from .....optimizer.adamw import AdamW
        if not isinstance(optimizer, AdamW) or not getattr(optimizer, "_decoupled", True):
            raise TypeError("DygraphShardingOptimizerV2 (split_param=True) updates flat slices with the AdamW rule; "
                            f"got {type(optimizer).__name__}.  Use split_param=False for other optimizers.")
        self._inner_opt = optimizer
        self._hcg = hcg
        self._group = hcg.get_sharding_parallel_group()
        self._n = hcg.get_sharding_parallel_world_size()
        self._rank = hcg.get_sharding_parallel_rank()
        self._parameter_list = [p for p in optimizer._parameter_list if p.requires_grad]
        self._step_count = 0
        cfg = sharding_configs if sharding_configs is not None else {}
        self._comm_buffer_bytes = int(float(_cfg_get(cfg, "comm_buffer_size_MB", DEFAULT_COMM_BUFFER_MB)) * (1 << 20))
        self._acc_steps = max(int(_cfg_get(cfg, "accumulate_steps", 1)), 1)
        self._overlap = bool(_cfg_get(cfg, "comm_overlap", False))
        self._comm_stream = None
        self._build_buffers()

    # ------------------------------------------------------------------ layout
    def _class_key(self, p, group):
        opt = self._inner_opt
        lr_mult = float(group.get("learning_rate", 1.0)) * float(getattr(p, "optimize_attr", {}).get("learning_rate", 1.0))
        if getattr(opt, "_lr_ratio", None) is not None:
            lr_mult *= float(opt._lr_ratio(p))
        return (bool(getattr(p, "is_distributed", False)), bool(getattr(p, "need_clip", True)), lr_mult,
                float(opt._decay_for(p, group)))

    def _build_buffers(self):
        group_of = {}
        for g in self._inner_opt._param_groups:
            for p in g["params"]:
                group_of[id(p)] = g
        buckets_params = []            # [(dtype, [params])]
        cur = {}
        for p in reversed(self._parameter_list):
            lst = cur.setdefault(p.dtype, [])
            lst.append(p)
            if sum(_numel(q) for q in lst) * p.element_size() >= self._comm_buffer_bytes:
                buckets_params.append((p.dtype, lst))
                cur[p.dtype] = []
        for dtype, lst in cur.items():
            if lst:
                buckets_params.append((dtype, lst))
        self._buffers = []
        self._bucket_of = {}
        for bi, (dtype, params) in enumerate(buckets_params):
            keys = {id(p): self._class_key(p, group_of.get(id(p), {})) for p in params}
            order = sorted(range(len(params)), key=lambda i: (tuple(-float(x) if isinstance(x, bool) else x
                                                                    for x in keys[id(params[i])][:2]),
                                                              keys[id(params[i])][2:], i))
            params = [params[i] for i in order]
            es = torch.empty(0, dtype=dtype).element_size()
            align = max(ALIGN_BYTES // es, 1) * self._n     # every slot is a multiple of 256 B x nranks
            offsets, total = [], 0
            for p in params:
                offsets.append(total)
                total += int(math.ceil(_numel(p) / align) * align)
            dev = params[0].device
            b = _Bucket()
            b.index, b.dtype, b.params, b.offsets, b.total = bi, dtype, params, offsets, total
            b.pbuf = torch.zeros(total, dtype=dtype, device=dev)
            b.gbuf = torch.zeros(total, dtype=torch.float32, device=dev)
            for p, off in zip(params, offsets):
                n = _numel(p)
                b.pbuf[off:off + n].copy_(p.data.reshape(-1))
                p.data = b.pbuf[off:off + n].view(p.shape)                # parameter storage now lives in the buffer
                p.main_grad = as_tensor(b.gbuf[off:off + n].view(p.shape))  # backward accumulates straight into it
                p._main_grad_persistent = True
                if not hasattr(p, "_main_grad_hook_handle"):
                    from ...utils.mix_precision_utils import _fold_grad_hook
                    p._main_grad_hook_handle = p.register_post_accumulate_grad_hook(_fold_grad_hook)
                self._bucket_of[id(p)] = b
                p.register_post_accumulate_grad_hook(self._make_ready_hook(b))
            b.shard = total // self._n
            b.lo = self._rank * b.shard
            b.gslice = torch.zeros(b.shard, dtype=torch.float32, device=dev)
            b.master = b.pbuf[b.lo:b.lo + b.shard].float().clone()
            b.m = torch.zeros(b.shard, dtype=torch.float32, device=dev)
            b.v = torch.zeros(b.shard, dtype=torch.float32, device=dev)
            # contiguous class ranges of the bucket, cut to the owned slice: (start, end, key) in slice coordinates
            b.segments = []
            for p, off, nxt in zip(params, offsets, offsets[1:] + [total]):
                a, e = max(off, b.lo) - b.lo, min(nxt, b.lo + b.shard) - b.lo
                if e <= a:
                    continue
                k = keys[id(p)]
                if b.segments and b.segments[-1][2] == k and b.segments[-1][1] == a:
                    b.segments[-1] = (b.segments[-1][0], e, k)
                else:
                    b.segments.append((a, e, k))
            b.hits, b.need = {}, len(params) * self._acc_steps
            b.launched, b.task, b.fused, b.inv_n, b.event = False, None, False, None, None
            self._buffers.append(b)

    # ------------------------------------------------------------------ gradient accounting and reduction
    def _make_ready_hook(self, b):
        def hook(param):
            # mirrors FusedCommBuffer.add_grad: count one arrival per parameter and accumulation step; the bucket is
            # complete when every parameter has been seen accumulate_steps times
            b.hits[id(param)] = b.hits.get(id(param), 0) + 1
            if b.hits[id(param)] > self._acc_steps:
                raise RuntimeError(f"gradient of {param.name} arrived {b.hits[id(param)]} times for "
                                   f"accumulate_steps={self._acc_steps}")
            if sum(b.hits.values()) == b.need and self._overlap and not b.launched:
                self._launch_reduce(b, overlap=True)
        return hook

    def _fused(self, b):
        """The one-kernel reduce over peer memory is used on GPUs with symmetric memory, up to 8 ranks."""
        if b.fused is False:
            b.fused = None
            if self._n > 1 and b.gbuf.is_cuda and self._n <= 8:
                from .....ops import functional as K
                from .....parallel import symm
                if K.get_kernel_policy() == "fused" and symm.supported():
                    from .....parallel.rs_adamw import FusedRSAdamW
                    b.fused = FusedRSAdamW(self._group, b.shard)
                    b.inv_n = torch.tensor([1.0 / self._n], dtype=torch.float32, device=b.gbuf.device)
        return b.fused

    def _launch_reduce(self, b, overlap=False):
        """Phase A for one bucket: the owned slice of the averaged gradient lands in ``b.gslice``."""
        b.launched = True
        if self._n == 1:
            b.gslice.copy_(b.gbuf)
            return
        side = None
        if overlap and b.gbuf.is_cuda:
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=b.gbuf.device)
            side = self._comm_stream
            side.wait_stream(torch.cuda.current_stream(b.gbuf.device))
        fused = self._fused(b)
        if side is not None:
            with torch.cuda.stream(side):
                if fused is not None:
                    fused.reduce(b.gbuf, b.gslice, grad_scale=b.inv_n)
                else:
                    C.reduce_scatter(b.gslice, b.gbuf, op=C.ReduceOp.AVG, group=self._group)
                b.event = torch.cuda.Event()
                b.event.record(side)
        elif fused is not None:
            fused.reduce(b.gbuf, b.gslice, grad_scale=b.inv_n)
        else:
            C.reduce_scatter(b.gslice, b.gbuf, op=C.ReduceOp.AVG, group=self._group)

    def reduce_gradients(self, parameter_list, hcg):
        """Start the reduction of every bucket that the hooks have not started (no overlap configured, a parameter
        without gradient this step) and make the current stream wait for all of them."""
        for b in self._buffers:
            if not b.launched:
                self._launch_reduce(b)
        for b in self._buffers:
            if b.event is not None:
                torch.cuda.current_stream(b.gbuf.device).wait_event(b.event)
                b.event = None

    # ------------------------------------------------------------------ clipping
    def _global_norm_sq(self):
        """Squared global gradient norm from the reduced slices.  A tensor-parallel parameter exists once per mp rank
        with different content: its part is summed over the mp group.  A replicated parameter is identical on all mp
        ranks and counted once.  Every rank holds a different slice: both parts are summed over the sharding group,
        and over pipeline stages."""
        dev = self._buffers[0].gslice.device
        dist = torch.zeros(1, dtype=torch.float32, device=dev)
        rep = torch.zeros(1, dtype=torch.float32, device=dev)
        for b in self._buffers:
            for a, e, key in b.segments:
                if not key[1]:                      # need_clip False: not part of the norm
                    continue
                sq = b.gslice[a:e].pow(2).sum().reshape(1)
                if key[0]:
                    dist += sq
                else:
                    rep += sq
        hcg = self._hcg
        mp = hcg.get_model_parallel_group()
        if mp is not None and mp.nranks > 1:
            C.all_reduce(dist, group=mp)
        total = dist + rep
        if self._n > 1:
            C.all_reduce(total, group=self._group)
        pp = hcg.get_pipe_parallel_group()
        if pp is not None and pp.nranks > 1:
            C.all_reduce(total, group=pp)
        return total

    # ------------------------------------------------------------------ update
    @torch.no_grad()
    def step(self):
        opt = self._inner_opt
        self.reduce_gradients(None, self._hcg)
        self._step_count += 1
        t = self._step_count
        base_lr = opt.get_lr()
        b1, b2, eps = opt._beta1, opt._beta2, opt._epsilon
        clip = opt._grad_clip
        scale = None
        if clip is not None:
            if not hasattr(clip, "clip_coef"):
                raise TypeError("split_param sharding supports ClipGradByGlobalNorm only")
            scale = clip.clip_coef(self._global_norm_sq())
        for b in self._buffers:
            pslice = b.pbuf[b.lo:b.lo + b.shard]
            for a, e, key in b.segments:
                lr, coeff = base_lr * key[2], key[3]
                seg_scale = scale if key[1] else None
                g, master, m, v = b.gslice[a:e], b.master[a:e], b.m[a:e], b.v[a:e]
                if g.is_cuda:
                    from .....ops import native
                    native.adamw_flat(pslice[a:e] if b.dtype == torch.bfloat16 else None, master, g, m, v, lr, b1, b2,
                                      eps, coeff, b1 ** t, b2 ** t, seg_scale, opt._skip_flag)
                    if b.dtype != torch.bfloat16:
                        pslice[a:e].copy_(master)
                else:
                    if opt._skip_flag is not None and int(opt._skip_flag.item()) != 0:
                        continue
                    gg = g * (seg_scale if seg_scale is not None else 1.0)
                    master.mul_(1 - lr * coeff)
                    m.mul_(b1).add_(gg, alpha=1 - b1)
                    v.mul_(b2).addcmul_(gg, gg, value=1 - b2)
                    denom = v.sqrt() / math.sqrt(1 - b2 ** t) + eps
                    master.addcdiv_(m, denom, value=-(lr / (1 - b1 ** t)))
                    pslice[a:e].copy_(master)
            if self._n > 1:
                if b.pbuf.is_cuda:
                    # in place: every rank's slice already sits at its offset of the output buffer
                    C.all_gather_into_tensor(b.pbuf, pslice, group=self._group)
                else:
                    C.all_gather_into_tensor(b.pbuf, pslice.clone(), group=self._group)

    def clear_grad(self, set_to_zero=True):
        for b in self._buffers:
            b.gbuf.zero_()
            b.hits.clear()
            b.launched = False
        for p in self._parameter_list:
            p.grad = None

    clear_gradients = clear_grad

    # ------------------------------------------------------------------ checkpoint
    def _gather_full(self, t):
        if self._n == 1:
            return t
        full = torch.empty(t.numel() * self._n, dtype=t.dtype, device=t.device)
        C.all_gather_into_tensor(full, t.contiguous(), group=self._group)
        return full

    def state_dict(self, gather=False):
        """Reference key layout (optimizer.py:376): ``{param.name}_moment1_0`` / ``_moment2_0`` / ``_beta1_pow_acc_0`` /
        ``_beta2_pow_acc_0`` per parameter, ``master_weights`` keyed by parameter name, ``LR_Scheduler``.

        ``gather=False`` (no communication, any rank may call it alone): the tensors are this rank's 1-D slices of the
        flattened parameters it owns a part of, and ``sharding_v2_meta`` records ``{name: (start, end)}`` - the form
        every rank writes to its own file, as the reference's split-param optimizer does.
        ``gather=True`` (collective over the sharding group): full per-parameter tensors, returned on the host and
        independent of the sharding degree - the form that loads under another degree or without sharding."""
        opt = self._inner_opt
        sd, masters, slices = {}, {}, {}
        t = self._step_count
        for b in self._buffers:
            if gather:
                src = {k: self._gather_full(getattr(b, k)).cpu() for k in ("m", "v", "master")}
                base = 0
            else:
                src = {"m": b.m, "v": b.v, "master": b.master}
                base = b.lo
            for p, off in zip(b.params, b.offsets):
                n = _numel(p)
                a, e = (off, off + n) if gather else (max(off, b.lo), min(off + n, b.lo + b.shard))
                if e <= a:
                    continue

                def cut(tn):
                    x = src[tn][a - base:e - base].clone()
                    return as_tensor(x.view(p.shape) if gather else x)
                sd[f"{p.name}_moment1_0"] = cut("m")
                sd[f"{p.name}_moment2_0"] = cut("v")
                sd[f"{p.name}_beta1_pow_acc_0"] = as_tensor(torch.tensor([opt._beta1 ** (t + 1)], dtype=torch.float32))
                sd[f"{p.name}_beta2_pow_acc_0"] = as_tensor(torch.tensor([opt._beta2 ** (t + 1)], dtype=torch.float32))
                if b.dtype != torch.float32 or getattr(opt, "_multi_precision", False):
                    masters[p.name] = cut("master")
                if not gather:
                    slices[p.name] = (a - off, e - off)
        if masters:
            sd["master_weights"] = masters
        if not gather:
            sd["sharding_v2_meta"] = {"degree": self._n, "rank": self._rank, "slices": slices}
        sched = getattr(opt, "_learning_rate", None)
        if hasattr(sched, "state_dict"):
            sd["LR_Scheduler"] = sched.state_dict()
        return sd

    def set_state_dict(self, sd):
        """Accepts both forms written by :meth:`state_dict`: full per-parameter tensors (any sharding degree) or this
        rank's slices (same degree and rank, checked through ``sharding_v2_meta``)."""
        opt = self._inner_opt
        masters = sd.get("master_weights", {})
        meta = sd.get("sharding_v2_meta")
        if meta is not None and (meta["degree"] != self._n or meta["rank"] != self._rank):
            raise ValueError(f"optimizer slices of rank {meta['rank']} / degree {meta['degree']} cannot be loaded on rank "
                             f"{self._rank} / degree {self._n}; save with state_dict(gather=True) to change the degree")
        steps = []
        for b in self._buffers:
            for p, off in zip(b.params, b.offsets):
                n = _numel(p)
                a, e = max(off, b.lo), min(off + n, b.lo + b.shard)
                if e <= a:
                    continue
                if meta is not None:
                    sa, se = meta["slices"].get(p.name, (a - off, e - off))
                    if (sa, se) != (a - off, e - off):
                        raise ValueError(f"slice of {p.name} in the checkpoint {(sa, se)} differs from this layout "
                                         f"{(a - off, e - off)}")
                    lo_src = 0
                else:
                    lo_src = a - off

                def part(x):
                    x = torch.as_tensor(x).reshape(-1)
                    return x[lo_src:lo_src + (e - a)]
                for key, dst in ((f"{p.name}_moment1_0", b.m), (f"{p.name}_moment2_0", b.v)):
                    if key in sd:
                        dst[a - b.lo:e - b.lo].copy_(part(sd[key]).to(dst.device, torch.float32))
                if p.name in masters:
                    b.master[a - b.lo:e - b.lo].copy_(part(masters[p.name]).to(b.master.device, torch.float32))
                    b.pbuf[a:e].copy_(b.master[a - b.lo:e - b.lo])
                k = f"{p.name}_beta1_pow_acc_0"
                if k in sd and opt._beta1 not in (0.0, 1.0):
                    v = float(torch.as_tensor(sd[k]).reshape(-1)[0])
                    if 0 < v < 1:
                        steps.append(int(round(math.log(v) / math.log(opt._beta1))) - 1)
        if steps:
            self._step_count = max(steps)
        if "LR_Scheduler" in sd and hasattr(getattr(opt, "_learning_rate", None), "set_state_dict"):
            opt._learning_rate.set_state_dict(sd["LR_Scheduler"])
        if self._n > 1:          # parameters restored from master weights: refresh the other ranks' copies
            for b in self._buffers:
                pslice = b.pbuf[b.lo:b.lo + b.shard]
                C.all_gather_into_tensor(b.pbuf, pslice if b.pbuf.is_cuda else pslice.clone(), group=self._group)

    def __getattr__(self, item):
        return getattr(self._inner_opt, item)


def _cfg_get(cfg, key, default):
    try:
        v = cfg[key] if key in cfg else default
    except TypeError:
        v = getattr(cfg, key, default)
    return default if v is None else v
