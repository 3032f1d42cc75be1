"""Pipeline-parallel schedules (python/paddle/distributed/fleet/meta_parallel/pipeline_parallel.py:
``PipelineParallel`` :242 with 1F1B ``forward_backward_pipeline`` :684 and ``train_batch`` :940,
``PipelineParallelWithInterleave`` :1308, ``...FthenB`` :2396) and the point-to-point helper
(pp_utils/p2p_communication.py: shape/dtype meta handshake ``SendRecvMeta`` :52, batched isend/irecv :327).

Activations travel over NCCL point-to-point (batched, on their own communication calls) exactly as in the
reference; everything inside a stage uses this framework's kernels.
"""
from __future__ import annotations

import torch

from ...._core.tensor import as_tensor
from ....nn.layer.layers import Layer
from ... import collective as C
from ..utils.hybrid_parallel_util import broadcast_dp_parameters, broadcast_mp_parameters, broadcast_sharding_parameters
from . import MetaParallelBase
from .parallel_layers.pp_layers import PipelineLayer

_DT = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32, torch.int64, torch.bool, torch.uint8,
       torch.int8, torch.int16]


class SendRecvMeta:
    """First exchange between two stages: number of tensors, ranks, shapes, dtypes, requires_grad."""

    def __init__(self):
        self.recv_meta = None
        self.sent = False

    def send(self, tensors, dst, group):
        ts = tensors if isinstance(tensors, (tuple, list)) else [tensors]
        dev = ts[0].device
        head = torch.tensor([len(ts)], dtype=torch.int64, device=dev)
        C.send(head, dst, group)
        for t in ts:
            meta = torch.tensor([t.dim(), _DT.index(t.dtype), int(t.requires_grad), *t.shape], dtype=torch.int64, device=dev)
            C.send(torch.tensor([meta.numel()], dtype=torch.int64, device=dev), dst, group)
            C.send(meta, dst, group)
        self.sent = True

    def recv(self, src, group, device):
        head = torch.zeros(1, dtype=torch.int64, device=device)
        C.recv(head, src, group)
        metas = []
        for _ in range(int(head.item())):
            n = torch.zeros(1, dtype=torch.int64, device=device)
            C.recv(n, src, group)
            meta = torch.zeros(int(n.item()), dtype=torch.int64, device=device)
            C.recv(meta, src, group)
            m = meta.tolist()
            metas.append({"shape": m[3:3 + m[0]], "dtype": _DT[m[1]], "requires_grad": bool(m[2])})
        self.recv_meta = metas


class P2pHelper:
    def __init__(self, hcg, use_cache=True):
        self._hcg = hcg
        self._group = hcg.get_pipe_parallel_group()
        self._fwd_meta, self._bwd_shapes = SendRecvMeta(), None
        self._dev = None
        self._use_cache = use_cache

    def _device(self):
        if self._dev is None:
            from ...._core.dtype import default_device
            self._dev = default_device()
        return self._dev

    def recv_forward(self, first_stage):
        if first_stage:
            return None
        if self._fwd_meta.recv_meta is None:
            self._fwd_meta.recv(self._hcg.prev_rank, self._group, self._device())
        outs = []
        for m in self._fwd_meta.recv_meta:
            t = torch.empty(m["shape"], dtype=m["dtype"], device=self._device())
            C.recv(t, self._hcg.prev_rank, self._group)
            t = as_tensor(t)
            t.requires_grad_(m["requires_grad"] and t.is_floating_point())
            outs.append(t)
        return outs[0] if len(outs) == 1 else tuple(outs)

    def send_forward(self, output, last_stage):
        if last_stage:
            return
        if not self._fwd_meta.sent:
            self._fwd_meta.send(output, self._hcg.next_rank, self._group)
        for t in (output if isinstance(output, (tuple, list)) else [output]):
            C.send(t.detach().contiguous(), self._hcg.next_rank, self._group)

    def recv_backward(self, output, last_stage):
        if last_stage:
            return None
        grads = []
        for t in (output if isinstance(output, (tuple, list)) else [output]):
            if t.requires_grad:
                g = torch.empty_like(t.detach())
                C.recv(g, self._hcg.next_rank, self._group)
                grads.append(g)
            else:
                grads.append(None)
        return grads

    def send_backward(self, input, first_stage):
        if first_stage or input is None:
            return
        for t in (input if isinstance(input, (tuple, list)) else [input]):
            if t.requires_grad:
                g = t.grad if t.grad is not None else torch.zeros_like(t.detach())
                C.send(g.contiguous(), self._hcg.prev_rank, self._group)


    # combined steps of the steady 1F1B phase: one batched call, so neighbouring stages cannot block each other
    def _batched(self, sends, recvs):
        ops = [C.P2POp(C.isend, t, peer, self._group) for t, peer in sends]
        ops += [C.P2POp(C.irecv, t, peer, self._group) for t, peer in recvs]
        for task in C.batch_isend_irecv(ops):
            task.wait()

    def send_forward_recv_backward(self, output, last_stage):
        if last_stage:
            return None
        outs = output if isinstance(output, (tuple, list)) else [output]
        if not self._fwd_meta.sent:
            self._fwd_meta.send(output, self._hcg.next_rank, self._group)
        grads = [torch.empty_like(t.detach()) if t.requires_grad else None for t in outs]
        self._batched([(t.detach().contiguous(), self._hcg.next_rank) for t in outs],
                      [(g, self._hcg.next_rank) for g in grads if g is not None])
        return grads

    def send_backward_recv_forward(self, input, first_stage, need_recv=True):
        if first_stage:
            return None
        ins = input if isinstance(input, (tuple, list)) else [input]
        sends = [((t.grad if t.grad is not None else torch.zeros_like(t.detach())).contiguous(), self._hcg.prev_rank)
                 for t in ins if t.requires_grad]
        bufs = []
        if need_recv:
            bufs = [torch.empty(m["shape"], dtype=m["dtype"], device=self._device()) for m in self._fwd_meta.recv_meta]
        self._batched(sends, [(b, self._hcg.prev_rank) for b in bufs])
        if not need_recv:
            return None
        outs = []
        for b, m in zip(bufs, self._fwd_meta.recv_meta):
            t = as_tensor(b)
            t.requires_grad_(m["requires_grad"] and t.is_floating_point())
            outs.append(t)
        return outs[0] if len(outs) == 1 else tuple(outs)


class PipelineParallel(MetaParallelBase):
    def __init__(self, layers, hcg, strategy):
        if not isinstance(layers, PipelineLayer):
            raise TypeError("The Layer should be a derived class of PipelineLayer.")
        self._strategy_ref = strategy
        super().__init__(layers, hcg, strategy)
        pp = strategy.pipeline_configs
        hpp = strategy.hybrid_configs["pp_configs"]
        self.micro_batch_size = pp["micro_batch_size"]
        self.accumulate_steps = pp["accumulate_steps"]
        self.num_stages = hcg.get_pipe_parallel_world_size()
        self.stage_id = hcg.get_stage_id()
        self.is_first_stage = self.stage_id == 0
        self.is_last_stage = self.stage_id == self.num_stages - 1
        self._delay_scale_loss = hpp["delay_scale_loss"]
        self._p2p = P2pHelper(hcg)
        self.total_loss = None

    def _prepare_for_model(self):
        hcg = self._hcg
        if hcg.get_model_parallel_world_size() > 1:
            broadcast_mp_parameters(self._layers, hcg)
        if hcg.get_sharding_parallel_world_size() > 1:
            broadcast_sharding_parameters(self._layers, hcg)
        if hcg.get_data_parallel_world_size() > 1:
            broadcast_dp_parameters(self._layers, hcg)

    # ------------------------------------------------------------------ micro-batches
    def _load_micro_batch(self, data, idx):
        if data is None:
            return None
        lo, hi = idx * self.micro_batch_size, (idx + 1) * self.micro_batch_size

        def cut(x):
            if isinstance(x, torch.Tensor):
                return x[lo:hi]
            if isinstance(x, (tuple, list)):
                return type(x)(cut(v) for v in x)
            return x
        return cut(data)

    def _forward_step(self, input_tensor, inputs, labels, mb):
        if self.is_first_stage:
            input_tensor = self._load_micro_batch(inputs, mb)
        out = self._layers.forward(input_tensor)
        if self.is_last_stage:
            assert self._layers._loss_fn is not None, "loss function should exist to compute loss"
            lab = self._load_micro_batch(labels, mb)
            loss = self._layers._loss_fn(out, lab) if not isinstance(lab, (tuple, list)) else self._layers._loss_fn(out, *lab)
            if self.accumulate_steps > 1 and not self._delay_scale_loss:
                loss = loss / self.accumulate_steps
            self.total_loss = loss.detach() if self.total_loss is None else self.total_loss + loss.detach()
            return loss
        return out

    def _backward_step(self, input_tensor, output_tensor, output_grads, scaler=None):
        if self.is_last_stage:
            (scaler.scale(output_tensor) if scaler else output_tensor).backward()
        else:
            outs = output_tensor if isinstance(output_tensor, (tuple, list)) else [output_tensor]
            pairs = [(o, g) for o, g in zip(outs, output_grads) if g is not None]
            torch.autograd.backward([C._plain(o) for o, _ in pairs], [C._plain(g) for _, g in pairs])

    def forward_backward_pipeline(self, data, scaler=None, forward_only=False):
        """1F1B: warm-up forwards, steady one-forward-one-backward, cool-down backwards (:684-884)."""
        inputs, labels = data if isinstance(data, (tuple, list)) and len(data) == 2 else (data, None)
        self.total_loss = None
        startup = min(self.num_stages - self.stage_id - 1, self.accumulate_steps)
        steady = self.accumulate_steps - startup
        in_buf, out_buf = [], []
        mb_f = 0
        for _ in range(startup):
            x = self._p2p.recv_forward(self.is_first_stage)
            y = self._forward_step(x, inputs, labels, mb_f)
            mb_f += 1
            self._p2p.send_forward(y, self.is_last_stage)
            in_buf.append(x)
            out_buf.append(y)
        x = self._p2p.recv_forward(self.is_first_stage) if steady > 0 else None
        for i in range(steady):
            y = self._forward_step(x, inputs, labels, mb_f)
            mb_f += 1
            in_buf.append(x)
            out_buf.append(y)
            more = i + 1 < steady
            if forward_only:
                self._p2p.send_forward(y, self.is_last_stage)
                x = self._p2p.recv_forward(self.is_first_stage) if more else None
                in_buf.clear(), out_buf.clear()
                continue
            grads = self._p2p.send_forward_recv_backward(y, self.is_last_stage)
            xi, yi = in_buf.pop(0), out_buf.pop(0)
            self._backward_step(xi, yi, grads, scaler)
            x = self._p2p.send_backward_recv_forward(xi, self.is_first_stage, need_recv=more)
        if not forward_only:
            for _ in range(startup):
                yi = out_buf[0]
                grads = self._p2p.recv_backward(yi, self.is_last_stage)
                xi, yi = in_buf.pop(0), out_buf.pop(0)
                self._backward_step(xi, yi, grads, scaler)
                self._p2p.send_backward(xi, self.is_first_stage)
            self._layers.allreduce_shared_weight_gradients()
        return self._broadcast_final_loss()

    def _loss_stage(self):
        """Pipeline stage that holds the last virtual stage (and so the loss): the last one, except under a zigzag
        placement with an even number of chunks, where the model ends on the first stage."""
        ex = getattr(self, "_executor", None)
        if ex is not None:
            return ex.place.owner(ex.P * ex.V - 1)[0]
        return self.num_stages - 1

    def _broadcast_final_loss(self):
        g = self._hcg.get_pipe_parallel_group()
        from ...._core.dtype import default_device
        holder = self._loss_stage()
        if self.stage_id == holder:
            loss = self.total_loss.float().reshape(1).clone()
            if self._delay_scale_loss:
                loss = loss / self.accumulate_steps
        else:
            loss = torch.zeros(1, dtype=torch.float32, device=default_device())
        last = self._hcg.get_rank_from_stage(holder)
        C.broadcast(loss, last, g)
        return as_tensor(loss.reshape([]))

    def train_batch(self, data, optimizer, lr_scheduler=None, scaler=None):
        self._layers.train()
        loss = self.forward_backward_pipeline(data, scaler)
        if scaler is not None:
            scaler.step(optimizer)
            scaler.update()
        else:
            optimizer.step()
        optimizer.clear_grad()
        if lr_scheduler is not None:
            lr_scheduler.step()
        return loss

    def eval_batch(self, data, compute_loss=False):
        self._layers.eval()
        with torch.no_grad():
            return self.forward_backward_pipeline(data, forward_only=True)

    def forward(self, *a, **k):
        return self._layers(*a, **k)


class PipelineParallelWithInterleaveFthenB(PipelineParallel):
    """Virtual pipeline stages, all forwards then all backwards (reference :2396).

    Each rank holds ``V`` model chunks; a micro-batch visits chunk 0 of every stage, returns over the ring
    from the last stage to the first, visits chunk 1 of every stage, and so on.  The schedule is systolic:
    work item ``k = (group, chunk, mb_in_group)`` runs on stage ``s`` at tick ``k + s`` and its output is
    consumed exactly one tick later (also across the ring hop, because a group holds ``P`` micro-batches), so
    every tick ends with ONE batched send/receive in which all ranks take part - no ordering deadlock is
    possible.  The backward pass runs the same items in reverse."""

    _META = 16

    def __init__(self, layers, hcg, strategy):
        super().__init__(layers, hcg, strategy)
        self._V = layers.get_num_virtual_stages() if hasattr(layers, "get_num_virtual_stages") else 1
        if self._V > 1:
            assert self.accumulate_steps % self.num_stages == 0, \
                "accumulate_steps must be a multiple of the pipeline degree for interleaved scheduling"
        self._act_meta = None
        self._meta_sent = False
        self._group = hcg.get_pipe_parallel_group()
        self._next = hcg.get_rank_from_stage((self.stage_id + 1) % self.num_stages)
        self._prev = hcg.get_rank_from_stage((self.stage_id - 1) % self.num_stages)

    def _item(self, k):
        P, V = self.num_stages, self._V
        if V == 1:
            return 0, k
        g, r = divmod(k, V * P)
        c, j = divmod(r, P)
        return c, g * P + j

    def _exchange(self, send_t, peer_s, want_recv, peer_r, meta_known_shape=None):
        from ...._core.dtype import default_device
        dev = default_device()
        if meta_known_shape is None and ((want_recv and self._act_meta is None) or
                                         (send_t is not None and not self._meta_sent)):
            ops = []
            if send_t is not None and not self._meta_sent:
                m = [send_t.dim(), _DT.index(send_t.dtype), int(send_t.requires_grad), *send_t.shape]
                m += [0] * (self._META - len(m))
                ops.append(C.P2POp(C.isend, torch.tensor(m, dtype=torch.int64, device=dev), peer_s, self._group))
                self._meta_sent = True
            meta_in = None
            if want_recv and self._act_meta is None:
                meta_in = torch.zeros(self._META, dtype=torch.int64, device=dev)
                ops.append(C.P2POp(C.irecv, meta_in, peer_r, self._group))
            for t in C.batch_isend_irecv(ops):
                t.wait()
            if meta_in is not None:
                m = meta_in.tolist()
                self._act_meta = {"shape": m[3:3 + m[0]], "dtype": _DT[m[1]], "requires_grad": bool(m[2])}
        ops, buf = [], None
        if send_t is not None:
            ops.append(C.P2POp(C.isend, send_t.detach().contiguous(), peer_s, self._group))
        if want_recv:
            shape = meta_known_shape if meta_known_shape is not None else self._act_meta
            buf = torch.empty(shape["shape"], dtype=shape["dtype"], device=dev)
            ops.append(C.P2POp(C.irecv, buf, peer_r, self._group))
        for t in C.batch_isend_irecv(ops):
            t.wait()
        return buf

    def forward_backward_pipeline(self, data, scaler=None, forward_only=False):
        inputs, labels = data if isinstance(data, (tuple, list)) and len(data) == 2 else (data, None)
        P, V, s = self.num_stages, self._V, self.stage_id
        K = self.accumulate_steps * V
        self.total_loss = None
        ins, outs = {}, {}
        recv_buf = None
        final = lambda c: self.is_last_stage and c == V - 1       # noqa: E731
        source = lambda c: self.is_first_stage and c == 0         # noqa: E731
        for t in range(K + P - 1):
            k = t - s
            y = None
            if 0 <= k < K:
                c, mb = self._item(k)
                if source(c):
                    x = self._load_micro_batch(inputs, mb)
                else:
                    x = as_tensor(recv_buf)
                    x.requires_grad_(self._act_meta["requires_grad"] and x.is_floating_point() and not forward_only)
                out = self._layers.forward(x, chunk_id=c) if V > 1 else self._layers.forward(x)
                if final(c):
                    lab = self._load_micro_batch(labels, mb)
                    loss = self._layers._loss_fn(out, lab)
                    if self.accumulate_steps > 1 and not self._delay_scale_loss:
                        loss = loss / self.accumulate_steps
                    self.total_loss = loss.detach() if self.total_loss is None else self.total_loss + loss.detach()
                    out = loss
                else:
                    y = out
                if not forward_only:
                    ins[k], outs[k] = x, out
            k2 = t + 1 - s
            want = 0 <= k2 < K and not source(self._item(k2)[0])
            recv_buf = self._exchange(y, self._next, want, self._prev)
        if not forward_only:
            act = self._act_meta
            gbuf = None
            for t in range(K + P - 1):
                k = K - 1 - (t - (P - 1 - s))
                gsend = None
                if 0 <= k < K:
                    c, _ = self._item(k)
                    x, y = ins.pop(k), outs.pop(k)
                    if final(c):
                        (scaler.scale(y) if scaler else y).backward()
                    else:
                        torch.autograd.backward([C._plain(y)], [C._plain(gbuf)])
                    if not source(c) and isinstance(x, torch.Tensor) and x.requires_grad:
                        gsend = x.grad
                k2 = K - 1 - (t + 1 - (P - 1 - s))
                want = 0 <= k2 < K and not final(self._item(k2)[0])
                shape = None
                if want:
                    yy = outs[k2]
                    shape = {"shape": list(yy.shape), "dtype": yy.dtype}
                gbuf = self._exchange(gsend, self._prev, want, self._next, meta_known_shape=shape or {"shape": [0], "dtype": torch.float32})
            self._layers.allreduce_shared_weight_gradients()
        return self._broadcast_final_loss()


class PipelineParallelWithInterleaveWindowed(PipelineParallelWithInterleaveFthenB):
    """Same systolic item order as the F-then-B class, run window by window: a window of ``P`` micro-batches (one
    group) goes forward through all chunks and then backward, so live activations are bounded by one group instead
    of the whole batch."""

    def forward_backward_pipeline(self, data, scaler=None, forward_only=False):
        P = self.num_stages
        window = getattr(self, "_window_groups", None)
        if forward_only or self._V == 1 or window is None:
            return super().forward_backward_pipeline(data, scaler, forward_only)
        inputs, labels = data
        acc, total = self.accumulate_steps, None
        per = window * P
        try:
            for lo in range(0, acc, per):
                n = min(per, acc - lo)
                sl = slice(lo * self.micro_batch_size, (lo + n) * self.micro_batch_size)
                self.accumulate_steps = n
                part = super().forward_backward_pipeline((inputs[sl] if inputs is not None else None,
                                                          labels[sl] if labels is not None else None), scaler, False)
                total = part * n if total is None else total + part * n
        finally:
            self.accumulate_steps = acc
        return total / acc


class PipelineParallelWithInterleave(PipelineParallel):
    """Interleaved 1F1B over virtual stages (reference :1308): each rank holds ``V`` chunks, warm-up is
    ``(P - rank - 1) * 2 + (V - 1) * P`` forwards, then forwards and backwards alternate, so the bubble shrinks by
    ``V`` compared with plain 1F1B.  The order is generated as data and run by the schedule executor
    (``pipeline_schedules.py``); ``schedule_mode`` in ``pipeline_configs`` selects another generator."""

    def __init__(self, layers, hcg, strategy):
        super().__init__(layers, hcg, strategy)
        from . import pipeline_schedules as S
        self._V = layers.get_num_virtual_stages()
        mode = strategy.pipeline_configs.get("schedule_mode", "VPP") if hasattr(strategy.pipeline_configs, "get") else "VPP"
        if self._V > 1 and mode in ("1F1B", "ZBH1"):
            mode = "VPP"
        elif self._V == 1 and mode in ("VPP", "interleaved_1f1b"):
            mode = "1F1B"
        self._executor = S.ScheduleExecutor(self, S.SCHEDULES.get(mode, S.interleaved_1f1b))
        S.validate(self._executor.fn, self.num_stages, self._V, self.accumulate_steps)

    def forward_backward_pipeline(self, data, scaler=None, forward_only=False):
        return self._executor.run(data, scaler, forward_only)
