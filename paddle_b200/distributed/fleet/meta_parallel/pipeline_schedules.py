"""Pipeline schedules as data plus one executor.

A *schedule* is, per pipeline rank, a list of steps ``(kind, chunk, micro_batch)`` with kind ``"F"`` (forward),
``"B"`` (whole backward), ``"Bx"`` (backward for the input gradient only; weight gradients are queued) or ``"W"``
(the queued weight gradients of an earlier ``"Bx"``).  ``interleaved_1f1b``
generates the virtual-pipeline order of python/paddle/distributed/fleet/meta_parallel/pipeline_parallel.py
``PipelineParallelWithInterleave`` (:1308-2390): warm-up forwards ``(P - rank - 1) * 2 + (V - 1) * P``, then one
forward / one backward, then the remaining backwards; virtual micro-batch ``k`` maps to chunk
``(k % (P * V)) // P`` (mirrored for backward) and micro-batch ``(k // (P * V)) * P + k % P``.

``ScheduleExecutor`` runs any such schedule.  A step's input (activation from virtual stage ``vs - 1`` or gradient
from ``vs + 1``) travels as one message on the channel (source rank -> this rank).  Because the schedule is static,
every rank derives the exact message order of each of its incoming channels by replaying the sender's list, and
receives strictly in that order (stashing what arrives early).  Sends are asynchronous and every ordered rank pair
has its own communicator, on which one side only sends and the other only receives, in the same order: a send can
never be stuck behind a receive, on NCCL as well as on gloo, so any dependency-respecting schedule runs without
deadlock and without the combined send/receive calls hand-written per schedule phase."""
from __future__ import annotations

import torch

from ... import collective as C
from ...._core.tensor import as_tensor


def f_then_b(P, V, M, rank):
    steps = [("F", c, m) for c, m in _virtual_order(P, V, M)]
    return steps + [("B", V - 1 - c, m) for c, m in _virtual_order(P, V, M)]


def one_f_one_b(P, V, M, rank):
    assert V == 1
    warm = min(P - rank - 1, M)
    steps = [("F", 0, m) for m in range(warm)]
    for i in range(M - warm):
        steps += [("F", 0, warm + i), ("B", 0, i)]
    return steps + [("B", 0, m) for m in range(M - warm, M)]


def _virtual_order(P, V, M):
    """(chunk, micro-batch) of virtual micro-batch k = 0 .. M * V - 1 in forward order."""
    out = []
    for k in range(M * V):
        g, r = divmod(k, P * V)
        out.append((r // P, g * P + r % P))
    return out


def interleaved_1f1b(P, V, M, rank):
    if M % P != 0:
        raise ValueError("interleaved 1F1B needs accumulate_steps to be a multiple of the pipeline degree")
    N = M * V
    fwd = _virtual_order(P, V, M)
    bwd = [(V - 1 - c, m) for c, m in fwd]
    warm = min((P - rank - 1) * 2 + (V - 1) * P, N)
    steps = [("F", *fwd[k]) for k in range(warm)]
    for i in range(N - warm):
        steps += [("F", *fwd[warm + i]), ("B", *bwd[i])]
    return steps + [("B", *bwd[k]) for k in range(N - warm, N)]


def zero_bubble_h1(P, V, M, rank):
    """ZB-H1: 1F1B with one more warm-up forward per stage, whose bubble is filled by postponing weight gradients.
    Stage ``rank`` runs its first ``rank`` backwards as ``Bx`` and pays their ``W`` steps at the very end, where
    1F1B would idle waiting for the upstream stages to drain; the memory peak stays that of 1F1B's first stage.
    Step counts follow python/paddle/distributed/passes/pipeline_scheduler_pass/pipeline_zero_bubble.py:66-140."""
    assert V == 1
    if M < P:
        raise ValueError("ZB-H1 needs at least as many micro-batches as pipeline stages")
    warm = P - rank
    steps = [("F", 0, m) for m in range(warm)]
    f, b = warm, 0
    while f < M:                                   # steady state: the first `rank` backwards leave W for later
        steps += [("Bx" if b < rank else "B", 0, b), ("F", 0, f)]
        f, b = f + 1, b + 1
    while b < M - 1:
        steps.append(("B", 0, b))
        b += 1
    steps += [("Bx", 0, b), ("W", 0, b)] if rank > 0 else [("B", 0, b)]
    return steps + [("W", 0, m) for m in range(rank)]


SCHEDULES = {"FThenB": f_then_b, "1F1B": one_f_one_b, "VPP": interleaved_1f1b, "interleaved_1f1b": interleaved_1f1b,
             "ZBH1": zero_bubble_h1}


STEP_COST = {"F": 1.0, "B": 2.0, "Bx": 1.0, "W": 1.0}


def validate(schedule_fn, P, V, M, cost=None):
    """Checks on the host that the per-rank lists form a deadlock-free global order (every step's input is produced
    by an earlier step of some rank, every ``Bx`` has exactly one later ``W``) and returns the makespan of a
    simulation in which a step starts when its rank is free and its input has been produced, with the step costs of
    ``cost`` (default: forward 1, input-gradient half 1, weight-gradient half 1, whole backward 2)."""
    cost = cost or STEP_COST
    lists = [list(schedule_fn(P, V, M, r)) for r in range(P)]
    pos, clock = [0] * P, [0.0] * P
    done = {}                                      # (kind, virtual stage, micro-batch) -> finish time
    open_w = set()
    last_vs = P * V - 1
    while any(pos[r] < len(lists[r]) for r in range(P)):
        moved = False
        for r in range(P):
            while pos[r] < len(lists[r]):
                kind, c, m = lists[r][pos[r]]
                vs = c * P + r
                need = None
                if kind == "F" and vs > 0:
                    need = ("F", vs - 1, m)
                elif kind in ("B", "Bx"):
                    if ("F", vs, m) not in done:
                        raise RuntimeError(f"rank {r} runs the backward of micro-batch {m} before its forward")
                    need = ("B", vs + 1, m) if vs < last_vs else ("F", vs, m)
                elif kind == "W":
                    if (vs, m) not in open_w:
                        raise RuntimeError(f"rank {r} runs W of micro-batch {m} without an earlier Bx")
                    open_w.discard((vs, m))
                if need is not None and need not in done:
                    if kind == "W":
                        open_w.add((vs, m))
                    break
                start = max(clock[r], done.get(need, 0.0))
                clock[r] = start + cost[kind]
                if kind == "Bx":
                    open_w.add((vs, m))
                if kind != "W":
                    done[("B" if kind == "Bx" else kind, vs, m)] = clock[r]
                pos[r] += 1
                moved = True
        if not moved:
            raise RuntimeError(f"schedule deadlocks at positions {pos}")
    if open_w:
        raise RuntimeError("a Bx step has no W step: its weight gradients would be lost")
    return max(clock)


class ScheduleExecutor:
    def __init__(self, owner, schedule_fn):
        self.o = owner
        hcg = owner._hcg
        self.P, self.rank = owner.num_stages, owner.stage_id
        self.V = owner._layers.get_num_virtual_stages() if hasattr(owner._layers, "get_num_virtual_stages") else 1
        self.fn = schedule_fn
        ranks = [hcg.get_rank_from_stage(s) for s in range(self.P)]
        self._global = ranks
        # one communicator per ordered neighbour pair of the ring (every rank creates all of them, in the same order)
        self._chan = {}
        for s in range(self.P):
            d = (s + 1) % self.P
            if self.P == 1:
                break
            for a, b in ((s, d), (d, s)):
                if (a, b) not in self._chan:
                    self._chan[(a, b)] = C.new_group(sorted({ranks[a], ranks[b]}))
        self._meta = {}              # "act" / "grad" per virtual stage -> (shape, dtype, requires_grad)

    # ------------------------------------------------------------------ static analysis
    def _producer(self, kind, vs):
        """(rank, message kind) that produces the input of a step of virtual stage ``vs``."""
        if kind == "F":
            return (vs - 1) % self.P
        return (vs + 1) % self.P

    def _sends_of(self, steps, r):
        """Messages rank ``r`` emits, in order: (dst rank, ("act" | "grad", consumer vs, mb))."""
        last = self.P * self.V - 1
        out = []
        for kind, c, m in steps:
            vs = c * self.P + r
            if kind == "F" and vs < last:
                out.append(((r + 1) % self.P, ("act", vs + 1, m)))
            elif kind in ("B", "Bx") and vs > 0:
                out.append(((r - 1) % self.P, ("grad", vs - 1, m)))
        return out

    # ------------------------------------------------------------------ messaging
    def _send(self, t, dst, pending):
        g = self._chan[(self.rank, dst)]
        t = t.detach().contiguous()
        pending.append((C.isend(t, self._global[dst], g), t))

    def _recv_next(self, src, msg, like):
        from ...._core.dtype import default_device
        shape, dtype = like
        buf = torch.empty(shape, dtype=dtype, device=default_device())
        C.recv(buf, self._global[src], self._chan[(src, self.rank)])
        return buf

    def run(self, data, scaler=None, forward_only=False):
        o, P, V, r = self.o, self.P, self.V, self.rank
        M = o.accumulate_steps
        inputs, labels = data if isinstance(data, (tuple, list)) and len(data) == 2 else (data, None)
        sched = {q: list(self.fn(P, V, M, q)) for q in range(P)}
        if forward_only:
            sched = {q: [s for s in sched[q] if s[0] == "F"] for q in range(P)}
        incoming = {}                 # src rank -> ordered message ids destined to this rank
        for q in range(P):
            if q == r:
                continue
            for dst, msg in self._sends_of(sched[q], q):
                if dst == r:
                    incoming.setdefault(q, []).append(msg)
        if P == 1:
            incoming = {}
        cursor = {q: 0 for q in incoming}
        stash, pending = {}, []
        last_vs = P * V - 1
        ins, outs = {}, {}
        o.total_loss = None
        act_like = getattr(self, "_act_like", None)

        # Receives are posted ahead of their use (``PD_PP_PREFETCH`` messages per source, default 2; 0 = blocking
        # receive at the point of use): the order of the messages a peer sends is known from its schedule, so the
        # transfer of the next activation / gradient runs on the communicator's stream under this stage's compute and
        # the compute stream only waits for the one it consumes (the reference overlaps its p2p the same way:
        # pp_utils/p2p_communication.py batched isend / irecv on the comm stream).
        import collections
        import os
        depth = int(os.environ.get("PD_PP_PREFETCH", "2"))
        posted = {q: collections.deque() for q in incoming}
        likes = {"act": act_like[:2] if act_like is not None else None, "grad": getattr(self, "_out_like", None)}

        def post(src):
            from ...._core.dtype import default_device
            while len(posted[src]) < depth and cursor[src] < len(incoming[src]):
                nxt = incoming[src][cursor[src]]
                like = likes[nxt[0]]
                if like is None:            # shape not known yet (before the first activation went through)
                    return
                buf = torch.empty(like[0], dtype=like[1], device=default_device())
                w = C.irecv(buf, self._global[src], self._chan[(src, self.rank)])
                posted[src].append((nxt, buf, w))
                cursor[src] += 1

        def need(src, msg, like):
            likes[msg[0]] = like
            while msg not in stash:
                if not posted[src]:
                    post(src)
                if posted[src]:
                    nxt, buf, w = posted[src].popleft()
                    w.wait()
                    stash[nxt] = buf
                else:
                    nxt = incoming[src][cursor[src]]
                    cursor[src] += 1
                    stash[nxt] = self._recv_next(src, nxt, likes[nxt[0]] or like)
            post(src)
            return stash.pop(msg)

        from ....ops.functional import WeightGradStore
        deferred = {}                 # (chunk, micro-batch) -> weight-gradient closures queued by its Bx step
        WeightGradStore.split = any(s[0] == "Bx" for s in sched[r])
        for kind, c, m in sched[r]:
            vs = c * P + r
            if kind == "W":
                WeightGradStore.run(deferred.pop((c, m)))
                continue
            WeightGradStore.enabled = kind == "Bx"
            if kind == "F":
                if vs == 0:
                    x = o._load_micro_batch(inputs, m)
                else:
                    if act_like is None:
                        act_like = self._act_like = self._exchange_meta(None, (vs - 1) % P)
                    x = as_tensor(need((vs - 1) % P, ("act", vs, m), act_like[:2]))
                    x.requires_grad_(act_like[2] and x.is_floating_point() and not forward_only)
                out = o._layers.forward(x, chunk_id=c) if V > 1 else o._layers.forward(x)
                if vs == last_vs:
                    lab = o._load_micro_batch(labels, m)
                    loss = o._layers._loss_fn(out, lab) if not isinstance(lab, (tuple, list)) else o._layers._loss_fn(out, *lab)
                    if M > 1 and not o._delay_scale_loss:
                        loss = loss / M
                    o.total_loss = loss.detach() if o.total_loss is None else o.total_loss + loss.detach()
                    out = loss
                else:
                    if not getattr(self, "_meta_sent", False):
                        self._exchange_meta(out, (r + 1) % P)
                        self._meta_sent = True
                    self._send(out, (r + 1) % P, pending)
                    if likes["grad"] is None:
                        likes["grad"] = self._out_like = (list(out.shape), out.dtype)
                if not forward_only:
                    ins[(c, m)], outs[(c, m)] = x, out
            else:
                x, y = ins.pop((c, m)), outs.pop((c, m))
                if vs == last_vs:
                    (scaler.scale(y) if scaler else y).backward()
                else:
                    g = need((vs + 1) % P, ("grad", vs, m), (list(y.shape), y.dtype))
                    torch.autograd.backward([C._plain(y)], [C._plain(g)])
                if vs > 0 and isinstance(x, torch.Tensor) and x.requires_grad:
                    self._send(x.grad, (r - 1) % P, pending)
                    x.grad = None
                if kind == "Bx":
                    deferred[(c, m)] = WeightGradStore.pop()
            for q in posted:                  # keep the receive window full while the next step computes
                post(q)
        WeightGradStore.split = WeightGradStore.enabled = False
        assert not deferred, "weight gradients left in the store"
        assert not any(posted.values()), "posted receives left over"
        for w, _ in pending:
            w.wait()
        assert not stash and all(cursor[q] == len(incoming[q]) for q in incoming), "pipeline messages left over"
        if not forward_only:
            o._layers.allreduce_shared_weight_gradients()
        return o._broadcast_final_loss()

    def _exchange_meta(self, out, peer):
        """First activation of a run: the producer tells its consumer shape / dtype / requires_grad (all activations
        between stages share them)."""
        from ...._core.dtype import default_device
        from .pipeline_parallel import _DT
        n = 16
        if out is not None:
            m = [out.dim(), _DT.index(out.dtype), int(out.requires_grad), *out.shape]
            t = torch.tensor(m + [0] * (n - len(m)), dtype=torch.int64, device=default_device())
            C.send(t, self._global[peer], self._chan[(self.rank, peer)])
            return None
        t = torch.zeros(n, dtype=torch.int64, device=default_device())
        C.recv(t, self._global[peer], self._chan[(peer, self.rank)])
        m = t.tolist()
        return (m[3:3 + m[0]], _DT[m[1]], bool(m[2]))
