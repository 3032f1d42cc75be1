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


class Placement:
    """Which rank holds which virtual stage.  ``interleaved``: chunk c of rank r is virtual stage ``c * P + r`` (the
    layout of interleaved 1F1B).  ``zigzag``: even chunks run up the ranks, odd chunks run down - with two chunks the
    "V" of the zero-bubble V schedule: rank r holds stages ``r`` and ``2P - 1 - r``, so the first and the last stage
    share rank 0 and the turn-around between the chunks (stage P-1 -> P) is local to rank P-1."""

    def __init__(self, P, V, kind="interleaved"):
        assert kind in ("interleaved", "zigzag")
        self.P, self.V, self.kind = P, V, kind

    def vs(self, c, r):
        return c * self.P + (r if (self.kind == "interleaved" or c % 2 == 0) else self.P - 1 - r)

    def owner(self, vs):
        c, i = divmod(vs, self.P)
        return (i if (self.kind == "interleaved" or c % 2 == 0) else self.P - 1 - i), c


_ZBV_CACHE = {}


def zero_bubble_v(P, V, M, rank):
    """Zero-bubble V schedule (ZB-V / ``ZBVPP``: python/paddle/distributed/passes/pipeline_scheduler_pass/
    pipeline_zero_bubble.py:150-222 builds it with a greedy V-schedule creator over measured program costs).  Two chunks
    per rank in zigzag placement; backward is split into ``Bx`` (input gradients, on the critical path) and ``W``
    (weight gradients, which fill what would be bubbles).  The order is produced by a unit-cost list scheduling of the
    whole pipeline - at every tick a rank runs, in this order of preference, a ready ``Bx``, a ready forward of its
    second chunk, a forward of its first chunk while fewer than ``2 P`` chunk activations are alive, else a pending
    ``W`` - so it respects every dependency by construction.  Activations alive on a rank stay below ``3 P`` chunk
    activations whatever the number of micro-batches (the hand-tuned ZB-V of the paper holds ``2 P``); simulated makespan
    with unit costs: within ``P + 3`` of the bubble-free ``6 M`` (P = 8, M = 16: 104 against 96; interleaved 1F1B: 117)."""
    if V != 2:
        raise ValueError("the zero-bubble V schedule places exactly two chunks on every rank")
    key = (P, M)
    if key not in _ZBV_CACHE:
        _ZBV_CACHE[key] = _build_zbv(P, M)
    return list(_ZBV_CACHE[key][rank])


def _build_zbv(P, M):
    place = Placement(P, 2, "zigzag")
    last = 2 * P - 1
    done = {}                                   # (kind, vs, m) -> finish tick
    lists = [[] for _ in range(P)]
    next_f = [[0, 0] for _ in range(P)]         # next micro-batch to forward, per chunk
    next_b = [[0, 0] for _ in range(P)]
    pending_w = [[] for _ in range(P)]
    alive = [0] * P                             # chunk activations held (forward done, W not yet)
    total = P * 2 * M * 3
    count, t = 0, 0
    cap = 2 * P
    while count < total:
        fired = []
        for r in range(P):
            choice = None
            # 1. input-gradient backward, deeper chunk first
            for c in (1, 0):
                m = next_b[r][c]
                if m >= M:
                    continue
                vs = place.vs(c, r)
                if done.get(("F", vs, m), 1 << 30) > t:
                    continue
                dep = ("Bx", vs + 1, m) if vs < last else ("F", vs, m)
                if done.get(dep, 1 << 30) <= t:
                    choice = ("Bx", c, m)
                    break
            # 2. forward: second chunk when its input is there, else first chunk within the memory cap
            if choice is None:
                for c in (1, 0):
                    m = next_f[r][c]
                    if m >= M:
                        continue
                    vs = place.vs(c, r)
                    if vs > 0 and done.get(("F", vs - 1, m), 1 << 30) > t:
                        continue
                    if c == 0 and alive[r] >= cap:
                        continue
                    choice = ("F", c, m)
                    break
            # 3. weight gradients fill the rest
            if choice is None and pending_w[r]:
                c, m = pending_w[r][0]
                choice = ("W", c, m)
            if choice is not None:
                fired.append((r, choice))
        if not fired and count < total:
            # nothing ready anywhere at this tick although work is left: only possible while results of this very tick
            # are pending, which cannot happen with unit costs - guard against an endless loop all the same
            if t > 16 * total:
                raise RuntimeError("zero-bubble V scheduling did not converge")
        for r, (kind, c, m) in fired:
            vs = place.vs(c, r)
            lists[r].append((kind, c, m))
            count += 1
            if kind == "F":
                done[("F", vs, m)] = t + 1
                next_f[r][c] += 1
                alive[r] += 1
            elif kind == "Bx":
                done[("Bx", vs, m)] = t + 1
                next_b[r][c] += 1
                pending_w[r].append((c, m))
            else:
                pending_w[r].pop(0)
                alive[r] -= 1
        t += 1
    return lists


SCHEDULES = {"FThenB": f_then_b, "1F1B": one_f_one_b, "VPP": interleaved_1f1b, "interleaved_1f1b": interleaved_1f1b,
             "ZBH1": zero_bubble_h1, "ZBVPP": zero_bubble_v, "ZBV": zero_bubble_v}
# placement of the virtual stages each schedule is written for (default: interleaved)
PLACEMENTS = {"ZBVPP": "zigzag", "ZBV": "zigzag"}
_PLACEMENT_OF_FN = {zero_bubble_v: "zigzag"}


def placement_of(schedule_fn):
    return _PLACEMENT_OF_FN.get(schedule_fn, "interleaved")


STEP_COST = {"F": 1.0, "B": 2.0, "Bx": 1.0, "W": 1.0}


def validate(schedule_fn, P, V, M, cost=None):
    """Checks on the host that the per-rank lists form a deadlock-free global order (every step's input is produced
    by an earlier step of some rank, every ``Bx`` has exactly one later ``W``) and returns the makespan of a
    simulation in which a step starts when its rank is free and its input has been produced, with the step costs of
    ``cost`` (default: forward 1, input-gradient half 1, weight-gradient half 1, whole backward 2)."""
    cost = cost or STEP_COST
    place = Placement(P, V, placement_of(schedule_fn))
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
                vs = place.vs(c, r)
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
        self.place = Placement(self.P, self.V, placement_of(schedule_fn))
        if self.place.kind == "zigzag" and getattr(owner._layers, "_virtual_placement", "interleaved") != "zigzag":
            raise ValueError("this schedule needs PipelineLayer(..., virtual_placement='zigzag'): rank r must hold the "
                             "virtual stages r and 2P-1-r")
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
    def _sends_of(self, steps, r):
        """Messages rank ``r`` emits, in order: (dst rank, ("act" | "grad", consumer vs, mb)).  A hand-over between two
        virtual stages of the same rank (the turn of a zigzag placement) is not a message."""
        last = self.P * self.V - 1
        out = []
        for kind, c, m in steps:
            vs = self.place.vs(c, r)
            if kind == "F" and vs < last:
                dst = self.place.owner(vs + 1)[0]
                if dst != r:
                    out.append((dst, ("act", vs + 1, m)))
            elif kind in ("B", "Bx") and vs > 0:
                dst = self.place.owner(vs - 1)[0]
                if dst != r:
                    out.append((dst, ("grad", vs - 1, m)))
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
        if not hasattr(self, "_like_from"):
            self._like_from, self._meta_sent_to = {}, set()      # activation meta per producing / consuming peer
        act_like = next(iter(self._like_from.values()), None)

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
        local_act, local_grad = {}, {}       # hand-overs between two virtual stages of this rank
        place = self.place
        for kind, c, m in sched[r]:
            vs = place.vs(c, r)
            if kind == "W":
                WeightGradStore.run(deferred.pop((c, m)))
                continue
            WeightGradStore.enabled = kind == "Bx"
            if kind == "F":
                if vs == 0:
                    x = o._load_micro_batch(inputs, m)
                elif place.owner(vs - 1)[0] == r:
                    x = as_tensor(local_act.pop((vs, m)))
                    x.requires_grad_(x.is_floating_point() and not forward_only)
                else:
                    src = place.owner(vs - 1)[0]
                    if src not in self._like_from:
                        self._like_from[src] = self._exchange_meta(None, src)
                    act_like = self._like_from[src]
                    likes["act"] = act_like[:2]
                    x = as_tensor(need(src, ("act", vs, m), act_like[:2]))
                    x.requires_grad_(act_like[2] and x.is_floating_point() and not forward_only)
                out = o._layers.forward(x, chunk_id=c) if V > 1 else o._layers.forward(x)
                if vs == last_vs:
                    lab = o._load_micro_batch(labels, m)
                    loss = o._layers._loss_fn(out, lab) if not isinstance(lab, (tuple, list)) else o._layers._loss_fn(out, *lab)
                    if M > 1 and not o._delay_scale_loss:
                        loss = loss / M
                    o.total_loss = loss.detach() if o.total_loss is None else o.total_loss + loss.detach()
                    out = loss
                elif place.owner(vs + 1)[0] == r:
                    local_act[(vs + 1, m)] = C._plain(out).detach()
                else:
                    dst = place.owner(vs + 1)[0]
                    if dst not in self._meta_sent_to:
                        self._exchange_meta(out, dst)
                        self._meta_sent_to.add(dst)
                    self._send(out, dst, pending)
                    if likes["grad"] is None:
                        likes["grad"] = self._out_like = (list(out.shape), out.dtype)
                if not forward_only:
                    ins[(c, m)], outs[(c, m)] = x, out
            else:
                x, y = ins.pop((c, m)), outs.pop((c, m))
                if vs == last_vs:
                    (scaler.scale(y) if scaler else y).backward()
                elif place.owner(vs + 1)[0] == r:
                    torch.autograd.backward([C._plain(y)], [local_grad.pop((vs, m))])
                else:
                    g = need(place.owner(vs + 1)[0], ("grad", vs, m), (list(y.shape), y.dtype))
                    torch.autograd.backward([C._plain(y)], [C._plain(g)])
                if vs > 0 and isinstance(x, torch.Tensor) and x.requires_grad:
                    if place.owner(vs - 1)[0] == r:
                        local_grad[(vs - 1, m)] = C._plain(x.grad).detach()
                    else:
                        self._send(x.grad, place.owner(vs - 1)[0], pending)
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
        assert not local_act and not local_grad, "local hand-overs left over"
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
