"""Attention over a sequence that is split across the ``sep`` (segment-parallel) group.

The reference only carries the ``sep`` axis through the topology and broadcasts parameters over it
(python/paddle/distributed/fleet/meta_parallel/segment_parallel.py:26-40; gradients are all-reduced over the axis in
fleet/utils/hybrid_parallel_util.py:262); the attention that has to see the whole sequence is left to the model.
Two standard ways to provide it, both differentiable, both on the group's collectives (NCCL on GPUs, gloo on CPU):

* :func:`ulysses_attention` - all-to-all: every rank swaps its sequence shard of all heads for the full sequence of
  ``heads / n`` heads, runs ordinary (flash) attention on them and swaps back.  Two all-to-alls per direction, the
  attention kernel itself is unchanged; needs ``heads % n == 0``.
* :func:`ring_attention` - the key/value shards travel around the ring (batched send / recv), each rank attends its
  queries to one shard per step and merges the partial results with their log-sum-exp; memory stays at one shard,
  any head count; causal masking uses the shards' global positions.

Layout ``[batch, seq_local, heads, head_dim]``; rank r of the group holds tokens ``[r * seq_local, (r + 1) * seq_local)``.
"""
from __future__ import annotations

import math

import torch

from ...._core.tensor import as_tensor
from ... import collective as C


def _plain(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


# ------------------------------------------------------------------------------------------------ Ulysses
class _SeqToHead(torch.autograd.Function):
    """[b, s/n, h, d] -> [b, s, h/n, d] (forward); the inverse exchange in backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _a2a(x, group, scatter_heads=True)

    @staticmethod
    def backward(ctx, g):
        return _a2a(g.contiguous(), ctx.group, scatter_heads=False), None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _a2a(x, group, scatter_heads=False)

    @staticmethod
    def backward(ctx, g):
        return _a2a(g.contiguous(), ctx.group, scatter_heads=True), None


def _a2a(x, group, scatter_heads):
    n = group.nranks
    if n == 1:
        return x
    b, s, h, d = x.shape
    if scatter_heads:
        assert h % n == 0, f"ulysses attention needs heads ({h}) divisible by the sep degree ({n})"
        # piece p = heads [p*h/n, (p+1)*h/n) of my tokens -> rank p; I receive my head group for every rank's tokens
        send = x.reshape(b, s, n, h // n, d).permute(2, 0, 1, 3, 4).contiguous()      # [n, b, s, h/n, d]
        recv = torch.empty_like(send)
        C._alltoall_single_io(send.view(n * b, -1), recv.view(n * b, -1), group=group)
        return recv.permute(1, 0, 2, 3, 4).reshape(b, n * s, h // n, d)               # sequence in rank order
    assert s % n == 0
    send = x.reshape(b, n, s // n, h, d).permute(1, 0, 2, 3, 4).contiguous()          # [n, b, s/n, h, d]
    recv = torch.empty_like(send)
    C._alltoall_single_io(send.view(n * b, -1), recv.view(n * b, -1), group=group)
    return recv.permute(1, 2, 0, 3, 4).reshape(b, s // n, n * h, d)                   # heads in rank order


def ulysses_attention(q, k, v, group, causal=False, scale=None, attn_fn=None):
    """Attention over the full sequence for ``q / k / v [b, s_local, h, d]`` sharded along the sequence over
    ``group``.  ``attn_fn(q, k, v, causal, scale)`` defaults to the framework's flash attention."""
    if attn_fn is None:
        attn_fn = _default_attention
    qh = _SeqToHead.apply(_plain(q), group)
    kh = _SeqToHead.apply(_plain(k), group)
    vh = _SeqToHead.apply(_plain(v), group)
    o = attn_fn(qh, kh, vh, causal, scale)
    return as_tensor(_HeadToSeq.apply(_plain(o).contiguous(), group))


def _default_attention(q, k, v, causal, scale):
    from ....nn.functional.flash_attention import flash_attention
    out = flash_attention(as_tensor(q), as_tensor(k), as_tensor(v), causal=causal, scale=scale) \
        if "scale" in flash_attention.__code__.co_varnames else flash_attention(as_tensor(q), as_tensor(k), as_tensor(v),
                                                                                causal=causal)
    return out[0] if isinstance(out, tuple) else out


# ------------------------------------------------------------------------------------------------ ring attention
def _block_attention(q, k, v, scale, mask):
    """Partial attention of q against one key/value shard: (unnormalised-by-global output, log-sum-exp) in fp32.
    q [b, sq, h, d], k / v [b, sk, hk, d] (grouped-query: h % hk == 0); mask [sq, sk] bool (True = visible) or None."""
    b, sq, h, d = q.shape
    hk = k.shape[2]
    if hk != h:
        k = k.repeat_interleave(h // hk, dim=2)
        v = v.repeat_interleave(h // hk, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                                  # [b, h, sq]; -inf where nothing is visible
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse).unsqueeze(-1))
    o = torch.einsum("bhqk,bkhd->bqhd", p, v.float())                 # normalised within this shard
    return o, lse


def _ring_exchange(t, group):
    """Send ``t`` to the next rank of the ring, receive the previous rank's tensor."""
    n, r = group.nranks, group.rank
    out = torch.empty_like(t)
    nxt, prv = group.ranks[(r + 1) % n], group.ranks[(r - 1) % n]
    ops = [C.P2POp(C.isend, t.contiguous(), nxt, group), C.P2POp(C.irecv, out, prv, group)]
    for task in C.batch_isend_irecv(ops):
        task.wait()
    return out


def ring_attention(q, k, v, group, causal=False, scale=None):
    """Blockwise attention with the key/value shards rotating around ``group``.  Written with differentiable torch
    ops, so backward sends the key/value gradients back around the ring through autograd of the exchanges."""
    q, k, v = _plain(q), _plain(k), _plain(v)
    n, r = group.nranks, group.rank
    b, s, h, d = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    acc_o = None
    acc_lse = None
    kv = torch.cat([k, v], dim=-1)
    pos_q = torch.arange(s, device=q.device) + r * s
    for step in range(n):
        src = (r - step) % n                                          # owner of the shard held at this step
        ks, vs = kv[..., :d], kv[..., d:]
        mask = None
        skip = False
        if causal:
            if src > r:
                skip = True                                           # entirely in the future
            elif src == r:
                pos_k = torch.arange(s, device=q.device) + src * s
                mask = pos_k[None, :] <= pos_q[:, None]
        if not skip:
            o, lse = _block_attention(q, ks, vs, scale, mask)
            if acc_o is None:
                acc_o, acc_lse = o, lse
            else:
                new_lse = torch.logaddexp(acc_lse, lse)
                w_old = torch.exp(acc_lse - new_lse).permute(0, 2, 1).unsqueeze(-1)
                w_new = torch.exp(lse - new_lse).permute(0, 2, 1).unsqueeze(-1)
                acc_o, acc_lse = acc_o * w_old + o * w_new, new_lse
        else:
            # a skipped shard still has to take part in backward: every rank must run the gradient exchange of every
            # shift, or the ranks that did use the shard wait for a partner that never comes
            acc_o = acc_o + kv.float().sum() * 0.0
        if step + 1 < n:
            kv = _RingShift.apply(kv, group)
    return as_tensor(acc_o.to(q.dtype))


class _RingShift(torch.autograd.Function):
    """Forward: pass the tensor to the next rank.  Backward: pass the gradient to the previous rank."""

    @staticmethod
    def forward(ctx, t, group):
        ctx.group = group
        return _ring_exchange(t, group)

    @staticmethod
    def backward(ctx, g):
        group = ctx.group
        n, r = group.nranks, group.rank
        out = torch.empty_like(g)
        nxt, prv = group.ranks[(r + 1) % n], group.ranks[(r - 1) % n]
        ops = [C.P2POp(C.isend, g.contiguous(), prv, group), C.P2POp(C.irecv, out, nxt, group)]
        for task in C.batch_isend_irecv(ops):
            task.wait()
        return out, None
