"""Re-export of the stage-to-stage transport used by the schedules
(fleet/meta_parallel/pp_utils/p2p_communication.py: ``SendRecvMeta`` :52, ``P2pHelper`` :573)."""
from ..pipeline_parallel import P2pHelper, SendRecvMeta  # noqa: F401

import torch

from .... import collective as _C
from .....framework.flags import flag as _flag

_hcg = None
_enable_partial_send_recv = True
_timers = None


def initialize_p2p_groups(hcg, enable_partial_send_recv=True, enable_timer=False):
    """Remembers the topology the module-level helpers use (p2p_communication.py:42)."""
    global _hcg, _enable_partial_send_recv, _timers
    _hcg, _enable_partial_send_recv = hcg, enable_partial_send_recv
    if enable_timer:
        from ....fleet.utils import timer_helper
        _timers = timer_helper.get_timers()


def _is_valid_send_recv_partial(tensor, mp_degree):
    """Partial send / receive cuts the flattened tensor into ``mp_degree`` equal parts: each tensor-parallel rank
    sends its part and the receivers all-gather, which divides pipeline traffic by the tensor-parallel degree."""
    return _enable_partial_send_recv and mp_degree > 1 and tensor.numel() % mp_degree == 0


def allgather_partial(tensor, nranks=1, rank_id=0, group=None, use_calc_stream=True):
    """Completes a tensor of which only part ``rank_id`` of ``nranks`` was received: all-gathers the parts over the
    tensor-parallel ``group`` in place (p2p_communication.py:272)."""
    if not _is_valid_send_recv_partial(tensor, nranks):
        return tensor
    flat = tensor.reshape(-1)
    parts = list(flat.chunk(nranks))
    _C.all_gather(parts, parts[rank_id].clone(), group=group)
    return tensor


class P2PonCalcStream:
    """One send or receive to run on the compute stream (p2p_communication.py:231); ``op`` is ``send`` / ``recv`` of
    ``paddle.distributed`` (or ``isend`` / ``irecv``)."""

    def __init__(self, op, tensor, peer, group, nranks=1, rank_id=0):
        name = getattr(op, "__name__", "")
        if name not in ("send", "recv", "isend", "irecv", "_send_on_calc_stream", "_recv_on_calc_stream"):
            raise RuntimeError("Invalid ``op`` function: expected a send or a receive")
        self.op, self.tensor, self.peer, self.group, self.nranks, self.rank_id = op, tensor, peer, group, nranks, rank_id
        self.is_send = "send" in name


def batch_send_recv_on_calc_stream(p2p_op_list):
    """Runs a list of ``P2PonCalcStream`` as one batch: all of them are posted before any is waited for, so a pair of
    ranks that send to each other cannot deadlock; with ``FLAGS_pp_check_naninf`` set, tensors to send are checked
    for inf / nan first (p2p_communication.py:286)."""
    import os

from .....framework.flags import flag as _flag
    if not p2p_op_list:
        return
    if _flag("pp_check_naninf"):
        for o in p2p_op_list:
            if o.is_send and o.tensor.is_floating_point() and not bool(torch.isfinite(o.tensor).all()):
                raise ValueError(f"Tensor contains inf or nan values at rank {_C.get_rank()}")
    ops = [_C.P2POp(_C.isend if o.is_send else _C.irecv, o.tensor, o.peer, o.group) for o in p2p_op_list]
    for task in _C.batch_isend_irecv(ops):
        task.wait()
