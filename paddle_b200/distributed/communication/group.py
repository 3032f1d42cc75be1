"""``paddle.distributed.communication.group`` module path (python/paddle/distributed/communication/group.py)."""
from ..collective import (Group, _get_default_group, _get_global_group, barrier, destroy_process_group,  # noqa: F401
                          get_backend, get_group, is_initialized, wait)


def is_available():
    import torch.distributed as tdist
    return tdist.is_available()


def _warn_cur_rank_not_in_group(group):
    return group is not None and not getattr(group, "is_member", lambda: True)()


def _get_or_throw_group_rank(global_rank, group):
    r = group.get_group_rank(global_rank)
    assert r >= 0, f"The input rank {global_rank} can not be found inside the group {group}"
    return r
