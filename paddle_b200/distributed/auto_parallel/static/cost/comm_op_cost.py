"""Costs of the collectives (python/paddle/distributed/auto_parallel/static/cost/comm_op_cost.py).  ``comm_count`` is the
size of the local buffer taking part - for an all-gather the gathered result; the factor of each class is the share of
it that crosses the links per rank."""
from .base_cost import CommOpCost, register_op_cost


@register_op_cost
class AllreduceSumOpCost(CommOpCost):
    OP_TYPE = "c_allreduce_sum"
    ALIASES = ("all_reduce",)

    def volume_factor(self):
        n = self.rank_count
        return 2.0 * (n - 1) / n


@register_op_cost
class AllgatherOpCost(CommOpCost):
    OP_TYPE = "c_allgather"
    ALIASES = ("all_gather",)

    def volume_factor(self):
        n = self.rank_count
        return (n - 1) / n


@register_op_cost
class ReduceScatterOpCost(AllgatherOpCost):
    OP_TYPE = "c_reducescatter"
    ALIASES = ("reduce_scatter",)


@register_op_cost
class AlltoallOpCost(AllgatherOpCost):
    OP_TYPE = "all_to_all"


@register_op_cost
class BroadcastOpCost(CommOpCost):
    OP_TYPE = "c_broadcast"
    ALIASES = ("broadcast",)


@register_op_cost
class IdentityOpCost(CommOpCost):
    OP_TYPE = "c_identity"
    ALIASES = ("slice",)

    def calc_time(self):
        return 0.0


@register_op_cost
class SendOpCost(CommOpCost):
    OP_TYPE = "send_v2"
    ALIASES = ("send",)


@register_op_cost
class RecvOpCost(CommOpCost):
    OP_TYPE = "recv_v2"
    ALIASES = ("recv",)
