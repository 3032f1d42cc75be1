"""Cost model of the planner (python/paddle/distributed/auto_parallel/static/cost/__init__.py)."""
from .base_cost import (COMM_OP_TYPE, NON_COMP_TYPE, CommContext, CommOpCost, CompOpCost, Cost, OpCost,  # noqa: F401
                        _g_op_cost_factory, build_comm_desc, register_op_cost)
from .comm_op_cost import (AllgatherOpCost, AllreduceSumOpCost, AlltoallOpCost, BroadcastOpCost, IdentityOpCost,  # noqa: F401
                           RecvOpCost, ReduceScatterOpCost, SendOpCost)
from .comp_op_cost import (ElementwiseOpCost, EmbeddingOpCost, FlashAttnOpCost, LayerNormOpCost, LayoutOpCost,  # noqa: F401
                           MatmulV2OpCost, OtherOpCost, ReduceSumOpCost, SoftmaxOpCost, SoftmaxWithCrossEntropyOpCost)
from .estimate_cost import CostEstimator, get_cost_from_engine  # noqa: F401
