"""Costs of compute operators by class (python/paddle/distributed/auto_parallel/static/cost/comp_op_cost.py lists one
class per operator type with measured tables; here a class per operator family computes flops and bytes of the LOCAL
piece from the completed shapes, and the base class turns them into time on the device's roofline)."""
from .base_cost import CompOpCost, register_op_cost


@register_op_cost
class MatmulV2OpCost(CompOpCost):
    OP_TYPE = "matmul"
    ALIASES = ("matmul_v2", "mul", "linear", "conv2d", "fused_gemm_epilogue")
    FLOP_EFFICIENCY = 0.9


@register_op_cost
class FlashAttnOpCost(CompOpCost):
    OP_TYPE = "attention"
    ALIASES = ("flash_attn", "scaled_dot_product_attention")
    FLOP_EFFICIENCY = 0.45          # the attention kernels reach a little under half of the GEMM rate


@register_op_cost
class EmbeddingOpCost(CompOpCost):
    OP_TYPE = "embedding"
    ALIASES = ("lookup_table_v2", "c_embedding")


@register_op_cost
class LayerNormOpCost(CompOpCost):
    OP_TYPE = "norm"
    ALIASES = ("layer_norm", "rms_norm")


@register_op_cost
class SoftmaxOpCost(CompOpCost):
    OP_TYPE = "softmax"


@register_op_cost
class SoftmaxWithCrossEntropyOpCost(CompOpCost):
    OP_TYPE = "loss"
    ALIASES = ("softmax_with_cross_entropy", "c_softmax_with_cross_entropy")


@register_op_cost
class ReduceSumOpCost(CompOpCost):
    OP_TYPE = "reduce"
    ALIASES = ("reduce_sum", "reduce_mean", "reduce_max")


@register_op_cost
class ElementwiseOpCost(CompOpCost):
    OP_TYPE = "elementwise"
    ALIASES = ("elementwise_add", "elementwise_mul", "gelu", "relu", "dropout", "cast", "scale")


@register_op_cost
class LayoutOpCost(CompOpCost):
    """Views cost nothing; a transpose that is materialised later is charged to its consumer."""
    OP_TYPE = "layout"
    ALIASES = ("reshape2", "transpose2", "squeeze2", "unsqueeze2", "slice", "split", "concat")

    def calc_time(self):
        return 0.0


@register_op_cost
class OtherOpCost(CompOpCost):
    OP_TYPE = "other"
