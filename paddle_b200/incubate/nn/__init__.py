"""``paddle.incubate.nn``"""
from . import functional  # noqa: F401
from .layer.fused_transformer import (FusedBiasDropoutResidualLayerNorm, FusedDropout, FusedDropoutAdd, FusedFeedForward,  # noqa: F401
                                      FusedLinear, FusedMultiHeadAttention, FusedMultiTransformer,
                                      FusedTransformerEncoderLayer)

__all__ = ["FusedMultiHeadAttention", "FusedFeedForward", "FusedTransformerEncoderLayer", "FusedMultiTransformer",
           "FusedLinear", "FusedBiasDropoutResidualLayerNorm", "FusedDropoutAdd", "FusedDropout"]
from . import attn_bias  # noqa: F401,E402
from .memory_efficient_attention import memory_efficient_attention  # noqa: F401,E402
