"""The closed set of primitive operators a decomposed program may contain
(python/paddle/decomposition/primitives.py; paddle/fluid/primitive/primitive.yaml).  Names are the recorded call names
of the static-graph mode: torch functions / tensor methods."""

_ELEMENTWISE = """add sub subtract mul multiply div divide true_divide neg abs exp log sqrt rsqrt pow erf tanh sin cos
    maximum minimum where eq ne lt le gt ge logical_and logical_or logical_not floor ceil round sign reciprocal
    __add__ __radd__ __sub__ __rsub__ __mul__ __rmul__ __truediv__ __rtruediv__ __neg__ __pow__ __rpow__
    __eq__ __ne__ __lt__ __le__ __gt__ __ge__ __and__ __or__ __invert__ expm1 log1p sigmoid clamp""".split()
_REDUCE = "sum amax amin max min prod mean".split()
_SHAPE = """reshape view transpose permute expand expand_as broadcast_to squeeze unsqueeze cat concat stack split chunk
    slice __getitem__ flatten contiguous t clone detach type_as to float bfloat16 half double _to_copy flip gather
    index_select scatter narrow unbind tile repeat long int bool""".split()
_CREATE = "zeros ones full zeros_like ones_like full_like empty empty_like arange tensor as_tensor scalar_tensor".split()
_CONTRACT = "matmul mm bmm".split()
_MISC = "cast assign cumsum argmax argmin topk sort rand rand_like randn bernoulli uniform_ dim size numel".split()

PRIMITIVES = frozenset(_ELEMENTWISE + _REDUCE + _SHAPE + _CREATE + _CONTRACT + _MISC)
