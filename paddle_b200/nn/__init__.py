"""``paddle.nn``"""
from . import functional, initializer  # noqa: F401
from .clip import ClipGradByGlobalNorm, ClipGradByNorm, ClipGradByValue  # noqa: F401
from .layer.common import *  # noqa: F401,F403
from .layer.layers import Layer, ParamAttr  # noqa: F401
from . import utils  # noqa: F401

from .layer.extras import *  # noqa: E402,F401,F403
from .layer.extras import (AdaptiveLogSoftmaxWithLoss, BeamSearchDecoder, BiRNN, Bilinear, GRUCell, HSigmoidLoss, LSTMCell,  # noqa: E402,F401
                           ParameterDict, RNN, RNNCellBase, SimpleRNNCell, SpectralNorm, dynamic_decode)


from .._core.submodule_alias import alias_submodules as _alias  # noqa: E402
_alias(__name__, ("loss", "activation", "conv", "norm", "pooling", "rnn", "transformer", "vision", "container", "distance", "common"))
_alias(__name__ + ".layer", ("loss", "activation", "conv", "norm", "pooling", "rnn", "transformer", "vision", "container", "distance"))
