"""``paddle.optimizer``"""
from . import lr  # noqa: F401
from .adamw import Adam, Adamax, AdamW  # noqa: F401
from .optimizer import L1Decay, L2Decay, Optimizer  # noqa: F401
from .sgd import SGD, Adadelta, Adagrad, Lamb, Momentum, RMSProp  # noqa: F401
from .extras import ASGD, LBFGS, NAdam, RAdam, Rprop  # noqa: F401
