"""``paddle.Tensor`` on top of ``torch.Tensor``.

The reference's Tensor is a pybind type (paddle/fluid/pybind/eager.cc, eager_method.cc) that Python
then patches with ~300 methods (python/paddle/base/dygraph/tensor_patch_methods.py,
math_op_patch.py).  Here the storage, dispatcher and autograd engine are PyTorch's; this subclass
supplies Paddle's names and semantics: ``stop_gradient`` (inverse of ``requires_grad``), ``shape`` as
a list, ``astype``, ``numpy``, ``clear_gradient``, ``_register_backward_hook``, axis-style reductions,
permutation-style ``transpose`` and so on.  Results of torch operators on a ``Tensor`` stay ``Tensor``
through ``__torch_function__``.
"""
from __future__ import annotations

import numpy as np
import torch

from . import dtype as _dt
from .unique_name import generate as _uniq


class _Size(int):
    def __new__(cls, numel, shape):
        o = int.__new__(cls, numel)
        o._shape = shape
        return o

    def __call__(self, dim=None):
        return self._shape if dim is None else self._shape[dim]


class _TensorMeta(type(torch.Tensor)):
    """``type(t)`` prints as the reference's ``<class 'paddle.Tensor'>``; the class keeps its real module so that pickles
    (data-loader workers, checkpoints) resolve it without the ``paddle`` alias package."""

    def __repr__(cls):
        return "<class 'paddle.Tensor'>" if cls.__name__ == "Tensor" else super().__repr__()


class Tensor(torch.Tensor, metaclass=_TensorMeta):
    """Dense tensor with PaddlePaddle's Python surface."""

    # ---- identity / meta
    @property
    def stop_gradient(self) -> bool:
        return not (self.requires_grad or getattr(self, "_int_wants_grad", False))

    @stop_gradient.setter
    def stop_gradient(self, v: bool):
        if not (self.dtype.is_floating_point or self.dtype.is_complex):
            # integer tensors carry the flag (the reference allows it) but never take part in autograd
            self._int_wants_grad = not v
            return
        if self.is_leaf or not v:
            self.requires_grad_(not v)
        # a non-leaf cannot be switched off in place; Paddle users then call detach()

    @property
    def shape(self):  # Paddle returns a python list
        return list(torch.Tensor.shape.__get__(self))

    @property
    def place(self):
        return self.device

    @property
    def persistable(self):
        return getattr(self, "_persistable", False)

    @persistable.setter
    def persistable(self, v):
        self._persistable = bool(v)

    @property
    def name(self):
        n = getattr(self, "_pd_name", None)
        if n is None:
            n = _uniq("generated_tensor")
            self._pd_name = n
        return n

    @name.setter
    def name(self, v):
        self._pd_name = v

    def numel(self):  # noqa: D401 - paddle returns a 0-d tensor; an int is accepted everywhere it matters
        return torch.Tensor.numel(self)

    @property
    def size(self):
        """Paddle: the number of elements (an int).  The returned int is also callable like ``torch.Tensor.size`` so
        that library code written against torch keeps working on this subclass."""
        return _Size(torch.Tensor.numel(self), torch.Tensor.shape.__get__(self))

    def dim(self):
        return torch.Tensor.dim(self)

    ndimension = dim

    @property
    def T(self):
        return self.permute(*reversed(range(self.dim())))

    # ---- conversion
    def numpy(self):
        t = self.detach()
        if t.dtype == torch.bfloat16:
            return t.float().cpu().numpy()
        return torch.Tensor.numpy(t.cpu().resolve_conj().resolve_neg())

    def astype(self, dtype):
        return self.to(_dt.to_torch(dtype))

    cast = astype

    def cpu(self):
        return torch.Tensor.cpu(self)

    def cuda(self, device_id=None, blocking=True):
        return torch.Tensor.cuda(self, device_id) if device_id is not None else torch.Tensor.cuda(self)

    def pin_memory(self):
        return torch.Tensor.pin_memory(self)

    def clone(self, *, memory_format=None):
        if memory_format is None:
            return torch.Tensor.clone(self)
        return torch.Tensor.clone(self, memory_format=memory_format)

    def tolist(self):
        return torch.Tensor.tolist(self)

    def item(self, *idx):
        """Python scalar of a one-element tensor; ``item(i)`` reads element ``i`` of the flattened tensor and
        ``item(i, j, ...)`` the element at that index."""
        plain = self.detach().as_subclass(torch.Tensor)
        if len(idx) == 1 and plain.dim() != 1:
            return plain.reshape(-1)[int(idx[0])].item()
        if idx:
            return plain[tuple(int(i) for i in idx)].item()
        return plain.item()

    @property
    def inplace_version(self):
        """How many in-place operations have written this tensor."""
        return self._version

    def _md5sum(self):
        """MD5 of the tensor's bytes (debugging aid to compare tensors across runs)."""
        import hashlib
        return hashlib.md5(self.detach().cpu().contiguous().as_subclass(torch.Tensor).numpy().tobytes()).hexdigest()

    def element_size(self):
        return torch.Tensor.element_size(self)

    # ---- autograd
    @property
    def grad(self):
        g = torch.Tensor.grad.__get__(self)
        return None if g is None else (g if isinstance(g, Tensor) else g.as_subclass(Tensor))

    @grad.setter
    def grad(self, v):
        torch.Tensor.grad.__set__(self, v)

    def backward(self, grad_tensor=None, retain_graph=False):
        """A non-scalar tensor starts its backward pass from a gradient of ones (the reference's rule)."""
        if grad_tensor is None and self.dim() > 0 and self.numel() != 1:
            grad_tensor = torch.ones_like(self.detach().as_subclass(torch.Tensor))
        torch.Tensor.backward(self, gradient=grad_tensor, retain_graph=retain_graph)

    def clear_gradient(self, set_to_zero=True):
        if self.grad is not None:
            if set_to_zero:
                self.grad.zero_()
            else:
                self.grad = None

    clear_grad = clear_gradient

    def gradient(self):
        return None if self.grad is None else self.grad.numpy()

    def _register_backward_hook(self, hook):
        """Hook fired once the gradient of a leaf has been accumulated (Paddle's reduce hooks:
        paddle/fluid/eager/accumulation/accumulation_node.cc)."""
        handle = self.register_post_accumulate_grad_hook(lambda p: hook())
        return handle

    def register_hook(self, hook):
        return torch.Tensor.register_hook(self, hook)

    def _clear_data(self):
        self.data = torch.empty(0, dtype=self.dtype, device=self.device)

    def _clear(self):
        self._clear_data()

    def _is_initialized(self):
        return torch.Tensor.numel(self) > 0 or self.dim() == 0

    def _share_buffer_to(self, other):
        other.data = self.data

    def get_tensor(self):
        return self

    def value(self):
        return self

    def set_value(self, value):
        v = value if isinstance(value, torch.Tensor) else torch.as_tensor(np.asarray(value))
        with torch.no_grad():
            self.data.copy_(v.to(self.dtype).reshape(self.data.shape))

    def copy_(self, other, blocking=True):
        return torch.Tensor.copy_(self, other, non_blocking=not blocking)

    def _copy_to(self, place, blocking=True):
        return self.to(place, non_blocking=not blocking)

    def fill_(self, v):
        return torch.Tensor.fill_(self, v)

    def zero_(self):
        return torch.Tensor.zero_(self)

    def scale_(self, scale=1.0, bias=0.0):
        return self.mul_(scale).add_(bias) if bias else self.mul_(scale)

    # ---- Paddle-semantics overrides of same-named torch methods
    def transpose(self, *perm, **kw):
        if "perm" in kw:
            perm = (kw["perm"],)
        if len(perm) == 1 and isinstance(perm[0], (list, tuple)):
            return self.permute(*perm[0])
        return torch.Tensor.transpose(self, *perm)

    def reshape(self, *shape, **kw):
        if "shape" in kw:
            shape = (kw["shape"],)
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = tuple(shape[0])
        shape = tuple(int(s) for s in shape)
        return torch.Tensor.reshape(self, shape)

    def reshape_(self, *shape):
        r = self.reshape(*shape)
        self.data = r.data
        return self

    def expand(self, *shape, **kw):
        if "shape" in kw:
            shape = (kw["shape"],)
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = tuple(shape[0])
        return torch.Tensor.expand(self, *shape)

    def split(self, num_or_sections, axis=0, dim=None):
        axis = axis if dim is None else dim
        if isinstance(num_or_sections, int):
            n = self.shape[axis]                       # the global size for a distributed tensor
            return list(torch.Tensor.split(self, n // num_or_sections, axis))
        secs = list(num_or_sections)
        if -1 in secs:
            n = self.shape[axis]
            secs[secs.index(-1)] = n - (sum(secs) + 1)
        return list(torch.Tensor.split(self, secs, axis))

    def chunk(self, chunks, axis=0, dim=None):
        return list(torch.Tensor.chunk(self, chunks, axis if dim is None else dim))

    def unbind(self, axis=0):
        return list(torch.Tensor.unbind(self, axis))

    def squeeze(self, axis=None):
        if axis is None:
            return torch.Tensor.squeeze(self)
        if isinstance(axis, (list, tuple)):
            return torch.Tensor.squeeze(self, tuple(axis))
        return torch.Tensor.squeeze(self, axis)

    def unsqueeze(self, axis):
        if isinstance(axis, (list, tuple)):
            r = self
            for a in sorted(axis):
                r = torch.Tensor.unsqueeze(r, a)
            return r
        return torch.Tensor.unsqueeze(self, axis)

    def flatten(self, start_axis=0, stop_axis=-1):
        return torch.Tensor.flatten(self, start_axis, stop_axis)

    def tile(self, repeat_times):
        return torch.Tensor.repeat(self, *repeat_times) if isinstance(repeat_times, (list, tuple)) else torch.Tensor.repeat(self, repeat_times)

    def gather(self, index, axis=0):
        if isinstance(index, int):  # torch-style call gather(dim, index)
            return torch.Tensor.gather(self, index, axis)
        return torch.index_select(self, axis, index.reshape(-1))

    def _reduce(self, fn, axis, keepdim, **kw):
        if axis is None:
            return fn(self, **kw) if not keepdim else fn(self, dim=tuple(range(self.dim())), keepdim=True, **kw)
        if isinstance(axis, (list, tuple)):
            axis = tuple(axis)
        return fn(self, dim=axis, keepdim=keepdim, **kw)

    def sum(self, axis=None, dtype=None, keepdim=False, dim=None):
        axis = axis if dim is None else dim
        kw = {"dtype": _dt.to_torch(dtype)} if dtype is not None else {}
        return self._reduce(torch.sum, axis, keepdim, **kw)

    def mean(self, axis=None, keepdim=False, dim=None):
        return self._reduce(torch.mean, axis if dim is None else dim, keepdim)

    def prod(self, axis=None, keepdim=False, dtype=None):
        if axis is None:
            return torch.prod(self)
        return torch.prod(self, dim=axis, keepdim=keepdim)

    def max(self, axis=None, keepdim=False, dim=None):
        axis = axis if dim is None else dim
        if isinstance(axis, torch.Tensor):
            return torch.maximum(self, axis)
        if axis is None:
            return torch.amax(self) if not keepdim else torch.amax(self, dim=tuple(range(self.dim())), keepdim=True)
        return torch.amax(self, dim=axis, keepdim=keepdim)

    def min(self, axis=None, keepdim=False, dim=None):
        axis = axis if dim is None else dim
        if isinstance(axis, torch.Tensor):
            return torch.minimum(self, axis)
        if axis is None:
            return torch.amin(self) if not keepdim else torch.amin(self, dim=tuple(range(self.dim())), keepdim=True)
        return torch.amin(self, dim=axis, keepdim=keepdim)

    def argmax(self, axis=None, keepdim=False, dtype="int64"):
        r = torch.argmax(self, dim=axis, keepdim=keepdim)
        return r.to(_dt.to_torch(dtype))

    def argmin(self, axis=None, keepdim=False, dtype="int64"):
        return torch.argmin(self, dim=axis, keepdim=keepdim).to(_dt.to_torch(dtype))

    def std(self, axis=None, unbiased=True, keepdim=False):
        return torch.std(self, dim=axis, unbiased=unbiased, keepdim=keepdim)

    def var(self, axis=None, unbiased=True, keepdim=False):
        return torch.var(self, dim=axis, unbiased=unbiased, keepdim=keepdim)

    def all(self, axis=None, keepdim=False):
        return torch.all(self) if axis is None else torch.all(self, dim=axis, keepdim=keepdim)

    def any(self, axis=None, keepdim=False):
        return torch.any(self) if axis is None else torch.any(self, dim=axis, keepdim=keepdim)

    def norm(self, p=2, axis=None, keepdim=False):
        if p == "fro":
            p = 2
        return torch.linalg.vector_norm(self, ord=p, dim=axis, keepdim=keepdim)

    def topk(self, k, axis=-1, largest=True, sorted=True):
        return torch.topk(self, k, dim=axis, largest=largest, sorted=sorted)

    def cumsum(self, axis=None, dtype=None):
        if axis is None:
            return torch.cumsum(self.reshape(-1), 0)
        return torch.cumsum(self, axis)

    def matmul(self, y, transpose_x=False, transpose_y=False):
        a = self.mT if transpose_x and self.dim() > 1 else self
        b = y.mT if transpose_y and y.dim() > 1 else y
        return torch.matmul(a, b)

    def scale(self, scale=1.0, bias=0.0, bias_after_scale=True):
        return self * scale + bias if bias_after_scale else (self + bias) * scale

    def concat(self, others, axis=0):
        return torch.cat([self, *others], axis)

    def astype_(self, dtype):
        self.data = self.data.to(_dt.to_torch(dtype))
        return self

    def is_dense(self):
        return not self.is_sparse

    def is_dist(self):
        return getattr(self, "_dist_attr", None) is not None

    def __deepcopy__(self, memo):
        r = as_tensor(self.detach().clone())
        r.stop_gradient = self.stop_gradient
        memo[id(self)] = r
        return r

    def __repr__(self):
        from ..tensor.to_string import to_string
        return to_string(self)

    __str__ = __repr__

    def __float__(self):
        return float(torch.Tensor.item(self.detach()))

    def __int__(self):
        return int(torch.Tensor.item(self.detach()))

    def __hash__(self):
        return id(self)

    def __bool__(self):
        return bool(torch.Tensor.item(self)) if torch.Tensor.numel(self) == 1 else torch.Tensor.__bool__(self)


class EagerParamBase(Tensor):
    """Trainable parameter (python/paddle/base/framework.py ``EagerParamBase``)."""

    def initialize(self):
        """Run the initializer that ``paddle.LazyGuard`` deferred (no effect on an initialised parameter)."""
        init = self.__dict__.pop("_deferred_init", None)
        if init is not None:
            with torch.no_grad():
                init(self)
        return self

    @staticmethod
    def __new__(cls, data, trainable=True, name=None):
        t = torch.Tensor._make_subclass(cls, data.detach(), trainable)
        return t

    def __init__(self, data, trainable=True, name=None):
        self._pd_name = name or _uniq("param")
        self.optimize_attr = {"learning_rate": 1.0}
        self.regularizer = None
        self.do_model_average = None
        self.need_clip = True
        self.is_distributed = False
        self._persistable = True
        self.main_grad = None

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        """The result of an operator on a parameter is an ordinary tensor (only in-place operators hand the
        parameter itself back)."""
        ret = super().__torch_function__(func, types, args, kwargs or {})

        def conv(r):
            if type(r) is EagerParamBase and not any(r is a for a in args):
                return r.as_subclass(Tensor)
            return r
        if isinstance(ret, (tuple, list)):
            return type(ret)(conv(r) for r in ret)
        return conv(ret)

    @property
    def trainable(self):
        return self.requires_grad

    @trainable.setter
    def trainable(self, v):
        self.requires_grad_(bool(v))

    def __deepcopy__(self, memo):
        r = EagerParamBase(self.detach().clone(), self.trainable, name=self._pd_name)
        for k in ("optimize_attr", "regularizer", "need_clip", "is_distributed"):
            setattr(r, k, getattr(self, k))
        memo[id(self)] = r
        return r

    def __reduce_ex__(self, proto):
        return (_rebuild_param, (self.detach().cpu().as_subclass(torch.Tensor), self.trainable, self._pd_name))


Parameter = EagerParamBase


def _rebuild_param(data, trainable, name):
    return EagerParamBase(data, trainable, name)


def as_tensor(t: torch.Tensor) -> Tensor:
    """View a plain torch tensor as a paddle Tensor (no copy)."""
    if isinstance(t, Tensor):
        return t
    return t.as_subclass(Tensor)



def to_tensor(data, dtype=None, place=None, stop_gradient=True):
    """``paddle.to_tensor`` (python/paddle/tensor/creation.py)."""
    td = _dt.to_torch(dtype) if dtype is not None else None
    dev = _dt.to_device(place)
    if isinstance(data, torch.Tensor):
        t = data.detach().clone()
        if td is not None:
            t = t.to(td)
        if dev is not None:
            t = t.to(dev)
    else:
        arr = np.asarray(data)
        if td is None:
            if arr.dtype == np.float64 and not isinstance(data, np.ndarray):
                td = _dt.get_default_dtype()
            elif arr.dtype == np.complex128 and not isinstance(data, np.ndarray):
                # Python complex numbers follow the default float dtype: complex64 unless the default is float64
                td = torch.complex128 if _dt.get_default_dtype() == torch.float64 else torch.complex64
            elif arr.dtype == np.uint16:  # bf16 bit pattern as stored by paddle.save
                t = torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
                t = t.to(dev or _dt.default_device())
                r = as_tensor(t)
                r.stop_gradient = stop_gradient
                return r
        t = torch.as_tensor(arr)
        if td is not None:
            t = t.to(td)
        t = t.to(dev or _dt.default_device())
    r = as_tensor(t)
    if not stop_gradient:
        r.stop_gradient = False
    return r
