"""Remaining ``paddle.nn`` layers (python/paddle/nn/layer/{rnn,pooling,loss,common,vision,norm,container}.py): RNN cells
and wrappers, beam-search decoding, un-pooling / fractional / Lp pooling, additional losses, small utility layers."""
from __future__ import annotations

import math

import torch

from ..._core.tensor import as_tensor
from .. import functional as F
from ..functional import extras as FX
from ..initializer import Constant, Uniform
from .layers import Layer


def _p(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else x


def _fn_layer(name, fn, arg_names, defaults=()):
    """Layer whose constructor stores ``arg_names`` and whose forward calls ``fn(*inputs, **stored)``."""
    d = dict(zip(arg_names[len(arg_names) - len(defaults):], defaults))

    def __init__(self, *args, **kwargs):
        Layer.__init__(self)
        kwargs.pop("name", None)
        vals = dict(d)
        vals.update(dict(zip(arg_names, args)))
        vals.update(kwargs)
        self._kw = vals

    def forward(self, *inputs, **named_inputs):
        return fn(*inputs, **named_inputs, **self._kw)
    return type(name, (Layer,), {"__init__": __init__, "forward": forward})


PairwiseDistance = _fn_layer("PairwiseDistance", F.pairwise_distance, ["p", "epsilon", "keepdim"], (2.0, 1e-6, False))
PixelUnshuffle = _fn_layer("PixelUnshuffle", F.pixel_unshuffle, ["downscale_factor", "data_format"], ("NCHW",))
ChannelShuffle = _fn_layer("ChannelShuffle", F.channel_shuffle, ["groups", "data_format"], ("NCHW",))
Unfold = _fn_layer("Unfold", F.unfold, ["kernel_sizes", "dilations", "paddings", "strides"], (1, 0, 1))
Fold = _fn_layer("Fold", F.fold, ["output_sizes", "kernel_sizes", "dilations", "paddings", "strides"], (1, 0, 1))
AdaptiveMaxPool3D = _fn_layer("AdaptiveMaxPool3D", FX.adaptive_max_pool3d, ["output_size", "return_mask"], (False,))
MaxUnPool1D = _fn_layer("MaxUnPool1D", FX.max_unpool1d, ["kernel_size", "stride", "padding", "data_format", "output_size"],
                        (None, 0, "NCL", None))
MaxUnPool2D = _fn_layer("MaxUnPool2D", FX.max_unpool2d, ["kernel_size", "stride", "padding", "data_format", "output_size"],
                        (None, 0, "NCHW", None))
MaxUnPool3D = _fn_layer("MaxUnPool3D", FX.max_unpool3d, ["kernel_size", "stride", "padding", "data_format", "output_size"],
                        (None, 0, "NCDHW", None))
FractionalMaxPool2D = _fn_layer("FractionalMaxPool2D", FX.fractional_max_pool2d,
                                ["output_size", "kernel_size", "random_u", "return_mask"], (None, None, False))
FractionalMaxPool3D = _fn_layer("FractionalMaxPool3D", FX.fractional_max_pool3d,
                                ["output_size", "kernel_size", "random_u", "return_mask"], (None, None, False))
LPPool1D = _fn_layer("LPPool1D", FX.lp_pool1d, ["norm_type", "kernel_size", "stride", "padding", "ceil_mode", "data_format"],
                     (None, 0, False, "NCL"))
LPPool2D = _fn_layer("LPPool2D", FX.lp_pool2d, ["norm_type", "kernel_size", "stride", "padding", "ceil_mode", "data_format"],
                     (None, 0, False, "NCHW"))
PoissonNLLLoss = _fn_layer("PoissonNLLLoss", FX.poisson_nll_loss, ["log_input", "full", "epsilon", "reduction"],
                           (True, False, 1e-8, "mean"))
MultiLabelSoftMarginLoss = _fn_layer("MultiLabelSoftMarginLoss", FX.multi_label_soft_margin_loss, ["weight", "reduction"],
                                     (None, "mean"))
MultiMarginLoss = _fn_layer("MultiMarginLoss", FX.multi_margin_loss, ["p", "margin", "weight", "reduction"],
                            (1, 1.0, None, "mean"))
SoftMarginLoss = _fn_layer("SoftMarginLoss", FX.soft_margin_loss, ["reduction"], ("mean",))
GaussianNLLLoss = _fn_layer("GaussianNLLLoss", FX.gaussian_nll_loss, ["full", "epsilon", "reduction"], (False, 1e-6, "mean"))
TripletMarginWithDistanceLoss = _fn_layer("TripletMarginWithDistanceLoss", FX.triplet_margin_with_distance_loss,
                                          ["distance_function", "margin", "swap", "reduction"], (None, 1.0, False, "mean"))
RNNTLoss = _fn_layer("RNNTLoss", FX.rnnt_loss, ["blank", "fastemit_lambda", "reduction"], (0, 0.001, "mean"))
FeatureAlphaDropout = None      # defined below (needs the training flag)


class FeatureAlphaDropout(Layer):      # noqa: F811
    def __init__(self, p=0.5, name=None):
        super().__init__()
        self.p = p

    def forward(self, x):
        return FX.feature_alpha_dropout(x, self.p, self.training)


class Softmax2D(Layer):
    def forward(self, x):
        assert x.dim() in (3, 4), "Softmax2D requires a 3D or 4D tensor as input"
        return as_tensor(torch.softmax(_p(x), -3))


class ZeroPad1D(Layer):
    def __init__(self, padding, data_format="NCL", name=None):
        super().__init__()
        self._pad = [padding] * 2 if isinstance(padding, int) else list(padding)

    def forward(self, x):
        return as_tensor(torch.nn.functional.pad(_p(x), self._pad))


class ZeroPad3D(Layer):
    def __init__(self, padding, data_format="NCDHW", name=None):
        super().__init__()
        self._pad = [padding] * 6 if isinstance(padding, int) else list(padding)

    def forward(self, x):
        return as_tensor(torch.nn.functional.pad(_p(x), self._pad))


class Bilinear(Layer):
    def __init__(self, in1_features, in2_features, out_features, weight_attr=None, bias_attr=None, name=None):
        super().__init__()
        self.weight = self.create_parameter([out_features, in1_features, in2_features], attr=weight_attr)
        self.bias = None if bias_attr is False else self.create_parameter([1, out_features], attr=bias_attr, is_bias=True)

    def forward(self, x1, x2):
        return F.bilinear(x1, x2, self.weight, self.bias)


class ParameterDict(Layer):
    def __init__(self, parameters=None):
        super().__init__()
        if parameters is not None:
            self.update(parameters)

    def __getitem__(self, key):
        return self._parameters[key]

    def __setitem__(self, key, p):
        self.add_parameter(key, p)

    def __delitem__(self, key):
        del self._parameters[key]

    def __len__(self):
        return len(self._parameters)

    def __iter__(self):
        return iter(self._parameters)

    def __contains__(self, key):
        return key in self._parameters

    def keys(self):
        return self._parameters.keys()

    def values(self):
        return self._parameters.values()

    def items(self):
        return self._parameters.items()

    def update(self, parameters):
        for k, v in (parameters.items() if hasattr(parameters, "items") else parameters):
            self.add_parameter(k, v)


class HSigmoidLoss(Layer):
    def __init__(self, feature_size, num_classes, weight_attr=None, bias_attr=None, is_custom=False, is_sparse=False, name=None):
        super().__init__()
        self._num_classes, self._custom = num_classes, is_custom
        rows = num_classes if is_custom else num_classes - 1
        self.weight = self.create_parameter([rows, feature_size], attr=weight_attr)
        self.bias = None if bias_attr is False else self.create_parameter([rows, 1], attr=bias_attr, is_bias=True)

    def forward(self, input, label, path_table=None, path_code=None):
        return FX.hsigmoid_loss(input, label, self._num_classes, self.weight, self.bias, path_table, path_code)


class AdaptiveLogSoftmaxWithLoss(Layer):
    def __init__(self, in_features, n_classes, cutoffs, div_value=4.0, head_bias=False, name=None):
        super().__init__()
        self.cutoffs = list(cutoffs) + [n_classes]
        self.n_clusters = len(self.cutoffs) - 1
        self.head_weight = self.create_parameter([in_features, self.cutoffs[0] + self.n_clusters])
        self.head_bias = self.create_parameter([self.cutoffs[0] + self.n_clusters], is_bias=True) if head_bias else None
        self.tail_weights = []
        for i in range(self.n_clusters):
            hsz = max(int(in_features // (div_value ** (i + 1))), 1)
            osz = self.cutoffs[i + 1] - self.cutoffs[i]
            w1, w2 = self.create_parameter([in_features, hsz]), self.create_parameter([hsz, osz])
            self.add_parameter(f"tail_{i}_0", w1), self.add_parameter(f"tail_{i}_1", w2)
            self.tail_weights.append([w1, w2])

    def forward(self, input, label):
        return FX.adaptive_log_softmax_with_loss(input, label, self.head_weight, self.tail_weights, self.cutoffs, self.head_bias)

    def log_prob(self, input):
        """Log-probabilities of all ``n_classes`` classes, [batch, n_classes]: head classes directly, tail classes as
        cluster log-probability plus the log-probability inside the cluster."""
        x = _p(input)
        head = x @ _p(self.head_weight)
        if self.head_bias is not None:
            head = head + _p(self.head_bias)
        head_lp = torch.log_softmax(head, 1)
        short = self.cutoffs[0]
        parts = [head_lp[:, :short]]
        for i, (w1, w2) in enumerate(self.tail_weights):
            lp = torch.log_softmax((x @ _p(w1)) @ _p(w2), 1)
            parts.append(head_lp[:, short + i:short + i + 1] + lp)
        return as_tensor(torch.cat(parts, 1))

    def predict(self, input):
        """The most likely class per row."""
        return as_tensor(torch.argmax(_p(self.log_prob(input)), 1))


class SpectralNorm(Layer):
    """Divides a weight by its largest singular value, estimated with ``power_iters`` power iterations."""

    def __init__(self, weight_shape, dim=0, power_iters=1, epsilon=1e-12, dtype="float32"):
        super().__init__()
        self._dim, self._iters, self._eps = dim, power_iters, epsilon
        h = weight_shape[dim]
        w = int(math.prod(weight_shape)) // h
        self.weight_u = self.create_parameter([h], default_initializer=None)
        self.weight_v = self.create_parameter([w], default_initializer=None)
        with torch.no_grad():
            self.weight_u.normal_(), self.weight_v.normal_()
        self.weight_u.stop_gradient = self.weight_v.stop_gradient = True

    def forward(self, weight):
        w = _p(weight)
        perm = [self._dim] + [i for i in range(w.dim()) if i != self._dim]
        mat = w.permute(perm).reshape(w.shape[self._dim], -1)
        u, v = _p(self.weight_u), _p(self.weight_v)
        with torch.no_grad():
            for _ in range(self._iters):
                v = torch.nn.functional.normalize(mat.t() @ u, dim=0, eps=self._eps)
                u = torch.nn.functional.normalize(mat @ v, dim=0, eps=self._eps)
            self.weight_u.copy_(u), self.weight_v.copy_(v)
        sigma = u @ (mat @ v)
        return as_tensor(w / sigma)


# ------------------------------------------------------------------ RNN cells and wrappers
class RNNCellBase(Layer):
    def get_initial_states(self, batch_ref, shape=None, dtype=None, init_value=0.0, batch_dim_idx=0):
        B = batch_ref.shape[batch_dim_idx]
        shape = shape or self.state_shape
        def make(s):
            return as_tensor(torch.full((B, *s), init_value, dtype=_p(batch_ref).dtype, device=batch_ref.device))
        if isinstance(shape[0], (list, tuple)):
            return tuple(make(s) for s in shape)
        return make(shape)


class _Cell(RNNCellBase):
    _gates = 1

    def __init__(self, input_size, hidden_size, weight_ih_attr=None, weight_hh_attr=None, bias_ih_attr=None,
                 bias_hh_attr=None, name=None, **kw):
        super().__init__()
        std = 1.0 / math.sqrt(hidden_size)
        g = self._gates * hidden_size
        init = Uniform(-std, std)
        self.weight_ih = self.create_parameter([g, input_size], attr=weight_ih_attr, default_initializer=init)
        self.weight_hh = self.create_parameter([g, hidden_size], attr=weight_hh_attr, default_initializer=init)
        self.bias_ih = None if bias_ih_attr is False else self.create_parameter([g], attr=bias_ih_attr, is_bias=True, default_initializer=init)
        self.bias_hh = None if bias_hh_attr is False else self.create_parameter([g], attr=bias_hh_attr, is_bias=True, default_initializer=init)
        self.input_size, self.hidden_size = input_size, hidden_size

    def _lin(self, x, h):
        a = torch.nn.functional.linear(_p(x), _p(self.weight_ih), _p(self.bias_ih))
        b = torch.nn.functional.linear(_p(h), _p(self.weight_hh), _p(self.bias_hh))
        return a, b

    @property
    def state_shape(self):
        return (self.hidden_size,)


class SimpleRNNCell(_Cell):
    def __init__(self, input_size, hidden_size, activation="tanh", **kw):
        super().__init__(input_size, hidden_size, **kw)
        self.activation = activation

    def forward(self, inputs, states=None):
        h = states if states is not None else self.get_initial_states(inputs)
        a, b = self._lin(inputs, h)
        out = torch.tanh(a + b) if self.activation == "tanh" else torch.relu(a + b)
        return as_tensor(out), as_tensor(out)


class LSTMCell(_Cell):
    _gates = 4

    def __init__(self, input_size, hidden_size, weight_ih_attr=None, weight_hh_attr=None, bias_ih_attr=None,
                 bias_hh_attr=None, proj_size=0, name=None):
        super().__init__(input_size, hidden_size, weight_ih_attr, weight_hh_attr, bias_ih_attr, bias_hh_attr)

    def forward(self, inputs, states=None):
        h, c = states if states is not None else self.get_initial_states(inputs)
        a, b = self._lin(inputs, h)
        i, f, g, o = (a + b).chunk(4, -1)
        c2 = torch.sigmoid(f) * _p(c) + torch.sigmoid(i) * torch.tanh(g)
        h2 = torch.sigmoid(o) * torch.tanh(c2)
        return as_tensor(h2), (as_tensor(h2), as_tensor(c2))

    @property
    def state_shape(self):
        return ((self.hidden_size,), (self.hidden_size,))


class GRUCell(_Cell):
    _gates = 3

    def forward(self, inputs, states=None):
        h = states if states is not None else self.get_initial_states(inputs)
        a, b = self._lin(inputs, h)
        ar, az, an = a.chunk(3, -1)
        br, bz, bn = b.chunk(3, -1)
        r, z = torch.sigmoid(ar + br), torch.sigmoid(az + bz)
        n = torch.tanh(an + r * bn)
        h2 = (_p(h) - n) * z + n
        return as_tensor(h2), as_tensor(h2)


class RNN(Layer):
    """Runs a cell over the time dimension (rnn.py ``RNN``)."""

    def __init__(self, cell, is_reverse=False, time_major=False):
        super().__init__()
        self.cell, self.is_reverse, self.time_major = cell, is_reverse, time_major

    def forward(self, inputs, initial_states=None, sequence_length=None, **kwargs):
        x = _p(inputs)
        if not self.time_major:
            x = x.transpose(0, 1)
        T = x.shape[0]
        states = initial_states if initial_states is not None else self.cell.get_initial_states(as_tensor(x[0]))
        steps = range(T - 1, -1, -1) if self.is_reverse else range(T)
        outs = [None] * T
        lens = _p(sequence_length) if sequence_length is not None else None
        for t in steps:
            out, new_states = self.cell(as_tensor(x[t]), states, **kwargs)
            if lens is not None:
                live = (t < lens).to(x.dtype).unsqueeze(-1)
                out = as_tensor(_p(out) * live)
                flat_new = new_states if isinstance(new_states, (tuple, list)) else [new_states]
                flat_old = states if isinstance(states, (tuple, list)) else [states]
                mixed = [as_tensor(_p(n) * live + _p(o) * (1 - live)) for n, o in zip(flat_new, flat_old)]
                new_states = tuple(mixed) if isinstance(new_states, (tuple, list)) else mixed[0]
            states = new_states
            outs[t] = _p(out)
        y = torch.stack(outs, 0)
        if not self.time_major:
            y = y.transpose(0, 1)
        return as_tensor(y), states


class BiRNN(Layer):
    def __init__(self, cell_fw, cell_bw, time_major=False):
        super().__init__()
        self.fw, self.bw = RNN(cell_fw, False, time_major), RNN(cell_bw, True, time_major)

    def forward(self, inputs, initial_states=None, sequence_length=None, **kwargs):
        s_fw, s_bw = initial_states if initial_states is not None else (None, None)
        of, sf = self.fw(inputs, s_fw, sequence_length, **kwargs)
        ob, sb = self.bw(inputs, s_bw, sequence_length, **kwargs)
        return as_tensor(torch.cat([_p(of), _p(ob)], -1)), (sf, sb)


class BeamSearchDecoder:
    """Beam search over a cell (rnn.py ``BeamSearchDecoder``): ``initialize`` / ``step`` / ``finalize`` used by
    :func:`dynamic_decode`."""

    def __init__(self, cell, start_token, end_token, beam_size, embedding_fn=None, output_fn=None):
        self.cell, self.start_token, self.end_token, self.beam_size = cell, start_token, end_token, beam_size
        self.embedding_fn, self.output_fn = embedding_fn, output_fn

    @staticmethod
    def tile_beam_merge_with_batch(x, beam_size):
        t = _p(x)
        return as_tensor(t.unsqueeze(1).expand(t.shape[0], beam_size, *t.shape[1:]).reshape(-1, *t.shape[1:]))

    def _map(self, states, fn):
        if isinstance(states, (tuple, list)):
            return type(states)(self._map(s, fn) for s in states)
        return as_tensor(fn(_p(states)))

    def initialize(self, initial_cell_states):
        ref = initial_cell_states[0] if isinstance(initial_cell_states, (tuple, list)) else initial_cell_states
        B = ref.shape[0]
        self.batch = B
        states = self._map(initial_cell_states, lambda t: t.unsqueeze(1).expand(B, self.beam_size, *t.shape[1:])
                           .reshape(B * self.beam_size, *t.shape[1:]))
        log_probs = torch.zeros(B, self.beam_size)
        log_probs[:, 1:] = -1e9
        ids = torch.full((B, self.beam_size), self.start_token, dtype=torch.long)
        finished = torch.zeros(B, self.beam_size, dtype=torch.bool)
        inputs = self.embedding_fn(as_tensor(ids.reshape(-1))) if self.embedding_fn else as_tensor(ids.reshape(-1))
        return inputs, (states, log_probs, finished, torch.zeros(B, self.beam_size, dtype=torch.long)), finished

    def step(self, time, inputs, states, **kwargs):
        cell_states, log_probs, finished, lengths = states
        out, new_cell = self.cell(inputs, cell_states, **kwargs)
        if self.output_fn is not None:
            out = self.output_fn(out)
        lp = torch.log_softmax(_p(out).float(), -1).reshape(self.batch, self.beam_size, -1)
        V = lp.shape[-1]
        # finished beams may only extend with the end token at no cost
        mask = torch.full((V,), -1e9)
        mask[self.end_token] = 0.0
        lp = torch.where(finished.unsqueeze(-1), mask.expand_as(lp), lp)
        total = (log_probs.unsqueeze(-1) + lp).reshape(self.batch, -1)
        top, idx = total.topk(self.beam_size, -1)
        parent, token = idx // V, idx % V
        gather = (parent + torch.arange(self.batch).unsqueeze(1) * self.beam_size).reshape(-1)
        new_cell = self._map(new_cell, lambda t: t[gather])
        was_finished = finished.gather(1, parent)
        lengths = lengths.gather(1, parent) + (~was_finished).long()
        finished = was_finished | (token == self.end_token)
        inputs = self.embedding_fn(as_tensor(token.reshape(-1))) if self.embedding_fn else as_tensor(token.reshape(-1))
        return (token, parent, top), (new_cell, top, finished, lengths), inputs, finished

    def finalize(self, outputs, final_states, sequence_lengths):
        tokens = torch.stack([o[0] for o in outputs], 0)
        parents = torch.stack([o[1] for o in outputs], 0)
        return FX.gather_tree(as_tensor(tokens), as_tensor(parents)), final_states


def dynamic_decode(decoder, inits=None, max_step_num=None, output_time_major=False, impute_finished=False,
                   is_test=False, return_length=False, **kwargs):
    inputs, states, finished = decoder.initialize(inits)
    outputs, step = [], 0
    # steps 0 .. max_step_num inclusive, as the reference's loop (``step_idx > max_step_num`` ends it)
    while not bool(finished.all()) and (max_step_num is None or step <= max_step_num):
        out, states, inputs, finished = decoder.step(step, inputs, states, **kwargs)
        outputs.append(out)
        step += 1
    ids, final_states = decoder.finalize(outputs, states, states[3])
    if not output_time_major:
        ids = as_tensor(_p(ids).permute(1, 0, 2))
    return (ids, final_states, as_tensor(states[3])) if return_length else (ids, final_states)
