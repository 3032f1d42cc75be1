"""Pipeline layer description and partitioning
(python/paddle/distributed/fleet/meta_parallel/parallel_layers/pp_layers.py: ``LayerDesc`` :57,
``SharedLayerDesc`` :77, ``SegmentLayers`` :93, ``PipelineLayer`` :258).  A model is given as a flat list of
layer descriptions; every pipeline stage builds only its own segment (optionally several virtual chunks).
Weights shared between stages (tied embeddings) are built on each owning stage and their gradients are
all-reduced over the sharing group (:537-575)."""
from __future__ import annotations

import math
import re

import torch

from .....nn.layer.layers import Layer
from .... import collective as C


class LayerDesc:
    def __init__(self, layer_func, *inputs, **kwargs):
        self.layer_func, self.inputs, self.kwargs = layer_func, inputs, kwargs
        if not (isinstance(layer_func, type) and issubclass(layer_func, Layer)):
            raise TypeError("The input(layer_func) should be a derived class of Layer.")

    def build_layer(self):
        return self.layer_func(*self.inputs, **self.kwargs)

    def __repr__(self):
        return f"LayerDesc({self.layer_func.__name__})"


class SharedLayerDesc(LayerDesc):
    def __init__(self, key, layer_func, forward_func=None, shared_weight_attr="weight", *inputs, **kwargs):
        super().__init__(layer_func, *inputs, **kwargs)
        self.layer_name, self.forward_func, self.shared_weight_attr = key, forward_func, shared_weight_attr


class SegmentLayers:
    """Split ``num_items`` layer descriptions into ``num_parts`` contiguous segments: ``uniform`` balances the
    count, ``layer:<regex>`` balances the number of layers whose class name matches."""

    def __init__(self, layers_desc, num_parts, method="uniform", num_virtual_pipeline_stage=None):
        self._layers_desc, self.method, self.num_parts = layers_desc, method, num_parts
        self.num_items = len(layers_desc)
        self.total_parts = num_parts * (num_virtual_pipeline_stage or 1)
        assert self.num_items >= self.total_parts, "layer number should be greater than number of segments"

    def do_segment(self):
        if isinstance(self.method, (list, tuple)):
            seg = list(self.method)
            assert len(seg) == self.total_parts + 1 and seg[0] == 0 and seg[-1] == self.num_items
            return seg
        if self.method == "uniform":
            return self.uniform(self.num_items, self.total_parts)
        if self.method.startswith("layer:"):
            pat = re.compile(self.method.split(":", 1)[1], re.IGNORECASE)
            weights = [1 if (isinstance(d, LayerDesc) and pat.search(d.layer_func.__name__)) or
                       (isinstance(d, Layer) and pat.search(type(d).__name__)) else 0 for d in self._layers_desc]
            total = sum(weights)
            assert total >= self.total_parts, "not enough matching layers for the requested number of stages"
            per = self.uniform(total, self.total_parts)
            result, seen, part = [0], 0, 1
            for i, w in enumerate(weights):
                if w and seen == per[part] and part < self.total_parts:
                    result.append(i)
                    part += 1
                seen += w
            result.append(self.num_items)
            while len(result) < self.total_parts + 1:
                result.insert(-1, result[-2])
            return result
        raise ValueError(f"unknown segment method {self.method}")

    @staticmethod
    def uniform(num_items, num_parts):
        result = [0] * (num_parts + 1)
        part = num_items // num_parts
        extra = num_items % num_parts
        for i in range(1, num_parts + 1):
            result[i] = result[i - 1] + part + (1 if i > num_parts - extra else 0)
        return result


class PipelineLayerChunk(Layer):
    def __init__(self):
        super().__init__()
        self.run_function = []

    def append(self, sublayer):
        if isinstance(sublayer, Layer):
            self.add_sublayer(str(len(self.run_function)), sublayer)
        self.run_function.append(sublayer)

    def forward(self, x):
        for f in self.run_function:
            x = f(*x) if isinstance(x, tuple) else f(x)
        return x


class PipelineLayer(Layer):
    def __init__(self, layers, num_stages=None, topology=None, loss_fn=None, seg_method="uniform", recompute_interval=0,
                 recompute_ctx=None, num_virtual_pipeline_stages=None, virtual_placement="interleaved"):
        super().__init__()
        from ... import fleet
        self._layers_desc = list(layers)
        self._loss_fn = loss_fn
        self._recompute_interval = recompute_interval
        self._num_virtual = num_virtual_pipeline_stages or 1
        assert virtual_placement in ("interleaved", "zigzag")
        self._virtual_placement = virtual_placement
        hcg = fleet.get_hybrid_communicate_group() if topology is None else None
        if hcg is not None:
            self._num_stages = hcg.get_pipe_parallel_world_size()
            self._stage_id = hcg.get_stage_id()
            self._topo = hcg.topology()
            self._hcg = hcg
        else:
            self._topo = topology
            self._num_stages = topology.get_dim("pipe")
            self._stage_id = topology.get_coord(C.get_rank()).pipe
            self._hcg = None
        if num_stages is not None:
            assert num_stages == self._num_stages
        self.segment_parts = SegmentLayers(self._layers_desc, self._num_stages, seg_method, self._num_virtual).do_segment()
        self.shared_layers = {}
        self.shared_weight_attrs = {}
        self.shared_comm = {}
        self._model_chunks = []
        self.run_function = []
        if self._num_virtual > 1:
            for chunk in range(self._num_virtual):
                # interleaved: chunk c of stage r is segment c * P + r; zigzag (zero-bubble V schedules): odd chunks
                # run down the ranks, so with two chunks stage r holds segments r and 2P - 1 - r
                pos = self._stage_id if (virtual_placement == "interleaved" or chunk % 2 == 0) \
                    else self._num_stages - 1 - self._stage_id
                part = chunk * self._num_stages + pos
                lo, hi = self.segment_parts[part], self.segment_parts[part + 1]
                ch = PipelineLayerChunk()
                for f in self._build(lo, hi):
                    ch.append(f)
                self.add_sublayer(f"chunk_{chunk}", ch)
                self._model_chunks.append(ch)
            self._start_pos, self._end_pos = self.segment_parts[self._stage_id], self.segment_parts[self._stage_id + 1]
        else:
            self._start_pos, self._end_pos = self.segment_parts[self._stage_id], self.segment_parts[self._stage_id + 1]
            for i, f in enumerate(self._build(self._start_pos, self._end_pos)):
                if isinstance(f, Layer) and not isinstance(self._layers_desc[self._start_pos + i], SharedLayerDesc):
                    self.add_sublayer(str(self._start_pos + i), f)
                self.run_function.append(f)
        self._build_shared_comm()

    def _build(self, lo, hi):
        fns = []
        for idx in range(lo, hi):
            d = self._layers_desc[idx]
            if isinstance(d, SharedLayerDesc):
                if d.layer_name not in self.shared_layers:
                    self.shared_layers[d.layer_name] = d.build_layer()
                    self.shared_weight_attrs[d.layer_name] = d.shared_weight_attr
                    self.add_sublayer(f"shared_{d.layer_name}", self.shared_layers[d.layer_name])
                layer = self.shared_layers[d.layer_name]
                if d.forward_func is None:
                    fns.append(layer)
                else:
                    fns.append((lambda fwd, l: (lambda *x: fwd(l, *x)))(d.forward_func, layer))
            elif isinstance(d, LayerDesc):
                fns.append(d.build_layer())
            elif isinstance(d, Layer) or callable(d):
                fns.append(d)
            else:
                raise TypeError(f"unsupported layer description {d!r}")
        return fns

    def _build_shared_comm(self):
        """Every rank creates the same groups: for each shared key, the pipeline stages that own a copy."""
        keys = {}
        for idx, d in enumerate(self._layers_desc):
            if isinstance(d, SharedLayerDesc):
                keys.setdefault(d.layer_name, []).append(idx)
        if not keys or self._num_stages == 1 or not C.is_initialized():
            return
        for key, idxs in keys.items():
            stages = sorted({self.get_stage_from_index(i) for i in idxs})
            if len(stages) < 2:
                continue
            pp_lists = self._topo.get_comm_list("pipe")
            for ranks in pp_lists:
                sub = [ranks[s] for s in stages]
                g = C.new_group(sub)
                if C.get_rank() in sub:
                    self.shared_comm[key] = {"group": g, "ranks": sub, "layer": self.shared_layers.get(key),
                                             "weight_attr": self.shared_weight_attrs.get(key)}
        # initial synchronisation: owners start from the first stage's weights
        with torch.no_grad():
            for key, info in self.shared_comm.items():
                w = getattr(info["layer"], info["weight_attr"])
                C.broadcast(w.data, info["ranks"][0], info["group"])

    def allreduce_shared_weight_gradients(self):
        for key, info in self.shared_comm.items():
            w = getattr(info["layer"], info["weight_attr"])
            g = getattr(w, "main_grad", None)
            g = g if g is not None else torch.Tensor.grad.__get__(w)
            if g is not None:
                C.all_reduce(g, group=info["group"])

    def get_stage_from_index(self, layer_idx):
        for part in range(len(self.segment_parts) - 1):
            if self.segment_parts[part] <= layer_idx < self.segment_parts[part + 1]:
                chunk, pos = divmod(part, self._num_stages)
                if self._virtual_placement == "zigzag" and chunk % 2 == 1:
                    return self._num_stages - 1 - pos
                return pos
        raise IndexError(layer_idx)

    def get_num_virtual_stages(self):
        return self._num_virtual

    def get_model_chunks(self):
        return self._model_chunks if self._num_virtual > 1 else None

    def forward_function(self, start, end):
        def run(*x):
            x = x[0] if len(x) == 1 else x
            for f in self.run_function[start:end]:
                x = f(*x) if isinstance(x, tuple) else f(x)
            return x
        return run

    def forward(self, input, chunk_id=None):
        if chunk_id is not None:
            return self._model_chunks[chunk_id](input)
        if self._recompute_interval == 0:
            return self.forward_function(0, len(self.run_function))(*(input if isinstance(input, tuple) else (input,)))
        from ...recompute import recompute
        x = input
        n = len(self.run_function)
        for lo in range(0, n, self._recompute_interval):
            hi = min(lo + self._recompute_interval, n)
            fn = self.forward_function(lo, hi)
            args = x if isinstance(x, tuple) else (x,)
            needs = any(isinstance(a, torch.Tensor) and a.requires_grad for a in args)
            x = recompute(fn, *args) if needs else fn(*args)
        return x

    # ------------------------------------------------------------------ per-layer checkpoint files (:844-937)
    def _ckpt_name(self, idx, mp_rank, chunk=None):
        v = f"-virtual_pp_stage_{chunk:02d}" if chunk is not None else ""
        return f"layer_{idx:02d}{v}-tensor_{mp_rank:02d}-model_states.pdparams"

    def save_state_dict(self, path):
        import os

        from .....framework.io import save
        hcg = self._hcg
        if hcg is not None and hcg.get_data_parallel_rank() != 0:
            return
        mp_rank = hcg.get_model_parallel_rank() if hcg is not None else 0
        os.makedirs(path, exist_ok=True)
        for i, f in enumerate(self.run_function):
            if isinstance(f, Layer):
                save(f.state_dict(), os.path.join(path, self._ckpt_name(self._start_pos + i, mp_rank)))

    def set_state_dir(self, path):
        import os

        from .....framework.io import load
        mp_rank = self._hcg.get_model_parallel_rank() if self._hcg is not None else 0
        for i, f in enumerate(self.run_function):
            if isinstance(f, Layer):
                fn = os.path.join(path, self._ckpt_name(self._start_pos + i, mp_rank))
                if os.path.exists(fn):
                    f.set_state_dict(load(fn))


class PipelineSublayers(Layer):
    """The callables of one pipeline chunk as a Layer: sub-layers are registered under their position so that
    ``state_dict`` keys are ``<index>.<parameter>`` (pp_layers.py:241)."""

    def __init__(self, run_function):
        super().__init__()
        self.run_function = run_function
        for idx, sub in enumerate(run_function):
            if isinstance(sub, Layer):
                self.add_sublayer(str(idx), sub)

    def forward(self, x):
        for f in self.run_function:
            x = f(x)
        return x
