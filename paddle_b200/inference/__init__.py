"""``paddle.inference``: predictor API over captured layers (paddle/fluid/inference/api/analysis_predictor.cc,
python/paddle/inference/__init__.py) plus the paged-KV generation engine used by the fused transformer path."""
from __future__ import annotations

import numpy as np
import torch

from .paged_kv import PagedKVCache  # noqa: F401


class PrecisionType:
    Float32, Half, Int8, Bfloat16 = 0, 1, 2, 3


class PlaceType:
    UNK, CPU, GPU = -1, 0, 1


class Config:
    """Predictor configuration.  ``Config(prog_file, params_file)`` or ``Config(path_prefix)`` names a model saved
    by ``paddle.jit.save``."""

    def __init__(self, *args):
        self._prefix = None
        if len(args) == 1:
            self._prefix = args[0][:-len(".pdmodel")] if args[0].endswith(".pdmodel") else args[0]
        elif len(args) == 2:
            self._prefix = args[0][:-len(".pdmodel")] if args[0].endswith(".pdmodel") else args[0]
        self._use_gpu, self._device_id, self._precision = False, 0, PrecisionType.Float32
        self._cuda_graph = True

    def set_model(self, prog_file, params_file=None):
        self._prefix = prog_file[:-len(".pdmodel")] if prog_file.endswith(".pdmodel") else prog_file

    def model_dir(self):
        return self._prefix

    def enable_use_gpu(self, memory_pool_init_size_mb=100, device_id=0, precision_mode=PrecisionType.Float32):
        self._use_gpu, self._device_id, self._precision = True, device_id, precision_mode

    def disable_gpu(self):
        self._use_gpu = False

    def use_gpu(self):
        return self._use_gpu

    def enable_memory_optim(self, *a):
        pass

    def switch_ir_optim(self, flag=True):
        self._cuda_graph = bool(flag)

    def enable_tensorrt_engine(self, *a, **k):
        raise NotImplementedError("TensorRT sub-graph engines are outside this framework; GPU inference runs on "
                                  "its own kernels and CUDA graphs")

    def disable_glog_info(self):
        pass

    def set_cpu_math_library_num_threads(self, n):
        torch.set_num_threads(int(n))

    def enable_mkldnn(self, *a, **k):
        pass                                   # CPU inference runs on the tensor library's own CPU kernels

    def gpu_device_id(self):
        return self._device_id

    def ir_optim(self):
        return self._cuda_graph

    def summary(self):
        return (f"model: {self._prefix}\nuse_gpu: {self._use_gpu}\ndevice_id: {self._device_id}\n"
                f"precision: {self._precision}\ncuda_graph: {self._cuda_graph}")

    _TOLERATED_PREFIXES = ("enable_", "disable_", "switch_", "set_", "delete_", "exp_", "collect_")

    def __getattr__(self, name):
        # The reference's AnalysisConfig has ~150 tuning switches for its pass pipeline and third-party engines
        # (analysis_config.cc); the ones without a meaning here are accepted and ignored so deployment scripts run.
        if name.startswith(Config._TOLERATED_PREFIXES):
            def ignored(*a, **k):
                return None
            ignored.__name__ = name
            return ignored
        raise AttributeError(name)


class _Handle:
    def __init__(self, name):
        self.name, self._value = name, None

    def reshape(self, shape):
        pass

    def copy_from_cpu(self, arr):
        self._value = np.asarray(arr)

    def copy_to_cpu(self):
        return self._value

    def shape(self):
        return list(self._value.shape) if self._value is not None else []

    def share_external_data(self, t):
        self._value = t


class Predictor:
    def __init__(self, config: Config):
        from .. import jit
        self._config = config
        self._device = torch.device("cuda", config._device_id) if config.use_gpu() and torch.cuda.is_available() \
            else torch.device("cpu")
        self._program = self._load_static_program(config.model_dir())
        if self._program is not None:
            return
        self._layer = jit.load(config.model_dir())
        if self._device.type == "cuda":
            self._layer.to(device=self._device)
        if config._cuda_graph:
            self._fn = jit.to_static(self._layer.forward)
        else:
            self._fn = self._layer.forward
        import inspect
        try:
            sig = inspect.signature(self._layer._inner.forward)
            self._in_names = [p for p in sig.parameters]
        except (TypeError, ValueError):
            self._in_names = ["x"]
        self._inputs = {n: _Handle(n) for n in self._in_names}
        self._outputs = []

    def _load_static_program(self, prefix):
        """Models written by ``static.save_inference_model`` hold a recorded program instead of a pickled layer."""
        from .. import static
        try:
            with open(prefix + ".pdmodel", "rb") as f:
                program = static.deserialize_program(f.read())
        except Exception:
            return None
        static.deserialize_persistables(program, static.load_from_file(prefix + ".pdiparams"))
        if self._device.type == "cuda":
            for slot, t in list(program._captured.items()):
                t.data = t.data.to(self._device)
            for name, (slot, ex) in list(program._placeholders.items()):
                ex.data = ex.data.to(self._device)
        bs = static.BuildStrategy()
        bs.use_cuda_graph = bool(self._config._cuda_graph) and self._device.type == "cuda"
        self._compiled = static.CompiledProgram(program, bs)
        self._in_names = list(program._feed_names)
        self._inputs = {n: _Handle(n) for n in self._in_names}
        self._fetch = []
        for s in program._fetch_slots:
            h = torch.empty(0)
            program._slot_of_id[id(h)] = s
            program._keep.append(h)
            self._fetch.append(h)
        self._outputs = []
        return program

    def _run_program(self, inputs):
        from ..static import graph as g
        feed = {n: (v if isinstance(v, torch.Tensor) else np.asarray(v)) for n, v in zip(self._in_names, inputs)}
        with g.suspend():
            outs = self._compiled._run(feed, self._fetch)
        self._outputs = []
        for i, o in enumerate(outs):
            h = _Handle(f"output_{i}")
            h._value = o.detach().float().cpu().numpy() if o.dtype == torch.bfloat16 else o.detach().cpu().numpy()
            self._outputs.append(h)
        return [h._value for h in self._outputs]

    def get_input_names(self):
        return list(self._in_names)

    def get_input_handle(self, name):
        return self._inputs[name]

    def run(self, inputs=None):
        from .._core.tensor import as_tensor
        if inputs is None:
            inputs = [self._inputs[n]._value for n in self._in_names if self._inputs[n]._value is not None]
        if self._program is not None:
            return self._run_program(inputs)
        tens = [as_tensor(torch.as_tensor(np.asarray(v) if not isinstance(v, torch.Tensor) else v).to(self._device))
                for v in inputs]
        with torch.no_grad():
            out = self._fn(*tens)
        outs = list(out) if isinstance(out, (list, tuple)) else [out]
        self._outputs = []
        for i, o in enumerate(outs):
            h = _Handle(f"output_{i}")
            h._value = o.detach().float().cpu().numpy() if o.dtype == torch.bfloat16 else o.detach().cpu().numpy()
            self._outputs.append(h)
        return [h._value for h in self._outputs]

    def get_output_names(self):
        return [h.name for h in self._outputs] or ["output_0"]

    def get_output_handle(self, name):
        for h in self._outputs:
            if h.name == name:
                return h
        raise KeyError(name)

    def clone(self):
        return Predictor(self._config)


def create_predictor(config: Config) -> Predictor:
    return Predictor(config)


def get_version():
    return "paddle_b200 inference"


import enum as _enum

import numpy as _np


class DataType(_enum.IntEnum):
    FLOAT32 = 0
    INT64 = 1
    INT32 = 2
    UINT8 = 3
    INT8 = 4
    FLOAT16 = 5
    BOOL = 6
    FLOAT64 = 7
    BFLOAT16 = 8


Tensor = _Handle

_DT_BYTES = {DataType.FLOAT32: 4, DataType.INT64: 8, DataType.INT32: 4, DataType.UINT8: 1, DataType.INT8: 1,
             DataType.FLOAT16: 2, DataType.BOOL: 1, DataType.FLOAT64: 8, DataType.BFLOAT16: 2}


def get_num_bytes_of_data_type(dtype):
    return _DT_BYTES[DataType(dtype)]


def get_trt_compile_version():
    return (0, 0, 0)


def get_trt_runtime_version():
    return (0, 0, 0)


def _get_phi_kernel_name(op_name):
    return op_name


def convert_to_mixed_precision(model_file, params_file, mixed_model_file, mixed_params_file, mixed_precision,
                               backend=None, keep_io_types=True, black_list=None, **kwargs):
    """Rewrites a saved inference model with its floating-point parameters cast to ``mixed_precision``."""
    import pickle
    import shutil

    import torch
    target = {PrecisionType.Half: torch.float16, PrecisionType.Bfloat16: torch.bfloat16}.get(mixed_precision, torch.float32)
    shutil.copyfile(model_file, mixed_model_file)
    with open(params_file, "rb") as f:
        state = pickle.load(f)
    skip = set(black_list or ())
    out = {}
    for k, v in state.items():
        a = _np.asarray(v)
        if a.dtype.kind == "f" and k not in skip:
            t = torch.from_numpy(a.astype(_np.float32)).to(target)
            a = t.view(torch.int16).numpy().view(_np.uint16) if target is torch.bfloat16 else t.numpy()
        out[k] = a
    with open(mixed_params_file, "wb") as f:
        pickle.dump(out, f)


class PredictorPool:
    def __init__(self, config, size=1):
        self._preds = [create_predictor(config) for _ in range(max(1, size))]

    def retrieve(self, idx):
        return self._preds[idx]

    retrive = retrieve


class XpuConfig:
    def __init__(self):
        raise RuntimeError("XPU devices are not supported")
