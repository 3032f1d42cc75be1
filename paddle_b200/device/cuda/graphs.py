"""CUDA-graph capture and replay (python/paddle/device/cuda/graphs.py ``CUDAGraph`` / ``wrap_cuda_graph``).

Besides wrapping the driver's graph object, ``CUDAGraph`` keeps the fused communication kernels replayable: their
slots' epochs live partly in device memory (a bias the kernels add to their constant arguments) and every replay ends
by advancing that bias, so a captured micro-batch can be replayed any number of times, interleaved with eager
launches on the same slots.  The launch counter used by the benchmarks is advanced by the number of kernels a
replay runs."""
from __future__ import annotations

import contextlib

import torch


def is_cuda_graph_supported():
    return torch.cuda.is_available()


class CUDAGraph:
    def __init__(self, place=None, mode="thread_local", pool=None):
        self._g = torch.cuda.CUDAGraph()
        self._pool = pool
        self._ctx = None
        self._comm = None
        self._launches = 0
        self._launch0 = 0

    def capture_begin(self):
        from ...ops import native
        from ...parallel import fused_linear_impl as FL
        self._comm = FL.GraphCapture()
        self._launch0 = native.LAUNCH_COUNT
        self._ctx = torch.cuda.graph(self._g, pool=self._pool)
        self._ctx.__enter__()

    def capture_end(self):
        from ...ops import native
        try:
            self._comm.end_capture()
        finally:
            ctx, self._ctx = self._ctx, None
            ctx.__exit__(None, None, None)
            self._comm.finish()
            self._launches = native.LAUNCH_COUNT - self._launch0
            native.LAUNCH_COUNT = self._launch0          # capturing launches nothing

    def capture_abort(self, exc_type=None, exc=None, tb=None):
        """Ends a capture that raised: the partial graph is dropped and the slot counters are rolled back."""
        from ...ops import native
        ctx, self._ctx = self._ctx, None
        try:
            if ctx is not None:
                ctx.__exit__(exc_type, exc, tb)
        except Exception:
            pass
        self._comm.finish()
        self._comm._adv = [(0, 0)] * len(self._comm._adv)
        native.LAUNCH_COUNT = self._launch0

    def replay(self):
        from ...ops import native
        self._g.replay()
        self._comm.replayed()
        native.LAUNCH_COUNT += self._launches

    @property
    def launches_per_replay(self):
        return self._launches

    def pool(self):
        return self._g.pool()

    def reset(self):
        self._g.reset()

    def print_to_dot_files(self, dirname, flags=None):
        self._g.enable_debug_mode()
        self._g.debug_dump(str(dirname) + "/graph.dot")


@contextlib.contextmanager
def cuda_graph_capture(graph):
    graph.capture_begin()
    try:
        yield graph
    except BaseException as e:
        graph.capture_abort(type(e), e, e.__traceback__)
        raise
    else:
        graph.capture_end()


def wrap_cuda_graph(function, mode="thread_local", memory_pool="default"):
    """Returns a callable that runs ``function`` from a CUDA graph captured on its first call per input signature
    (inference-style: inputs are copied into static buffers, outputs are the graph's static outputs)."""
    cache = {}

    def flat(args):
        return [a for a in args if isinstance(a, torch.Tensor)]

    def wrapped(*args):
        if not torch.cuda.is_available():
            return function(*args)
        key = tuple((tuple(a.shape), a.dtype) for a in flat(args))
        ent = cache.get(key)
        if ent is None:
            static = [a.detach().clone() if isinstance(a, torch.Tensor) else a for a in args]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                function(*static)
            torch.cuda.current_stream().wait_stream(side)
            g = CUDAGraph()
            with cuda_graph_capture(g):
                out = function(*static)
            ent = cache[key] = (g, static, out)
        g, static, out = ent
        for s, a in zip(static, args):
            if isinstance(a, torch.Tensor):
                s.copy_(a)
        g.replay()
        return out
    return wrapped


def cuda_graph_transform(program):
    """Static programs are replayed from a CUDA graph by ``static.CompiledProgram`` with
    ``BuildStrategy.use_cuda_graph``; there is no program rewriting step."""
    return program
