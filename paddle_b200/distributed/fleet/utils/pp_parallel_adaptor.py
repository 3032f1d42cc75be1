"""Re-partitions pipeline-parallel checkpoints for another pipeline / virtual-pipeline degree
(python/paddle/distributed/fleet/utils/pp_parallel_adaptor.py:82 ``PipeLineModelAdaptor``).

Layout handled: one directory per (mp, sharding, pp) rank, ``<root>/mp_XX_sharding_XX_pp_XX/model.pdparams``, whose keys
are ``<prefix><local layer index>.<parameter>`` for the layers of that stage and ``shared_layers.<name>.<parameter>`` for
tied layers.  With virtual stages a rank holds several chunks; their keys carry ``<chunk>.`` in front of the layer
index (``_layers.<chunk>.<idx>.w``) when ``vpp > 1``.  The adaptor collects the layers of one (mp, sharding) group in
global order, cuts the list into ``pp * vpp`` new segments (``uniform``: equal counts; ``layer``: equal numbers of
transformer blocks, first / last layers free) and writes the new directories.  Optimizer state files are not
re-partitioned (their accumulators follow parameter names and are rebuilt by the first step)."""
from __future__ import annotations

import math
import os
import re

from ....framework.io import load, save

_LAYER_KEY = re.compile(r"^(?P<prefix>(?:[A-Za-z_]\w*\.)*?)(?:(?P<chunk>\d+)\.)?(?P<idx>\d+)\.(?P<rest>.+)$")


class ParallelConfig:
    def __init__(self, mp, pp, vpp=1, sharding=1):
        self.mp, self.pp, self.vpp, self.sharding = mp, pp, vpp, sharding

    def pipe_parallel_group(self, i, j):
        return [(i, j, k) for k in range(self.pp)]


def _dir(root, mp, sharding, pp):
    return os.path.join(root, f"mp_{mp:02d}_sharding_{sharding:02d}_pp_{pp:02d}")


class PipeLineModelAdaptor:
    def __init__(self, src_parallel_config, dst_parallel_config, transformer_layer_num=0, segment_method="layer"):
        assert src_parallel_config.mp == dst_parallel_config.mp, "the tensor-parallel degree cannot change here"
        assert src_parallel_config.sharding == dst_parallel_config.sharding
        self._src, self._dst = src_parallel_config, dst_parallel_config
        self._n_blocks, self._method = transformer_layer_num, segment_method

    # ------------------------------------------------------------------ reading
    def extract_layers(self, stage_dir, vpp):
        """[(chunk, local index, {param: tensor})...] of one rank, shared layers as a separate dict."""
        sd = load(os.path.join(stage_dir, "model.pdparams"))
        layers, shared, prefix = {}, {}, ""
        for k, v in sd.items():
            if "shared_layers." in k:
                shared[k] = v
                continue
            m = _LAYER_KEY.match(k)
            if m is None:
                raise ValueError(f"cannot find a layer index in checkpoint key {k!r}")
            chunk, idx, rest = 0, int(m.group("idx")), m.group("rest")
            if m.group("chunk") is not None:
                if vpp > 1:
                    chunk = int(m.group("chunk"))
                else:                                            # "a.3.4.w" without virtual stages: 3 is the layer
                    idx, rest = int(m.group("chunk")), f"{m.group('idx')}.{m.group('rest')}"
            prefix = m.group("prefix")
            layers.setdefault((chunk, idx), {})[rest] = v
        return layers, shared, prefix

    def collect(self, root, i, j):
        """Layers of the (mp i, sharding j) group in global order: virtual stage ``c * pp + rank`` holds chunk ``c`` of
        ``rank``."""
        cfg, per_vs, shared, prefix = self._src, {}, {}, ""
        for (_, _, k) in cfg.pipe_parallel_group(i, j):
            layers, sh, prefix = self.extract_layers(_dir(root, i, j, k), cfg.vpp)
            shared.update(sh)
            for (c, idx), params in layers.items():
                per_vs.setdefault(c * cfg.pp + k, {})[idx] = params
        ordered = []
        for vs in sorted(per_vs):
            ordered += [per_vs[vs][idx] for idx in sorted(per_vs[vs])]
        return ordered, shared, prefix

    # ------------------------------------------------------------------ cutting
    def segment_layers(self, n_layers, config, method=None):
        method = method or self._method
        stages = config.pp * config.vpp
        if method == "uniform":
            base, extra = divmod(n_layers, stages)
            cuts = [0]
            for s in range(stages):
                cuts.append(cuts[-1] + base + (1 if s >= stages - extra else 0))
            return cuts
        blocks = self._n_blocks or max(n_layers - 2, 0)
        first = 1 if n_layers > blocks else 0               # layers in front of the transformer blocks (embedding)
        if blocks % stages != 0:
            raise ValueError(f"{blocks} transformer layers cannot be cut into {stages} equal stages")
        per = blocks // stages
        cuts = [0] + [first + per * s for s in range(1, stages)] + [n_layers]
        return cuts

    # ------------------------------------------------------------------ writing
    def apply(self, src_model_path, dst_model_path):
        dst = self._dst
        for i in range(self._src.mp):
            for j in range(self._src.sharding):
                layers, shared, prefix = self.collect(src_model_path, i, j)
                cuts = self.segment_layers(len(layers), dst)
                for k in range(dst.pp):
                    out = {}
                    for c in range(dst.vpp):
                        vs = c * dst.pp + k
                        for local, params in enumerate(layers[cuts[vs]:cuts[vs + 1]]):
                            head = f"{prefix}{c}.{local}." if dst.vpp > 1 else f"{prefix}{local}."
                            for name, v in params.items():
                                out[head + name] = v
                    if k in (0, dst.pp - 1):                     # tied layers live on the first and the last stage
                        out.update(shared)
                    d = _dir(dst_model_path, i, j, k)
                    os.makedirs(d, exist_ok=True)
                    save(out, os.path.join(d, "model.pdparams"))

    def peek_model(self, model_dir):
        for i in range(self._src.mp):
            for j in range(self._src.sharding):
                for (_, _, k) in self._src.pipe_parallel_group(i, j):
                    d = _dir(model_dir, i, j, k)
                    print(f"{d}:")
                    for key, v in load(os.path.join(d, "model.pdparams")).items():
                        print(f"\t{key} {list(v.shape)}")


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description="re-partition a pipeline-parallel checkpoint")
    ap.add_argument("--src_path", required=True)
    ap.add_argument("--dst_path", required=True)
    ap.add_argument("--src_mp", type=int, default=1)
    ap.add_argument("--src_pp", type=int, required=True)
    ap.add_argument("--src_vp", type=int, default=1)
    ap.add_argument("--dst_mp", type=int, default=None)
    ap.add_argument("--dst_pp", type=int, required=True)
    ap.add_argument("--dst_vp", type=int, default=1)
    ap.add_argument("--sharding", type=int, default=1)
    ap.add_argument("--method", default="layer", choices=["layer", "uniform"])
    ap.add_argument("--transformer_layer_num", type=int, default=0)
    a = ap.parse_args(argv)
    adaptor = PipeLineModelAdaptor(ParallelConfig(a.src_mp, a.src_pp, a.src_vp, a.sharding),
                                   ParallelConfig(a.dst_mp or a.src_mp, a.dst_pp, a.dst_vp, a.sharding),
                                   a.transformer_layer_num, a.method)
    adaptor.apply(a.src_path, a.dst_path)


if __name__ == "__main__":
    main()
