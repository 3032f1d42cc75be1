from . import hybrid_parallel_util, mix_precision_utils  # noqa: F401


def __getattr__(name):
    import importlib
    if name in ("sequence_parallel_utils", "tensor_fusion_helper", "timer_helper", "log_util", "fs",
                "tensor_parallel_utils", "pp_parallel_adaptor", "hybrid_parallel_inference"):
        return importlib.import_module(f"{__name__}.{name}")
    if name == "recompute":
        from ..recompute import recompute
        return recompute
    if name in ("LocalFS", "HDFSClient"):
        from . import fs
        return getattr(fs, name)
    raise AttributeError(name)


class DistributedInfer:
    """Inference helper of parameter-server jobs (python/paddle/distributed/fleet/utils/ps_util.py): in a
    collective job the sparse tables are ordinary parameters, so the "distributed" program is the program itself."""

    def __init__(self, main_program=None, startup_program=None):
        from .... import static
        self.origin_main_program = main_program or static.default_main_program()
        self.origin_startup_program = startup_program or static.default_startup_program()
        self.sparse_table_maps = {}

    def init_distributed_infer_env(self, exe, loss, role_maker=None, dirname=None):
        if dirname:
            from .... import static
            static.load(self.origin_main_program, dirname, exe)

    def get_dist_infer_program(self):
        return self.origin_main_program
