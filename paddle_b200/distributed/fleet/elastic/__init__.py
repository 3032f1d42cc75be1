"""Elastic training driver (python/paddle/distributed/fleet/elastic/__init__.py:51-89)."""
from .manager import ELASTIC_EXIT_CODE, ElasticLevel, ElasticManager, ElasticStatus, LauncherInterface  # noqa: F401


def enable_elastic(args, distribute_mode=None):
    return bool(getattr(args, "elastic_server", None)) and bool(getattr(args, "job_id", None)) and \
        ":" in str(getattr(args, "np", getattr(args, "nnodes", "")))


def launch_elastic(args, distribute_mode=None, kv_client=None):
    """Run the watch loop: (re)launch the trainers whenever membership settles, until completion or error."""
    elastic = ElasticManager(args, kv_client)
    while True:
        elastic.wait()
        elastic.run(args.launcher_cls(args) if hasattr(args, "launcher_cls") else LauncherInterface(args))
        ret = elastic.watch()
        if ret == ElasticStatus.COMPLETED:
            break
        if ret in (ElasticStatus.HOLD, ElasticStatus.RESTART):
            continue
        if ret in (ElasticStatus.ERROR, ElasticStatus.EXIT):
            break
    elastic.exit(completed=ret == ElasticStatus.COMPLETED)
    return ret
