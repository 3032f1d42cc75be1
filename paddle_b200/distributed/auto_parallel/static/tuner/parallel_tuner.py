"""``ParallelTuner`` (python/paddle/distributed/auto_parallel/static/tuner/parallel_tuner.py)."""
from ..planner import ParallelTuner, Plan  # noqa: F401
