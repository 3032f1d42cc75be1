"""Plan search under the reference's module path (python/paddle/distributed/auto_parallel/static/tuner/)."""
from ..planner import ParallelTuner, Plan, Planner, RuleBasedTuner  # noqa: F401
