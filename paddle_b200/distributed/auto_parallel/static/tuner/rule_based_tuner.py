"""``RuleBasedTuner`` (python/paddle/distributed/auto_parallel/static/tuner/rule_based_tuner.py)."""
from ..planner import Plan, RuleBasedTuner  # noqa: F401
