"""Pruning rules of the auto tuner (python/paddle/distributed/auto_tuner/prune.py:30-900).  A rule takes
``(tuner_cfg, cur_cfg, history_cfgs)`` and returns True when the configuration must not be run; rules registered with
``register_prune`` look at the configuration alone, those with ``register_prune_history`` compare it with the trials
that already ran (an out-of-memory trial rules out everything that needs at least as much memory; a successful trial
rules out the same shape with a strictly slower setting)."""
from __future__ import annotations

import logging

from .cost_model import get_mem
from .utils import __SUPPORTED_RECOMPUTE_GRANULARITY__

logger = logging.getLogger("auto_tuner")

_PRUNE_FUNC = []
_PRUNE_HISTORY_FUNC = []


def register_prune(fn):
    _PRUNE_FUNC.append(fn)
    return fn


def register_prune_history(fn):
    _PRUNE_HISTORY_FUNC.append(fn)
    return fn


def log_pruned_info(cur_cfg, pruned_reason, tuner_cfg=None):
    cur_cfg["pruned_reason"] = pruned_reason
    logger.info("pruned %s: %s", {k: cur_cfg.get(k) for k in ("dp_degree", "mp_degree", "pp_degree", "sharding_degree",
                                                            "sharding_stage", "micro_batch_size", "use_recompute")}, pruned_reason)


def same_cfgs_beside(attrs, cur_cfg, history_cfgs=()):
    """Trials that agree with ``cur_cfg`` on every tuned key except ``attrs`` (one name or a list)."""
    attrs = [attrs] if isinstance(attrs, str) else list(attrs)
    skip = set(attrs) | {"job_id", "time", "pruned_reason", "error_info", "max_mem_usage", "has_error", "exec_time"}
    keys = [k for k in ("dp_degree", "mp_degree", "pp_degree", "vpp_degree", "sharding_degree", "sharding_stage",
                        "micro_batch_size", "use_recompute", "recompute_granularity", "global_batch_size") if k not in skip]
    return [h for h in history_cfgs if all(h.get(k) == cur_cfg.get(k) for k in keys if k in cur_cfg or k in h)]


def same_cfgs_beside_sharding_overlap(tuner_cfg, cur_cfg, history_cfgs=()):
    return same_cfgs_beside(["sharding_overlap"], cur_cfg, history_cfgs)


def _cand(tuner_cfg, key):
    c = tuner_cfg.get("candidates") or {}
    return c.get(key)


def _oom(h):
    return h.get("max_mem_usage") == "OOM" or h.get("error_info") == "OOM" or h.get("error") == "OOM"


def _ran_ok(h, tuner_cfg):
    metric = tuner_cfg.get("metric_cfg", {}).get("name", "tokens_per_second")
    return isinstance(h.get(metric), (int, float)) and not h.get("error_info") and not _oom(h)


# ------------------------------------------------------------------------------------------- rules on the configuration
@register_prune
def prune_by_mp(tuner_cfg, cur_cfg, history_cfgs=()):
    """Tensor parallelism must divide the hidden size, the vocabulary and the head count, be one of the candidates and
    stay inside a node."""
    mp = cur_cfg.get("mp_degree")
    if mp is None:
        return False
    m = tuner_cfg.get("model_cfg", {})
    for key in ("hidden_size", "vocab_size", "num_attention_heads"):
        if m.get(key) and m[key] % mp:
            log_pruned_info(cur_cfg, f"{key} {m[key]} is not divisible by mp_degree {mp}")
            return True
    cands = _cand(tuner_cfg, "mp_degree")
    if cands and mp not in cands:
        return True
    per_node = tuner_cfg.get("gpus_per_node") or tuner_cfg["num_gpus"] // max(1, tuner_cfg.get("nodes", 1))
    if mp > per_node:
        log_pruned_info(cur_cfg, f"mp_degree {mp} spans more than one node ({per_node} GPUs)")
        return True
    return False


@register_prune
def prune_by_pp(tuner_cfg, cur_cfg, history_cfgs=()):
    """The layer count must split evenly over the stages; virtual stages need a real pipeline."""
    pp = cur_cfg.get("pp_degree")
    if pp is None:
        return False
    layers = tuner_cfg.get("model_cfg", {}).get("num_layers")
    if layers and layers % pp:
        log_pruned_info(cur_cfg, f"num_layers {layers} is not divisible by pp_degree {pp}")
        return True
    cands = _cand(tuner_cfg, "pp_degree")
    if cands and pp not in cands:
        return True
    if pp == 1 and cur_cfg.get("vpp_degree", 1) not in (None, 1):
        log_pruned_info(cur_cfg, "vpp_degree > 1 without a pipeline")
        return True
    nodes = tuner_cfg.get("nodes", 1)
    if nodes > 1 and tuner_cfg.get("pp_cross_node_only") and pp % nodes and pp != 1:
        return True
    return False


@register_prune
def prune_by_vpp(tuner_cfg, cur_cfg, history_cfgs=()):
    """Every (stage, chunk) pair needs the same number of layers; interleaving needs at least ``pp`` micro-batches."""
    vpp, pp = cur_cfg.get("vpp_degree"), cur_cfg.get("pp_degree", 1)
    if vpp in (None, 1):
        return False
    layers = tuner_cfg.get("model_cfg", {}).get("num_layers")
    if layers and layers % (pp * vpp):
        log_pruned_info(cur_cfg, f"num_layers {layers} is not divisible by pp * vpp = {pp * vpp}")
        return True
    cands = _cand(tuner_cfg, "vpp_degree")
    if cands and vpp not in cands:
        return True
    return False


def _local_batch(tuner_cfg, cur_cfg):
    gbs = cur_cfg.get("global_batch_size") or tuner_cfg.get("model_cfg", {}).get("global_batch_size")
    if gbs is None:
        return None
    ways = cur_cfg.get("dp_degree", 1) * cur_cfg.get("sharding_degree", 1)
    return None if gbs % ways else gbs // ways


@register_prune
def prune_by_mbs(tuner_cfg, cur_cfg, history_cfgs=()):
    """The per-replica batch must be a whole number of micro-batches; a pipeline needs at least ``pp`` of them (a
    multiple of ``pp`` when interleaved)."""
    mbs = cur_cfg.get("micro_batch_size")
    if mbs is None:
        return False
    gbs = cur_cfg.get("global_batch_size") or tuner_cfg.get("model_cfg", {}).get("global_batch_size")
    if gbs is None:
        return False
    local = _local_batch(tuner_cfg, cur_cfg)
    if local is None or local < mbs or local % mbs:
        log_pruned_info(cur_cfg, f"global batch {gbs} does not split into micro-batches of {mbs}")
        return True
    cands = _cand(tuner_cfg, "micro_batch_size")
    if cands and mbs not in cands:
        return True
    acc = local // mbs
    pp = cur_cfg.get("pp_degree", 1)
    if pp > 1 and acc < pp:
        log_pruned_info(cur_cfg, f"{acc} micro-batches cannot fill a {pp}-stage pipeline")
        return True
    if cur_cfg.get("vpp_degree", 1) not in (None, 1) and acc % pp:
        log_pruned_info(cur_cfg, f"interleaved pipeline needs a multiple of {pp} micro-batches, got {acc}")
        return True
    return False


@register_prune
def prune_by_sharding(tuner_cfg, cur_cfg, history_cfgs=()):
    """Stage > 1 without a sharding group is the same run as stage 1; gradient / parameter sharding is not combined
    with a pipeline (each micro-batch would re-gather); degrees and stages must be among the candidates."""
    deg, stage = cur_cfg.get("sharding_degree"), cur_cfg.get("sharding_stage")
    if deg is None:
        return False
    cands = _cand(tuner_cfg, "sharding_degree")
    if cands and deg not in cands:
        return True
    if stage is not None:
        cands = _cand(tuner_cfg, "sharding_stage")
        if cands and stage not in cands:
            return True
        if deg == 1 and stage != (min(cands) if cands else 1):
            log_pruned_info(cur_cfg, "sharding_stage > 1 with sharding_degree 1 duplicates stage 1")
            return True
        if cur_cfg.get("pp_degree", 1) > 1 and stage > 1:
            log_pruned_info(cur_cfg, f"sharding stage {stage} is not combined with pipeline parallelism")
            return True
    return False


@register_prune
def prune_by_recompute(tuner_cfg, cur_cfg, history_cfgs=()):
    """A granularity only means something with recompute on, and must be a supported one."""
    use, gran = cur_cfg.get("use_recompute"), cur_cfg.get("recompute_granularity")
    if use is None:
        return False
    cands = _cand(tuner_cfg, "use_recompute")
    if cands and use not in cands:
        return True
    if gran is not None and gran not in __SUPPORTED_RECOMPUTE_GRANULARITY__:
        log_pruned_info(cur_cfg, f"recompute_granularity {gran} is not supported")
        return True
    cg = _cand(tuner_cfg, "recompute_granularity")
    if not use and gran is not None and cg and gran != cg[0]:
        return True
    return False


@register_prune
def prune_by_num_gpus(tuner_cfg, cur_cfg, history_cfgs=()):
    n = cur_cfg.get("num_gpus", tuner_cfg.get("num_gpus"))
    if n is None:
        return False
    prod = 1
    for k in ("dp_degree", "mp_degree", "pp_degree", "sharding_degree"):
        prod *= cur_cfg.get(k, 1) or 1
    if prod != n:
        log_pruned_info(cur_cfg, f"degrees multiply to {prod}, not to {n} GPUs")
        return True
    return False


@register_prune
def prune_by_memory_estimation(tuner_cfg, cur_cfg, history_cfgs=()):
    """Skip what the closed-form model puts above ``max_mem_usage`` (GB, default the 180 GB of a B200).  A user-supplied
    estimator (``tuner_cfg["memory_estimation_tool"]``, a callable ``(tuner_cfg, cfg) -> GB``) replaces the model."""
    m = tuner_cfg.get("model_cfg", {})
    need = ("num_layers", "hidden_size", "vocab_size")
    if any(k not in m for k in need) or "micro_batch_size" not in cur_cfg:
        return False
    limit = tuner_cfg.get("max_mem_usage", tuner_cfg.get("max_mem_usage_gb", 180.0))
    tool = tuner_cfg.get("memory_estimation_tool")
    if callable(tool):
        est = tool(tuner_cfg, cur_cfg)
    else:
        n = cur_cfg.get("num_gpus", tuner_cfg["num_gpus"])
        if prune_by_num_gpus(tuner_cfg, dict(cur_cfg), ()):
            return True
        est = get_mem(n, cur_cfg, m["num_layers"], m["hidden_size"], m.get("num_attention_heads", m["hidden_size"] // 128),
                      m["vocab_size"], m.get("seq_length", m.get("max_seq_length", 2048)),
                      cur_cfg.get("global_batch_size") or m.get("global_batch_size", 1), m.get("use_flash_attention", True))
    cur_cfg["estimated_memory_usage"] = round(est, 2)
    if est > limit:
        log_pruned_info(cur_cfg, f"estimated {est:.1f} GB exceeds the limit of {limit} GB")
        return True
    return False


@register_prune
def prune_by_invalid_strategy(tuner_cfg, cur_cfg, history_cfgs=()):
    """User-declared exclusions: ``tuner_cfg["invalid_strategy"]`` is a list of patterns such as ``"mp8_pp1"`` or
    ``"sharding2_stage3"``; a configuration matching every ``<name><value>`` token of a pattern is skipped."""
    pats = tuner_cfg.get("invalid_strategy") or []
    short = {"dp": "dp_degree", "mp": "mp_degree", "pp": "pp_degree", "vpp": "vpp_degree", "sharding": "sharding_degree",
             "stage": "sharding_stage", "mbs": "micro_batch_size", "recompute": "use_recompute"}
    import re
    for pat in pats:
        toks = re.findall(r"([a-z]+)(\d+|true|false)", pat.lower())
        if toks and all(short.get(n) in cur_cfg and str(cur_cfg[short[n]]).lower() in (v, {"1": "true", "0": "false"}.get(v, v))
                        for n, v in toks if short.get(n)) and all(short.get(n) for n, _ in toks):
            log_pruned_info(cur_cfg, f"matches invalid_strategy {pat}")
            return True
    return False


# ------------------------------------------------------------------------------------------------ rules on the history
@register_prune_history
def prune_by_mp_pp_history(tuner_cfg, cur_cfg, history_cfgs=(), pruned_cfgs=()):
    """With everything else equal, LESS model splitting needs more memory: if a trial with a larger ``mp * pp`` product
    ran out of memory, so will this one."""
    mppp = cur_cfg.get("mp_degree", 1) * cur_cfg.get("pp_degree", 1)
    for h in same_cfgs_beside(["mp_degree", "pp_degree", "dp_degree"], cur_cfg, history_cfgs):
        if _oom(h) and h.get("mp_degree", 1) * h.get("pp_degree", 1) >= mppp and \
                (h.get("mp_degree", 1), h.get("pp_degree", 1)) != (cur_cfg.get("mp_degree", 1), cur_cfg.get("pp_degree", 1)):
            log_pruned_info(cur_cfg, f"mp*pp = {h.get('mp_degree', 1) * h.get('pp_degree', 1)} already ran out of memory")
            return True
    return False


@register_prune_history
def prune_by_vpp_history(tuner_cfg, cur_cfg, history_cfgs=(), pruned_cfgs=()):
    """More virtual stages keep more activations alive: an out-of-memory trial at a smaller ``vpp`` rules this one out;
    a successful trial at a larger ``vpp`` makes a smaller one (more bubble) pointless only when asked to
    (``prune_slower``)."""
    vpp = cur_cfg.get("vpp_degree")
    if vpp in (None,):
        return False
    for h in same_cfgs_beside("vpp_degree", cur_cfg, history_cfgs):
        hv = h.get("vpp_degree") or 1
        if _oom(h) and hv < vpp:
            log_pruned_info(cur_cfg, f"vpp_degree {hv} already ran out of memory")
            return True
    return False


@register_prune_history
def prune_by_mbs_history(tuner_cfg, cur_cfg, history_cfgs=(), pruned_cfgs=()):
    """A larger micro-batch needs more memory: out of memory at a smaller one rules this one out."""
    mbs = cur_cfg.get("micro_batch_size")
    if mbs is None:
        return False
    for h in same_cfgs_beside("micro_batch_size", cur_cfg, history_cfgs):
        if _oom(h) and h.get("micro_batch_size", 0) <= mbs and h.get("micro_batch_size") != mbs:
            log_pruned_info(cur_cfg, f"micro_batch_size {h['micro_batch_size']} already ran out of memory")
            return True
    return False


@register_prune_history
def prune_by_sharding_history(tuner_cfg, cur_cfg, history_cfgs=(), pruned_cfgs=()):
    """A lower stage keeps more state per GPU (out of memory at a higher stage rules it out); a higher stage
    communicates more (a successful lower stage makes it slower, so it is skipped)."""
    stage = cur_cfg.get("sharding_stage")
    if stage is None:
        return False
    for h in same_cfgs_beside("sharding_stage", cur_cfg, history_cfgs):
        hs = h.get("sharding_stage")
        if hs is None or hs == stage:
            continue
        if _oom(h) and hs > stage:
            log_pruned_info(cur_cfg, f"sharding_stage {hs} already ran out of memory")
            return True
        if _ran_ok(h, tuner_cfg) and hs < stage:
            log_pruned_info(cur_cfg, f"sharding_stage {hs} fits and communicates less")
            return True
    return False


_GRAN_COST = {None: 0, "core_attn": 1, "full_attn": 2, "full": 3}          # more recompute: less memory, slower


@register_prune_history
def prune_by_recompute_history(tuner_cfg, cur_cfg, history_cfgs=(), pruned_cfgs=()):
    """Recompute trades speed for memory: if the shape already ran WITHOUT it (or with a lighter granularity), turning
    it on can only be slower; if it ran out of memory WITH it, turning it off cannot fit."""
    use = cur_cfg.get("use_recompute")
    if use is None:
        return False
    level = (_GRAN_COST.get(cur_cfg.get("recompute_granularity"), 3) or 3) if use else 0
    for h in same_cfgs_beside(["use_recompute", "recompute_granularity"], cur_cfg, history_cfgs):
        hl = (_GRAN_COST.get(h.get("recompute_granularity"), 3) or 3) if h.get("use_recompute") else 0
        if hl == level:
            continue
        if _ran_ok(h, tuner_cfg) and hl < level:
            log_pruned_info(cur_cfg, "the same shape already fits with less recompute")
            return True
        if _oom(h) and hl > level:
            log_pruned_info(cur_cfg, "the same shape ran out of memory with more recompute")
            return True
    return False


@register_prune_history
def prune_by_same_cfg_history(tuner_cfg, cur_cfg, history_cfgs=(), pruned_cfgs=()):
    """Never hand out a configuration twice (a resumed search replays its CSV into the history)."""
    return any(h is not cur_cfg for h in same_cfgs_beside([], cur_cfg, history_cfgs))


def is_pruned(tuner_cfg, cur_cfg, history_cfgs=(), pruned_cfgs=()):
    """Run the configuration rules, then the history rules; True at the first that fires."""
    for fn in _PRUNE_FUNC:
        if fn(tuner_cfg, cur_cfg, history_cfgs):
            return True
    for fn in _PRUNE_HISTORY_FUNC:
        if fn(tuner_cfg, cur_cfg, history_cfgs, pruned_cfgs):
            return True
    return False
