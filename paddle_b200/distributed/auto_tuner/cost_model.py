"""Closed-form memory model of a decoder-only transformer under hybrid parallelism
(python/paddle/distributed/auto_tuner/cost_model.py:16-110): parameters, optimizer state and activations per GPU."""
from __future__ import annotations


def all_params(mp, pp, sharding, h, l, V):
    """Bytes of bf16 weights + fp32 gradients, master weights and Adam moments per GPU: 12 h^2 parameters per layer
    (attention 4 h^2 + feed-forward 8 h^2) plus the embedding on the first pipeline stage; master weights and
    moments are divided by the sharding degree (stage 1)."""
    params = l // pp * 12 * h * h / mp + V * h / mp
    return params * (2 + 4) + params * 12 / sharding


def full_recompute_acts(mp, pp, s, b, h, l):
    """Only every layer's input survives the forward pass (2 bytes per element)."""
    return 2 * s * b * h * (l // pp)


def all_acts(mp, pp, s, b, h, l, a, flash=True):
    """All activations of a layer kept for backward: 34 s b h bytes, the tensor-parallel part divided by mp (the usual
    Megatron accounting); the 5 a s^2 b bytes of attention matrices only when attention is NOT the flash kernel, which
    keeps one fp32 log-sum-exp per row instead."""
    per_layer = s * b * h * (10 + 24 / mp) + (4 * a * s * b / mp if flash else 5 * a * s * s * b / mp)
    return per_layer * (l // pp)


def to_gb(nbytes):
    return nbytes / 2 ** 30


def get_mem(total_cards, parallel_cfg, l, h, a, V, s, gbs, flash=True):
    """Estimated GB per GPU of one configuration ``(dp, mp, pp, sharding, micro_batch, recompute)`` - the first
    pipeline stage, which holds ``pp`` micro-batches in flight under 1F1B."""
    dp, mp, pp = parallel_cfg["dp_degree"], parallel_cfg["mp_degree"], parallel_cfg["pp_degree"]
    sharding = parallel_cfg.get("sharding_degree", 1)
    b = parallel_cfg["micro_batch_size"]
    assert dp * mp * pp * sharding == total_cards, "degrees do not multiply to the number of GPUs"
    stage = parallel_cfg.get("sharding_stage", 1)
    params = l // pp * 12 * h * h / mp + V * h / mp
    weights = 2 * params / (sharding if stage >= 3 else 1)
    grads = 4 * params / (sharding if stage >= 2 else 1)
    opt = 12 * params / sharding
    if parallel_cfg.get("use_recompute"):
        acts = full_recompute_acts(mp, pp, s, b, h, l) + all_acts(mp, pp, s, b, h, pp, a, flash) / max(pp, 1)
    else:
        acts = all_acts(mp, pp, s, b, h, l, a, flash)
    in_flight = min(pp, max(1, gbs // (dp * sharding) // b))
    return to_gb(weights + grads + opt + acts * in_flight)


def divisor(num, reverse=False):
    out = [d for d in range(1, num + 1) if num % d == 0]
    return out[::-1] if reverse else out


def get_not_oom_cfgs(cfgs, tuner_cfg):
    """The configurations whose estimate fits ``max_mem_usage`` (GB; default: the 180 GB of a B200)."""
    m = tuner_cfg["model_cfg"]
    limit = tuner_cfg.get("max_mem_usage", 180.0)
    n = tuner_cfg["num_gpus"]
    return [c for c in cfgs if get_mem(n, c, m["num_layers"], m["hidden_size"], m["num_attention_heads"], m["vocab_size"],
                                       m.get("seq_length", m.get("max_seq_length", 2048)), m["global_batch_size"],
                                       m.get("use_flash_attention", True)) <= limit]
