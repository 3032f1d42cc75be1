"""Analytic cost model of transformer training on B200 nodes (the role of
python/paddle/distributed/auto_parallel/static/cost/: ``base_cost.py`` alpha-beta communication costs,
``comp_op_cost.py`` / ``comm_op_cost.py`` per-operator costs, ``estimate_cost.py`` whole-program estimate).

Computation is a roofline over three rates, communication an alpha-beta model over NVLink / NVSwitch; the constants are
the figures measured for this repository's kernels (GEMM, attention, fused all-gather / reduce-scatter GEMMs, HBM copy,
NCCL bus bandwidth).  ``estimate_step_time`` composes them for a decoder-only model under a hybrid-parallel configuration
(dp x mp x pp x sharding, micro-batches, recompute) and is what the auto tuner orders its candidates by."""
from __future__ import annotations

import math
from dataclasses import dataclass, field


@dataclass
class Cluster:
    """Rates of one B200 and of the NVLink domain it sits in.  Defaults: measured in-step rates of this repository
    (GEMM inside a training step, flash attention forward / backward, stream copy), the payload rate the fused
    tensor-parallel kernels reach per GPU, NCCL all-reduce bus bandwidth at large sizes, and the per-launch latency of a
    kernel that synchronises with its peers."""
    gpus_per_node: int = 8
    gemm_flops: float = 1.30e15            # bf16 GEMM rate inside a step (burst 1.64e15, sustained cuBLAS 1.38e15)
    attn_fwd_flops: float = 0.58e15
    attn_bwd_flops: float = 0.53e15
    hbm_bytes: float = 6.5e12
    fused_link_bytes: float = 0.53e12      # per direction, reached inside the all-gather / reduce-scatter GEMMs
    nccl_bus_bytes: float = 0.72e12        # all-reduce bus bandwidth at >= 256 MB
    peer_copy_bytes: float = 0.77e12
    coll_latency: float = 25e-6            # a fused compute + collective launch (peer flags, epoch hand-shake)
    nccl_latency: float = 20e-6            # a small NCCL collective
    internode_bytes: float = 0.05e12       # per GPU between nodes (400 Gb/s class NIC)
    other_fraction: float = 0.15           # norms, rope, swiglu, embeddings, loss, optimizer: share of the GEMM + attention time
    hbm_capacity: float = 180e9


# ------------------------------------------------------------------------------------------------- single operators
def matmul_time(m, n, k, cluster=None, dtype_bytes=2):
    """max(FLOPs / GEMM rate, bytes / HBM rate); small GEMMs lose efficiency as tiles stop filling 148 SMs."""
    c = cluster or Cluster()
    flops = 2.0 * m * n * k
    tiles = math.ceil(m / 256) * math.ceil(n / 256)
    waves = math.ceil(tiles / 74)                                   # 74 CTA pairs of the 2-CTA kernel
    fill = tiles / (waves * 74)
    bytes_ = dtype_bytes * (m * k + k * n + m * n)
    return max(flops / (c.gemm_flops * max(fill, 0.25)), bytes_ / c.hbm_bytes)


def attention_time(batch, seq, heads, head_dim, causal=True, backward=False, cluster=None):
    c = cluster or Cluster()
    flops = 4.0 * batch * heads * seq * seq * head_dim * (0.5 if causal else 1.0)
    if backward:
        return 2.5 * flops / c.attn_bwd_flops
    return flops / c.attn_fwd_flops


def elementwise_time(nbytes, cluster=None):
    return nbytes / (cluster or Cluster()).hbm_bytes


def _bw(n, cluster, fused=False):
    """Payload rate per GPU of a collective over ``n`` ranks.  NCCL's bus bandwidth grows with the rank count on an
    NVSwitch node (about half of the 8-rank figure between two GPUs, three quarters among four)."""
    c = cluster
    if n > c.gpus_per_node:
        return c.internode_bytes
    if fused:
        return c.fused_link_bytes
    scale = {2: 0.51, 4: 0.76, 8: 1.0}
    if n in scale:
        return c.nccl_bus_bytes * scale[n]
    lo = max(k for k in scale if k <= n) if n >= 2 else 2
    hi = min(k for k in scale if k >= n) if n <= 8 else 8
    if lo == hi:
        return c.nccl_bus_bytes * scale[lo]
    f = (math.log2(n) - math.log2(lo)) / (math.log2(hi) - math.log2(lo))
    return c.nccl_bus_bytes * (scale[lo] + f * (scale[hi] - scale[lo]))


def all_gather_time(nbytes_out, n, cluster=None, fused=False):
    """``nbytes_out``: size of the gathered result; every GPU receives (n - 1) / n of it."""
    c = cluster or Cluster()
    if n <= 1:
        return 0.0
    return (n - 1) / n * nbytes_out / _bw(n, c, fused) + (c.coll_latency if fused else c.nccl_latency)


def reduce_scatter_time(nbytes_in, n, cluster=None, fused=False):
    return all_gather_time(nbytes_in, n, cluster, fused)


def all_reduce_time(nbytes, n, cluster=None):
    c = cluster or Cluster()
    if n <= 1:
        return 0.0
    return 2.0 * (n - 1) / n * nbytes / _bw(n, c) + c.nccl_latency


def all_to_all_time(nbytes, n, cluster=None):
    c = cluster or Cluster()
    if n <= 1:
        return 0.0
    return (n - 1) / n * nbytes / _bw(n, c) + c.nccl_latency


def p2p_time(nbytes, cluster=None, internode=False):
    c = cluster or Cluster()
    return nbytes / (c.internode_bytes if internode else c.peer_copy_bytes) + c.nccl_latency


# ------------------------------------------------------------------------------------------------- whole training step
@dataclass
class StepEstimate:
    seconds: float
    tokens_per_second: float
    memory_gb: float
    parts: dict = field(default_factory=dict)

    def fits(self, cluster=None):
        return self.memory_gb * 2 ** 30 <= (cluster or Cluster()).hbm_capacity


def _model_numbers(m):
    h, L, V = m["hidden_size"], m["num_layers"], m["vocab_size"]
    ffn = m.get("intermediate_size", int(8 * h / 3 + 255) // 256 * 256)
    heads = m.get("num_attention_heads", h // 128)
    kv = m.get("num_key_value_heads", heads)
    hd = h // heads
    per_layer = h * (heads + 2 * kv) * hd + h * h + 3 * h * ffn
    return h, L, V, ffn, heads, hd, per_layer, per_layer * L + 2 * V * h


def estimate_step_time(model_cfg, cfg, cluster=None):
    """One optimizer step of a Llama-style decoder.  ``model_cfg``: hidden_size, num_layers, vocab_size, seq_length,
    global_batch_size (sequences) and optionally intermediate_size / num_attention_heads / num_key_value_heads.
    ``cfg``: dp_degree, mp_degree, pp_degree, sharding_degree, sharding_stage, micro_batch_size, use_recompute,
    vpp_degree.  Tensor parallelism is the sequence-parallel form (all-gather in front of the column-parallel GEMMs,
    reduce-scatter behind the row-parallel ones), run by the fused kernels."""
    c = cluster or Cluster()
    h, L, V, ffn, heads, hd, per_layer, params = _model_numbers(model_cfg)
    S = model_cfg.get("seq_length", 4096)
    gbs = cfg.get("global_batch_size") or model_cfg["global_batch_size"]
    dp, mp, pp = cfg.get("dp_degree", 1), cfg.get("mp_degree", 1), cfg.get("pp_degree", 1)
    sh, stage = cfg.get("sharding_degree", 1), cfg.get("sharding_stage", 1)
    mbs, vpp = cfg.get("micro_batch_size", 1), cfg.get("vpp_degree", 1) or 1
    replicas = dp * sh
    n_micro = max(1, gbs // (replicas * mbs))
    tokens_mb = mbs * S
    layers_local = L / pp
    recompute = 1.0 + (1.0 / 3.0 if cfg.get("use_recompute") else 0.0)          # one extra forward
    # --- computation per micro-batch on one GPU
    # decoder layers + the output projection (on the last stage; averaged over the stages of a pipeline)
    gemm_flops = 6.0 * per_layer * tokens_mb / mp * layers_local + 6.0 * V * h * tokens_mb / mp / pp
    rows = tokens_mb
    fill_penalty = 1.0
    if mp > 1:                                                                   # narrower GEMMs fill the SMs less evenly
        cols = min((heads + 2 * model_cfg.get("num_key_value_heads", heads)) * hd, ffn) / mp
        tiles = math.ceil(rows / 256) * math.ceil(cols / 256)
        fill_penalty = (math.ceil(tiles / 74) * 74) / max(tiles, 1)
        fill_penalty = min(fill_penalty, 1.5)
    t_gemm = gemm_flops * recompute / c.gemm_flops * (0.5 + 0.5 * fill_penalty)
    attn_flops_f = 4.0 * mbs * heads / mp * S * S * hd * 0.5 * layers_local
    t_attn = attn_flops_f * (recompute + 0.0) / c.attn_fwd_flops + 2.5 * attn_flops_f / c.attn_bwd_flops
    t_other = c.other_fraction * (t_gemm + t_attn)
    t_compute_mb = t_gemm + t_attn + t_other
    # --- tensor-parallel traffic: 4 collectives forward + 4 backward per layer on [tokens, h] bf16 activations
    t_tp_mb = 0.0
    if mp > 1:
        act = tokens_mb * h * 2.0
        per_coll = (mp - 1) / mp * act / _bw(mp, c, fused=True) + c.coll_latency
        t_tp_mb = 8.0 * recompute * layers_local * per_coll
    # --- pipeline: bubble of 1F1B (interleaving divides it by the number of virtual stages) + boundary transfers
    t_mb = t_compute_mb + t_tp_mb
    bubble = (pp - 1) / vpp * t_mb if pp > 1 else 0.0
    t_pp_p2p = 2.0 * n_micro * p2p_time(tokens_mb * h * 2.0 / (mp if mp > 1 else 1), c) if pp > 1 else 0.0
    # --- data parallel / sharding traffic once per step (gradients in fp32 main_grad buffers)
    p_local = params / (mp * pp)
    t_dp = 0.0
    if replicas > 1:
        if stage >= 3 and sh > 1:
            # parameters gathered for every micro-batch forward and backward, gradients reduce-scattered per micro-batch
            gather = 2.0 * n_micro * all_gather_time(p_local * 2.0, sh, c)
            scatter = n_micro * reduce_scatter_time(p_local * 2.0, sh, c)
            t_dp = 0.9 * (gather + scatter)                                      # a tenth hides behind the GEMMs (prefetch)
        else:
            grad_bytes = p_local * 4.0
            t_dp = 0.25 * all_reduce_time(grad_bytes, replicas, c)               # bucketed, mostly under backward
            if sh > 1:
                t_dp += 0.5 * all_gather_time(p_local * 2.0, sh, c)             # updated shards back to every rank
    # --- optimizer: fp32 master + two moments + bf16 weight, read and written
    opt_elems = p_local / (sh if sh > 1 else 1)
    t_opt = opt_elems * (4 * 3 * 2 + 4 + 2) / c.hbm_bytes
    seconds = n_micro * t_mb + bubble + t_pp_p2p + t_dp + t_opt
    # --- memory per GPU
    w = 2.0 * p_local / (sh if stage >= 3 else 1)
    g = 4.0 * p_local / (sh if stage >= 2 else 1)
    o = 12.0 * p_local / max(sh, 1)
    act_layer = tokens_mb * h * (2.0 if cfg.get("use_recompute") else (10.0 + 24.0 / mp))
    in_flight = min(pp, n_micro) if pp > 1 else 1
    acts = act_layer * layers_local * in_flight + (tokens_mb * h * 34.0 / mp if cfg.get("use_recompute") else 0.0)
    memory_gb = (w + g + o + acts) / 2 ** 30 + 2.0                                # + workspace, communication buffers
    tokens = gbs * S
    return StepEstimate(seconds, tokens / seconds, memory_gb,
                        {"compute": n_micro * t_compute_mb, "tensor_parallel": n_micro * t_tp_mb, "pipeline_bubble": bubble,
                         "pipeline_p2p": t_pp_p2p, "data_parallel": t_dp, "optimizer": t_opt, "micro_batches": n_micro})


def rank_configs(model_cfg, cfgs, cluster=None, memory_limit_gb=None):
    """Configurations that fit, fastest estimated first, each with its ``estimated_step_time`` / ``estimated_tokens_per_second``
    / ``estimated_memory_usage`` filled in."""
    c = cluster or Cluster()
    limit = memory_limit_gb if memory_limit_gb is not None else c.hbm_capacity / 2 ** 30
    out = []
    for cfg in cfgs:
        est = estimate_step_time(model_cfg, cfg, c)
        if est.memory_gb > limit:
            continue
        cfg = dict(cfg)
        cfg.update(estimated_step_time=round(est.seconds, 4), estimated_tokens_per_second=round(est.tokens_per_second, 1),
                   estimated_memory_usage=round(est.memory_gb, 2))
        out.append(cfg)
    out.sort(key=lambda x: x["estimated_step_time"])
    return out
