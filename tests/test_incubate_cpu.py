"""incubate: fused functional operators against plain formulas, FusedMultiTransformer prefill/decode consistency
with dense caches, MoE layer against a per-token dense evaluation, routing helpers."""
import math

import numpy as np
import torch

import paddle_b200 as paddle
from paddle_b200 import nn
from paddle_b200.incubate.nn import FusedMultiTransformer
from paddle_b200.incubate.nn import functional as IF


def test_fused_rms_norm_and_layer_norm():
    x, r = paddle.randn([2, 5, 16]), paddle.randn([2, 5, 16])
    w, b = paddle.rand([16]) + 0.5, paddle.randn([16])
    out, res = IF.fused_rms_norm(x, w, None, 1e-6, 2, bias=b, residual=r)
    s = x + b + r
    ref = s * torch.rsqrt((s ** 2).mean(-1, keepdim=True) + 1e-6) * w
    assert np.allclose(out.numpy(), ref.numpy(), atol=1e-5) and np.allclose(res.numpy(), s.numpy(), atol=1e-6)
    out2 = IF.fused_layer_norm(x, w, b, 1e-5, begin_norm_axis=2)
    assert np.allclose(out2.numpy(), torch.nn.functional.layer_norm(x, (16,), w, b, 1e-5).numpy(), atol=1e-5)


def test_swiglu_rope_bias_act():
    x = paddle.randn([3, 8])
    a, b = x[:, :4], x[:, 4:]
    assert np.allclose(IF.swiglu(x).numpy(), (torch.nn.functional.silu(a) * b).numpy(), atol=1e-6)
    assert np.allclose(IF.swiglu(a, b).numpy(), IF.swiglu(x).numpy(), atol=1e-6)
    q = paddle.randn([2, 6, 3, 8])
    qo, ko, vo = IF.fused_rotary_position_embedding(q, q.clone(), None, use_neox_rotary_style=False)
    inv = 1.0 / (10000 ** (torch.arange(0, 8, 2).float() / 8))
    ang = torch.arange(6).float()[:, None] * inv[None]
    cos, sin = torch.cat([ang.cos()] * 2, -1)[None, :, None], torch.cat([ang.sin()] * 2, -1)[None, :, None]
    rot = torch.cat([-q[..., 4:], q[..., :4]], -1)
    assert np.allclose(qo.numpy(), (q * cos + rot * sin).numpy(), atol=1e-5) and vo is None
    assert np.allclose(ko.numpy(), qo.numpy())
    y = IF.fused_bias_act(x, paddle.ones([8]), act_method="relu")
    assert np.allclose(y.numpy(), torch.relu(x + 1).numpy())
    lin = IF.fused_linear_activation(x, paddle.randn([8, 5]), paddle.zeros([5]), activation="gelu")
    assert lin.shape == [3, 5]


def test_masked_multihead_attention_matches_dense():
    torch.manual_seed(0)
    B, H, D, S = 2, 3, 8, 10
    cache = paddle.zeros([2, B, H, S, D])
    hist_k, hist_v = [], []
    for step in range(4):
        x = paddle.randn([B, 3 * H * D])
        out, cache = IF.masked_multihead_attention(x, cache, sequence_lengths=paddle.full([B], step, dtype="int32"))
        q, k, v = x.reshape([B, 3, H, D]).unbind(1)
        hist_k.append(k), hist_v.append(v)
        K_, V_ = torch.stack(hist_k, 2), torch.stack(hist_v, 2)
        s = torch.einsum("bhd,bhsd->bhs", q, K_) / math.sqrt(D)
        ref = torch.einsum("bhs,bhsd->bhd", torch.softmax(s, -1), V_).reshape(B, H * D)
        assert np.allclose(out.numpy(), ref.numpy(), atol=1e-5)


def test_block_attention_prefill_then_decode_equals_full_attention():
    torch.manual_seed(1)
    B, Hq, Hkv, D, bs = 2, 4, 2, 16, 64
    lens = [70, 5]
    kc, vc = paddle.zeros([8, Hkv, bs, D]), paddle.zeros([8, Hkv, bs, D])
    tables = paddle.to_tensor(np.array([[0, 1, 2], [3, 4, 5]], dtype=np.int32))
    qkv = paddle.randn([sum(lens), (Hq + 2 * Hkv) * D])
    enc = paddle.to_tensor(np.array(lens, dtype=np.int32))
    zero = paddle.zeros([B], dtype="int32")
    out, _, kc, vc = IF.block_multihead_attention(qkv, kc, vc, enc, zero, enc, block_tables=tables)
    step = paddle.randn([B, (Hq + 2 * Hkv) * D])
    out2, _, kc, vc = IF.block_multihead_attention(step, kc, vc, zero, enc, paddle.ones([B], dtype="int32"),
                                                   block_tables=tables)
    tok = 0
    for b in range(B):
        rows = torch.cat([qkv[tok:tok + lens[b]], step[b:b + 1]]).reshape(-1, Hq + 2 * Hkv, D)
        tok += lens[b]
        q, k, v = rows[:, :Hq], rows[:, Hq:Hq + Hkv].repeat_interleave(2, 1), rows[:, Hq + Hkv:].repeat_interleave(2, 1)
        s = torch.einsum("hd,shd->hs", q[-1], k) / math.sqrt(D)
        ref = torch.einsum("hs,shd->hd", torch.softmax(s, -1), v).reshape(-1)
        assert np.allclose(out2[b].numpy(), ref.numpy(), atol=1e-5)


def test_fused_multi_transformer_prefill_decode_consistency():
    paddle.seed(2)
    E, H, L, B, S = 32, 4, 2, 2, 6
    fmt = FusedMultiTransformer(E, H, 64, num_layers=L, activation="gelu")
    x = paddle.randn([B, S + 1, E])
    full = fmt(x)                                            # causal full pass over S+1 tokens
    caches = [paddle.zeros([2, B, H, 16, E // H]) for _ in range(L)]
    fmt(x[:, :S], caches=caches)                             # prompt -> caches
    out, _ = fmt(x[:, S:], caches=caches, time_step=paddle.to_tensor([S]))
    assert np.allclose(out[:, 0].detach().numpy(), full[:, S].detach().numpy(), atol=1e-4)
    assert len(fmt.parameters()) == 12 * L


def test_moe_layer_and_routing_helpers():
    from paddle_b200.distributed.models.moe import utils as U
    from paddle_b200.incubate.distributed.models.moe import MoELayer
    paddle.seed(0)

    class Expert(nn.Layer):
        def __init__(self):
            super().__init__()
            self.a, self.b = nn.Linear(16, 32), nn.Linear(32, 16)

        def forward(self, x):
            return self.b(paddle.tanh(self.a(x)))
    experts = nn.LayerList([Expert() for _ in range(4)])
    layer = MoELayer(16, experts, gate={"type": "naive", "top_k": 2})
    x = paddle.randn([3, 5, 16])
    y = layer(x).reshape([-1, 16])
    xf = x.reshape([-1, 16])
    val, idx = layer.gate(xf)
    ref = torch.stack([sum(val[t, k] * experts[int(idx[t, k])](xf[t:t + 1])[0] for k in range(2)) for t in range(15)])
    assert np.allclose(y.detach().numpy(), ref.detach().numpy(), atol=1e-5)
    for kind, k in (("gshard", 2), ("switch", 1)):
        l2 = MoELayer(16, experts, gate={"type": kind, "top_k": k})
        assert l2(x).shape == [3, 5, 16] and float(l2.gate.get_loss()) > 0
    g = paddle.to_tensor(np.array([[0, 1], [1, 2], [1, -1], [3, 1]]))
    assert U._number_count(g, 4).tolist() == [1, 4, 1, 1]
    assert U._assign_pos(g, None).tolist() == [0, 1, 2, 4, 7, 3, 6]
    lim = U._limit_by_capacity(paddle.to_tensor(np.array([3, 1, 2, 2])), paddle.to_tensor(np.array([4, 2])), 2)
    assert lim.tolist() == [3, 1, 1, 1]
    pr = U._prune_gate_by_capacity(paddle.to_tensor(np.array([0, 0, 1, 0, 1])), paddle.to_tensor(np.array([2, 1])), 2, 1)
    assert pr.tolist() == [0, 0, 1, -1, -1]
    out = IF.fused_moe(paddle.randn([4, 8]), paddle.randn([8, 3]), paddle.randn([3, 8, 12]), paddle.randn([3, 6, 8]))
    assert out.shape == [4, 8]


def test_mixtral_tiny_trains_on_cpu():
    from paddle_b200.models.mixtral import MixtralConfig, MixtralForCausalLM
    paddle.seed(0)
    cfg = MixtralConfig.tiny(dtype="float32", hidden_size=64, intermediate_size=64, num_attention_heads=4,
                             num_key_value_heads=2)
    m = MixtralForCausalLM(cfg)
    opt = paddle.optimizer.AdamW(1e-3, parameters=m.parameters())
    ids = paddle.to_tensor(torch.randint(0, 512, (2, 17), generator=torch.Generator().manual_seed(0)).numpy())
    losses = []
    for _ in range(3):
        loss = m(ids[:, :-1], ids[:, 1:])
        loss.backward(), opt.step(), opt.clear_grad()
        losses.append(float(loss))
    assert losses[-1] < losses[0] and all(np.isfinite(losses))
    assert all(getattr(p, "is_moe_param", False) for p in m.layers[0].moe.experts.parameters())


def test_mixtral_grouped_experts_equal_per_expert_layers():
    """``expert_impl="grouped_fp8"`` stacks the experts' weights; off the GPU it computes plain per-expert products, so
    loss and gradients equal those of the per-expert Linear layers holding the same weights."""
    import torch
    import paddle_b200 as paddle
    from paddle_b200.models.mixtral import MixtralConfig, MixtralForCausalLM
    paddle.seed(0)
    grouped = MixtralForCausalLM(MixtralConfig.tiny(dtype="float32", expert_impl="grouped_fp8"))
    paddle.seed(0)
    loop = MixtralForCausalLM(MixtralConfig.tiny(dtype="float32"))
    named = dict(loop.named_parameters())
    with torch.no_grad():
        for lg, ll in zip(grouped.layers, loop.layers):
            for e, ex in enumerate(ll.moe.experts):
                ex.gate_up_proj.weight.copy_(lg.moe.experts.gate_up_weight[e])
                ex.down_proj.weight.copy_(lg.moe.experts.down_weight[e])
        for k, p in grouped.named_parameters():
            if "experts" not in k:
                named[k].copy_(p)
    ids = paddle.to_tensor(torch.randint(0, 512, (2, 16), generator=torch.Generator().manual_seed(1)).numpy())
    a, b = grouped(ids, ids), loop(ids, ids)
    a.backward(); b.backward()
    assert abs(float(a) - float(b)) < 1e-6
    lg, ll = grouped.layers[0], loop.layers[0]
    for e, ex in enumerate(ll.moe.experts):
        assert torch.allclose(lg.moe.experts.gate_up_weight.grad[e], ex.gate_up_proj.weight.grad, atol=1e-6)
        assert torch.allclose(lg.moe.experts.down_weight.grad[e], ex.down_proj.weight.grad, atol=1e-6)
    assert all(getattr(p, "is_moe_param", False) for p in lg.moe.experts.parameters())
