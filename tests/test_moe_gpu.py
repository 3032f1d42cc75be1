"""MoE kernels on the GPU against plain fp32 references: router, fp8 block quantisation, grouped block-scaled fp8
GEMM (uneven expert sizes, an empty expert)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_router_topk_softmax():
    from paddle_b200.ops import native
    torch.manual_seed(0)
    T, E, k = 300, 8, 2
    logits = torch.randn(T, E, device="cuda")
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    w, idx = native.moe_topk_softmax(logits, k, True, counts)
    p = torch.softmax(logits, -1)
    rv, ri = p.topk(k, -1)
    assert torch.equal(idx.long(), ri)
    assert (w - rv / rv.sum(-1, keepdim=True)).abs().max() < 1e-5
    assert torch.equal(counts.long(), torch.bincount(ri.reshape(-1), minlength=E))


def test_fp8_quantisation_blocks():
    from paddle_b200.ops import native
    torch.manual_seed(1)
    x = (torch.randn(70, 512, device="cuda") * 3).bfloat16()
    q, s = native.fp8_quant_1x128(x)
    deq = q.float().reshape(70, 4, 128) * s[:, :, None]
    assert (deq.reshape(70, 512) - x.float()).abs().max() <= x.float().abs().max() * 0.07
    assert torch.allclose(s, x.float().reshape(70, 4, 128).abs().amax(-1).clamp(min=1e-12) / 448.0, rtol=1e-5)
    w = (torch.randn(256, 384, device="cuda") * 0.1).bfloat16()
    wq, ws = native.fp8_quant_weight(w)
    assert wq.shape == (384, 256) and ws.shape == (2, 3)
    deq = wq.float().t().reshape(2, 128, 3, 128) * ws[:, None, :, None]
    assert (deq.reshape(256, 384) - w.float()).abs().max() <= w.float().abs().max() * 0.07


@pytest.mark.parametrize("N", [384, 512])        # 128-wide tiles (one epilogue warpgroup) / 256-wide tiles (two)
def test_grouped_gemm_fp8_matches_dequantised_reference(N):
    from paddle_b200.ops import _lib, native
    torch.manual_seed(2)
    E, K = 4, 512
    rows = [200, 0, 77, 300]
    M = sum(rows)
    offs = torch.tensor([0, 200, 200, 277, 577], dtype=torch.int32, device="cuda")
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(E, K, N, device="cuda") * 0.05).bfloat16()
    xq, xs = native.fp8_quant_1x128(x)
    wq, ws = native.fp8_quant_weight(w)
    out = native.grouped_gemm_fp8(xq, xs, wq, ws, offs)
    torch.cuda.synchronize()
    _lib.check_status()
    xd = (xq.float().reshape(M, K // 128, 128) * xs[:, :, None]).reshape(M, K)
    ref = torch.empty(M, N, device="cuda")
    start = 0
    for e, r in enumerate(rows):
        wd = (wq[e].float().t().reshape(K // 128, 128, N // 128, 128) * ws[e][:, None, :, None]).reshape(K, N)
        ref[start:start + r] = xd[start:start + r] @ wd
        start += r
    assert (out.float() - ref).abs().max() / ref.abs().max() < 1e-2
    full = torch.cat([x[s:s + r].float() @ w[e].float() for e, (s, r) in enumerate(zip([0, 200, 200, 277], rows))])
    assert (out.float() - full).abs().max() / full.abs().max() < 0.08      # fp8 quantisation error allowance


def test_fused_moe_fp8_path_close_to_bf16():
    import paddle_b200 as paddle
    from paddle_b200.incubate.nn import functional as IF
    torch.manual_seed(3)
    T, H, F, E = 256, 256, 384, 4
    x = torch.randn(T, H, device="cuda").bfloat16()
    gate_w = torch.randn(H, E, device="cuda").bfloat16()
    w1 = (torch.randn(E, H, 2 * F, device="cuda") * 0.05).bfloat16()
    w2 = (torch.randn(E, F, H, device="cuda") * 0.05).bfloat16()
    gate = x.float() @ gate_w.float()
    permuted, counts, inv, scales, topk = IF.moe_dispatch(paddle.to_tensor(x), paddle.to_tensor(gate), 2)
    ref = IF.moe_ffn(permuted, counts, paddle.to_tensor(w1), paddle.to_tensor(w2))
    q1, s1 = IF.quantize_expert_weights_fp8(w1)
    q2, s2 = IF.quantize_expert_weights_fp8(w2)
    out = IF.moe_ffn_fp8(permuted, counts, q1, s1, q2, s2)
    err = (out.float() - ref.float()).abs().max() / ref.float().abs().max()
    assert err < 0.1, float(err)
    y = IF.moe_reduce(out, scales, inv, topk, norm_topk_prob=True)
    assert y.shape == [T, H]


def test_fp8_grouped_experts_train_step_matches_bf16_experts():
    """The trainable grouped fp8 expert block against per-expert bf16 matmuls with the same weights: output, input
    gradient and both weight gradients (uneven expert sizes, one empty expert); the quantised weights are cached
    across micro-batches and refreshed when the parameters change."""
    import paddle_b200 as paddle
    from paddle_b200.incubate.distributed.models.moe.fp8_experts import FP8GroupedExperts
    torch.manual_seed(5)
    E, H, F = 4, 256, 384
    counts = [200, 0, 33, 331]
    M = sum(counts)
    paddle.seed(5)
    ex = FP8GroupedExperts(E, H, F, initializer_range=0.05).to(device="cuda", dtype="bfloat16")
    x = torch.randn(M, H, device="cuda").bfloat16()
    xt = paddle.to_tensor(x)
    xt.stop_gradient = False
    dy = (torch.randn(M, H, device="cuda") * 0.1).bfloat16()
    y = ex(xt, counts)
    y.backward(dy)
    w1, w2 = ex.gate_up_weight, ex.down_weight
    xr = x.detach().float().requires_grad_(True)
    w1r, w2r = w1.detach().float().requires_grad_(True), w2.detach().float().requires_grad_(True)
    outs, s = [], 0
    for e, n in enumerate(counts):
        if n:
            h = xr[s:s + n] @ w1r[e]
            g, u = h.chunk(2, -1)
            outs.append((torch.nn.functional.silu(g) * u) @ w2r[e])
        s += n
    yr = torch.cat(outs, 0)
    yr.backward(dy.float())

    def rel(a, b):
        return float((a.float() - b).abs().max() / b.abs().max())
    assert rel(y, yr) < 0.08, rel(y, yr)
    assert rel(xt.grad, xr.grad) < 0.1, rel(xt.grad, xr.grad)
    assert rel(w1.grad, w1r.grad) < 0.1, rel(w1.grad, w1r.grad)
    assert rel(w2.grad, w2r.grad) < 0.1, rel(w2.grad, w2r.grad)
    assert float(w1.grad[1].abs().max()) == 0.0                     # the empty expert gets a zero gradient
    # cache: a second micro-batch reuses the e4m3 weights; an in-place update invalidates them
    q_first = ex._cache[1].fwd[0]
    ex(paddle.to_tensor(x), counts)
    assert ex._cache[1].fwd[0] is q_first
    with torch.no_grad():
        w2.mul_(0.5)                                                  # the down projection is linear in its weight
    y2 = ex(paddle.to_tensor(x), counts)
    assert ex._cache[1].fwd[0] is not q_first
    assert rel(y2, yr.detach() * 0.5) < 0.08
