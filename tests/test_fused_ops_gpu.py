"""Bandwidth-bound fused kernels vs plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def test_rms_norm_fwd_bwd():
    from paddle_b200.ops import native
    torch.manual_seed(0)
    x = torch.randn(37, 4096, device="cuda").to(BF)
    res = torch.randn(37, 4096, device="cuda").to(BF)
    w = (1 + 0.1 * torch.randn(4096, device="cuda")).to(BF)
    y, inv, res_out = native.rms_norm_fwd(x, w, 1e-5, residual=res, want_residual_out=True)
    s = (x.float() + res.float()).to(BF).float()
    r = torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5)
    ref = s * r * w.float()
    assert torch.allclose(res_out.float(), s)
    assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2)
    assert torch.allclose(inv, r.squeeze(-1), rtol=1e-4, atol=1e-5)
    # backward against autograd
    xs = s.clone().requires_grad_(True)
    wf = w.float().clone().requires_grad_(True)
    dy = torch.randn(37, 4096, device="cuda").to(BF)
    (xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-5) * wf).backward(dy.float())
    dx, dw = native.rms_norm_bwd(dy, res_out, w, inv)
    assert torch.allclose(dx.float(), xs.grad, rtol=3e-2, atol=3e-2)
    assert torch.allclose(dw, wf.grad, rtol=2e-2, atol=5e-2)


def test_layer_norm_fwd_bwd():
    from paddle_b200.ops import native
    torch.manual_seed(1)
    x = torch.randn(65, 1024, device="cuda").to(BF)
    w = (1 + 0.1 * torch.randn(1024, device="cuda"))
    b = 0.1 * torch.randn(1024, device="cuda")
    y, mean, rstd = native.layer_norm_fwd(x, w, b, 1e-5)
    xf = x.float().requires_grad_(True)
    wf, bf = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    ref = torch.nn.functional.layer_norm(xf, (1024,), wf, bf, 1e-5)
    assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2)
    dy = torch.randn(65, 1024, device="cuda").to(BF)
    ref.backward(dy.float())
    dx, dw, db = native.layer_norm_bwd(dy, x, w, mean, rstd)
    assert torch.allclose(dx.float(), xf.grad, rtol=3e-2, atol=3e-2)
    assert torch.allclose(dw, wf.grad, rtol=2e-2, atol=5e-2)
    assert torch.allclose(db, bf.grad, rtol=2e-2, atol=5e-2)


@pytest.mark.parametrize("half_style", [True, False])
def test_rope(half_style):
    from paddle_b200.ops import native
    torch.manual_seed(2)
    B, S, H, D = 2, 48, 4, 128
    x = torch.randn(B, S, H, D, device="cuda").to(BF)
    inv_freq = 1.0 / (10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(S, device="cuda").float()[:, None] * inv_freq[None]
    if half_style:
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    else:
        cos, sin = ang.cos().repeat_interleave(2, -1), ang.sin().repeat_interleave(2, -1)
    out = native.rope(x, cos.contiguous(), sin.contiguous(), half_style=half_style)
    xf = x.float()
    if half_style:
        rot = torch.cat([-xf[..., D // 2:], xf[..., :D // 2]], -1)
    else:
        rot = torch.stack([-xf[..., 1::2], xf[..., 0::2]], -1).reshape(xf.shape)
    ref = xf * cos[None, :, None, :] + rot * sin[None, :, None, :]
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    back = native.rope(out, cos.contiguous(), sin.contiguous(), half_style=half_style, backward=True)
    assert torch.allclose(back.float(), xf, rtol=3e-2, atol=3e-2)


def test_swiglu():
    from paddle_b200.ops import native
    torch.manual_seed(3)
    x = torch.randn(33, 2 * 1376, device="cuda").to(BF)
    out = native.swiglu_fwd(x)
    a, b = x.float().chunk(2, -1)
    a.requires_grad_(True); b.requires_grad_(True)
    ref = torch.nn.functional.silu(a) * b
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    do = torch.randn_like(out)
    ref.backward(do.float())
    dx, _ = native.swiglu_bwd(x, None, do)
    assert torch.allclose(dx.float(), torch.cat([a.grad, b.grad], -1), rtol=3e-2, atol=3e-2)
    o2 = native.swiglu_fwd(x[:, :1376].contiguous(), x[:, 1376:].contiguous())
    assert torch.equal(o2, out)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_softmax_ce(dtype):
    from paddle_b200.ops import native
    torch.manual_seed(4)
    T, V = 77, 32000
    logits = (torch.randn(T, V, device="cuda") * 3).to(dtype)
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[5] = -100
    mx, sm, tg, loss = native.ce_stats(logits, labels)
    lf = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, labels, reduction="none", ignore_index=-100)
    assert torch.allclose(loss, ref, rtol=1e-3, atol=1e-3)
    dl = torch.rand(T, device="cuda")
    ref.backward(dl)
    lse = mx + sm.log()
    dlog = native.ce_bwd(logits, labels, lse, dl)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert torch.allclose(dlog.float(), lf.grad, rtol=tol, atol=tol * 0.1)
    # vocab-parallel partial statistics combine to the same loss
    half = V // 2
    parts = [native.ce_stats(logits[:, i * half:(i + 1) * half].contiguous(), labels, vocab_start=i * half,
                             want_loss=False) for i in range(2)]
    gm = torch.maximum(parts[0][0], parts[1][0])
    gs = sum(p[1] * torch.exp(p[0] - gm) for p in parts)
    tgt = parts[0][2] + parts[1][2]
    l2 = torch.where(labels == -100, torch.zeros_like(gm), gs.log() + gm - tgt)
    assert torch.allclose(l2, ref.detach(), rtol=1e-3, atol=1e-3)


def test_embedding():
    from paddle_b200.ops import native
    torch.manual_seed(5)
    V, H = 1000, 256
    table = torch.randn(V, H, device="cuda").to(BF)
    ids = torch.randint(0, V, (4, 37), device="cuda")
    out = native.embedding_fwd(ids, table)
    assert torch.equal(out, table[ids])
    # sharded: rows outside the shard give zeros
    out2 = native.embedding_fwd(ids, table[500:], vocab_start=500)
    ref2 = torch.where((ids >= 500)[..., None], table[ids], torch.zeros_like(out))
    assert torch.equal(out2, ref2)
    dout = torch.randn(4, 37, H, device="cuda").to(BF)
    dt = torch.zeros(V, H, device="cuda")
    native.embedding_bwd(ids, dout, dt)
    ref = torch.zeros(V, H, device="cuda").index_add_(0, ids.reshape(-1), dout.reshape(-1, H).float())
    assert torch.allclose(dt, ref, rtol=1e-4, atol=1e-4)


def test_accumulate_and_add():
    from paddle_b200.ops import native
    a = torch.randn(100003, device="cuda").to(BF)[:100000]
    acc = torch.ones(100000, device="cuda")
    native.accumulate_into_f32(a, acc)
    assert torch.allclose(acc, 1 + a.float())
    b = torch.randn(100000, device="cuda").to(BF)
    assert torch.allclose(native.add_bf16(a.contiguous(), b).float(), (a.float() + b.float()).to(BF).float())


@pytest.mark.parametrize("act", [None, "relu", "gelu", "silu"])
def test_gemm_bias_activation_epilogue(act):
    """act(x @ W + b) from the GEMM epilogue against fp32."""
    import paddle_b200 as paddle
    from paddle_b200.ops import _lib
    torch.manual_seed(3)
    x = (torch.randn(3, 100, 256, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(256, 520, device="cuda") * 0.1).bfloat16()
    b = torch.randn(520, device="cuda").bfloat16()
    with torch.no_grad():
        y = paddle.incubate.nn.functional.fused_linear_activation(x, w, b, activation=act)
    _lib.check_status()
    ref = x.float() @ w.float() + b.float()
    ref = {None: lambda t: t, "relu": torch.relu, "gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu}[act](ref)
    assert (y.float() - ref).abs().max().item() < 3e-2 * ref.abs().max().item() + 2e-2
    # training path: bias in the epilogue, gradients through autograd
    xg, wg, bg = x.clone().requires_grad_(True), w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    out = paddle.nn.functional.linear(xg, wg, bg)
    out.float().pow(2).sum().backward()
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    (xf @ wf + bf).bfloat16().float().pow(2).sum().backward()
    for a, r in ((xg.grad, xf.grad), (wg.grad, wf.grad), (bg.grad, bf.grad)):
        assert (a.float() - r).abs().max().item() < 3e-2 * r.abs().max().item() + 1e-1


def test_gemm_swiglu_epilogue():
    import paddle_b200 as paddle
    from paddle_b200.ops import _lib
    IF = paddle.incubate.nn.functional
    torch.manual_seed(4)
    x = (torch.randn(300, 512, device="cuda") * 0.5).bfloat16()
    gate = (torch.randn(512, 1376, device="cuda") * 0.05).bfloat16()
    up = (torch.randn(512, 1376, device="cuda") * 0.05).bfloat16()
    y = IF.fused_linear_swiglu_interleaved(x, IF.interleave_gate_up(gate, up))
    _lib.check_status()
    ref = torch.nn.functional.silu(x.float() @ gate.float()) * (x.float() @ up.float())
    assert list(y.shape) == [300, 1376]
    assert (y.float() - ref).abs().max().item() < 3e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("act", ["gelu", "relu", "silu", "swiglu", "geglu"])
def test_bias_act_kernel(act):
    import paddle_b200 as paddle
    torch.manual_seed(5)
    x = torch.randn(7, 33, 512, device="cuda").bfloat16()
    b = torch.randn(512, device="cuda").bfloat16()
    with torch.no_grad():
        y = paddle.incubate.nn.functional.fused_bias_act(x, b, act_method=act)
    h = x.float() + b.float()
    if act in ("swiglu", "geglu"):
        g, u = h.chunk(2, -1)
        ref = (torch.nn.functional.silu(g) if act == "swiglu" else torch.nn.functional.gelu(g)) * u
    else:
        ref = getattr(torch.nn.functional, act)(h)
    assert list(y.shape) == list(ref.shape)
    assert (y.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dropout_add_philox(dtype):
    """Keep rate, scaling, reproducibility from (seed, offset), backward mask = forward mask, generator advance."""
    import paddle_b200 as paddle
    from paddle_b200.ops import functional as K
    n, p = 1 << 20, 0.3
    x = torch.ones(n + 5, device="cuda", dtype=dtype).requires_grad_(True)
    y = torch.full((n + 5,), 2.0, device="cuda", dtype=dtype).requires_grad_(True)
    out, (seed, off) = K.dropout_add(x, y, p)
    kept = (out.float() - 2.0) > 0
    assert abs(kept.float().mean().item() - (1 - p)) < 5e-3
    assert torch.allclose(out.float()[kept], torch.tensor(2.0 + 1 / (1 - p), device="cuda"), atol=2e-2)
    out.sum().backward()
    assert torch.equal(x.grad.float() > 0, kept) and torch.all(y.grad.float() == 1)
    out2, _ = K.dropout_add(x.detach(), y.detach(), p, seed_offset=(seed, off))
    assert torch.equal(out2, out.detach())
    out3 = paddle.incubate.nn.functional.fused_dropout_add(x.detach(), y.detach(), p)      # generator moved on
    assert not torch.equal(out3, out.detach())
    paddle.seed(123)
    a = paddle.nn.functional.dropout(x.detach(), p)
    paddle.seed(123)
    b = paddle.nn.functional.dropout(x.detach(), p)
    assert torch.equal(a, b)
