"""Flash attention kernels vs an fp32 PyTorch reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, causal, scale):
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    if kf.shape[1] != qf.shape[1]:
        rep = qf.shape[1] // kf.shape[1]
        kf, vf = kf.repeat_interleave(rep, 1), vf.repeat_interleave(rep, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        Sq, Sk = s.shape[-2:]
        mask = torch.ones(Sq, Sk, dtype=torch.bool, device=s.device).tril(Sk - Sq)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    return (torch.softmax(s, -1) @ vf).transpose(1, 2), lse


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 1, 1), (2, 256, 2, 2), (1, 384, 4, 2), (1, 200, 2, 1), (1, 1024, 2, 2)])
def test_flash_fwd(causal, B, S, Hq, Hkv):
    from paddle_b200.ops import _lib, attention
    torch.manual_seed(S + Hq)
    q = torch.randn(B, S, Hq, 128, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, 128, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, 128, device="cuda").to(torch.bfloat16)
    scale = 1 / math.sqrt(128)
    o, lse = attention.fwd(q, k, v, causal, scale)
    _lib.check_status()
    ro, rl = _ref(q, k, v, causal, scale)
    assert torch.allclose(lse, rl, rtol=1e-3, atol=2e-3), (lse - rl).abs().max()
    assert torch.allclose(o.float(), ro, rtol=2e-2, atol=2e-2), (o.float() - ro).abs().max()


def test_flash_fwd_packed_qkv_view():
    from paddle_b200.ops import _lib, attention
    torch.manual_seed(0)
    B, S, H = 1, 512, 4
    qkv = torch.randn(B, S, 3 * H, 128, device="cuda").to(torch.bfloat16)
    q, k, v = qkv[:, :, :H], qkv[:, :, H:2 * H], qkv[:, :, 2 * H:]
    o, lse = attention.fwd(q, k, v, True, 0.088)
    _lib.check_status()
    ro, _ = _ref(q, k, v, True, 0.088)
    assert torch.allclose(o.float(), ro, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 1, 1), (1, 256, 2, 2), (2, 384, 2, 1), (1, 200, 1, 1), (1, 1024, 2, 2)])
def test_flash_bwd(causal, B, S, Hq, Hkv):
    from paddle_b200.ops import _lib, attention
    if not hasattr(_lib.kernels(), "pd_flash_attn_bwd"):
        pytest.skip("backward kernel not built")
    torch.manual_seed(S * 3 + Hq)
    q = torch.randn(B, S, Hq, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
    k = torch.randn(B, S, Hkv, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(B, S, Hkv, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
    do = torch.randn(B, S, Hq, 128, device="cuda").to(torch.bfloat16)
    scale = 1 / math.sqrt(128)
    o = attention.flash_attn_func(q, k, v, causal, scale)
    o.backward(do)
    _lib.check_status()
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ro, _ = _ref(qf, kf, vf, causal, scale)
    ro.backward(do.float())
    for name, a, b in (("dq", q.grad, qf.grad), ("dk", k.grad, kf.grad), ("dv", v.grad, vf.grad)):
        err = (a.float() - b).abs().max().item()
        assert err <= 3e-2 * b.abs().max().item() + 2e-2, f"{name}: {err}"


def _dense_from_flashmask(idx, sq, sk, causal):
    from paddle_b200.nn.functional.flash_attention import _flashmask_dense
    return _flashmask_dense(idx, sq, sk, causal, idx.device)


def _masked_ref(q, k, v, masked, scale):
    """fp32 attention with a boolean [B, Hm, Sq, Sk] mask (True = hidden); rows with nothing visible give zeros."""
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    if kf.shape[1] != qf.shape[1]:
        rep = qf.shape[1] // kf.shape[1]
        kf, vf = kf.repeat_interleave(rep, 1), vf.repeat_interleave(rep, 1)
    s = (qf @ kf.transpose(-1, -2) * scale).masked_fill(masked, float("-inf"))
    dead = masked.all(-1, keepdim=True)
    p = torch.softmax(s.masked_fill(dead, 0.0), -1).masked_fill(dead, 0.0)
    return (p @ vf).transpose(1, 2)


def _flashmask_cases(S, device):
    g = torch.Generator(device="cpu").manual_seed(S)
    # causal document mask: three documents of uneven length
    cuts = sorted(torch.randint(1, S, (2,), generator=g).tolist())
    ends = torch.zeros(S, dtype=torch.int32)
    lo = 0
    for hi in cuts + [S]:
        ends[lo:hi] = hi
        lo = hi
    starts = torch.zeros(S, dtype=torch.int32)
    lo = 0
    for hi in cuts + [S]:
        starts[lo:hi] = lo
        lo = hi
    cols = torch.arange(S, dtype=torch.int32)
    yield "causal_document", True, ends.view(1, 1, S, 1)
    yield "causal_blockwise", True, torch.stack([(cols + S // 4).clamp(max=S), (cols + S // 2).clamp(max=S)], -1).view(1, 1, S, 2)
    yield "document", False, torch.stack([ends, starts], -1).view(1, 1, S, 2)
    yield "global_sliding", False, torch.stack([(cols + 40).clamp(max=S), torch.full((S,), S, dtype=torch.int32),
                                               torch.full((S,), 8, dtype=torch.int32), (cols - 40).clamp(min=8)], -1).view(1, 1, S, 4)


@pytest.mark.parametrize("S,Hq,Hkv", [(200, 2, 1), (1024, 4, 2)])
def test_flashmask_fwd_bwd(S, Hq, Hkv):
    """Column-sparse masks inside the flash kernels (forward, backward, whole-tile skipping) against a dense fp32 mask."""
    import paddle_b200 as paddle
    from paddle_b200.ops import _lib
    scale = 1 / math.sqrt(128)
    for name, causal, idx in _flashmask_cases(S, "cuda"):
        idx = idx.cuda()
        torch.manual_seed(S)
        q = torch.randn(2, S, Hq, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
        k = torch.randn(2, S, Hkv, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
        v = torch.randn(2, S, Hkv, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
        do = torch.randn(2, S, Hq, 128, device="cuda").to(torch.bfloat16)
        idx2 = idx.expand(2, 1, S, idx.shape[-1]).contiguous()
        o = paddle.nn.functional.flashmask_attention(q, k, v, idx2, causal=causal)
        o.backward(do)
        _lib.check_status()
        masked = _dense_from_flashmask(idx2, S, S, causal)
        qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
        ro = _masked_ref(qf, kf, vf, masked, scale)
        ro.backward(do.float())
        assert (o.float() - ro).abs().max().item() < 3e-2, name
        for nm, a, b in (("dq", q.grad, qf.grad), ("dk", k.grad, kf.grad), ("dv", v.grad, vf.grad)):
            err = (a.float() - b).abs().max().item()
            assert err <= 3e-2 * b.abs().max().item() + 2e-2, f"{name} {nm}: {err}"


def test_varlen_packed_single_launch():
    """flash_attn_unpadded on a ragged packing runs as one masked launch and equals per-sequence attention."""
    import paddle_b200 as paddle
    from paddle_b200.ops import _lib, native
    lens = [37, 300, 128, 515]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    total, H = sum(lens), 2
    torch.manual_seed(1)
    scale = 1 / math.sqrt(128)
    for causal in (True, False):
        q = torch.randn(total, H, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
        k = torch.randn(total, H, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
        v = torch.randn(total, H, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
        do = torch.randn(total, H, 128, device="cuda").to(torch.bfloat16)
        before = native.LAUNCH_COUNT
        o, _ = paddle.nn.functional.flash_attn_unpadded(q, k, v, cu, cu, max(lens), max(lens), scale, causal=causal)
        assert native.LAUNCH_COUNT - before == 1
        o.backward(do)
        _lib.check_status()
        qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
        outs = []
        for i in range(len(lens)):
            sl = slice(int(cu[i]), int(cu[i + 1]))
            r, _ = _ref(qf[sl].unsqueeze(0), kf[sl].unsqueeze(0), vf[sl].unsqueeze(0), causal, scale)
            outs.append(r.squeeze(0))
        ro = torch.cat(outs, 0)
        ro.backward(do.float())
        assert (o.float() - ro).abs().max().item() < 3e-2
        for nm, a, b in (("dq", q.grad, qf.grad), ("dk", k.grad, kf.grad), ("dv", v.grad, vf.grad)):
            err = (a.float() - b).abs().max().item()
            assert err <= 3e-2 * b.abs().max().item() + 2e-2, f"{nm}: {err}"


def test_flash_long_sequence_bwd():
    """S = 4096, 8 heads, causal: forward and backward against the fp32 reference."""
    from paddle_b200.ops import _lib, attention
    torch.manual_seed(11)
    B, S, H = 1, 4096, 8
    q = torch.randn(B, S, H, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
    k = torch.randn(B, S, H, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(B, S, H, 128, device="cuda").to(torch.bfloat16).requires_grad_(True)
    do = torch.randn(B, S, H, 128, device="cuda").to(torch.bfloat16)
    scale = 1 / math.sqrt(128)
    o = attention.flash_attn_func(q, k, v, True, scale)
    o.backward(do)
    _lib.check_status()
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ro, _ = _ref(qf, kf, vf, True, scale)
    ro.backward(do.float())
    assert (o.float() - ro).abs().max().item() < 3e-2
    for nm, a, b in (("dq", q.grad, qf.grad), ("dk", k.grad, kf.grad), ("dv", v.grad, vf.grad)):
        err = (a.float() - b).abs().max().item()
        assert err <= 3e-2 * b.abs().max().item() + 2e-2, f"{nm}: {err}"
