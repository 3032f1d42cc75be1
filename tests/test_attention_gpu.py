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
