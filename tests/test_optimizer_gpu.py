"""Multi-tensor optimizer kernels vs the AdamW formula evaluated in PyTorch fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _adamw_ref(p, g, m, v, lr, b1, b2, eps, wd, t):
    p = p * (1 - lr * wd)
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    denom = v.sqrt() / (1 - b2 ** t) ** 0.5 + eps
    p = p - (lr / (1 - b1 ** t)) * (m / denom)
    return p, m, v


def test_adamw_multi_and_flat():
    from paddle_b200.ops import native
    torch.manual_seed(0)
    sizes = [5, 4096, 12345, 70001]
    masters = [torch.randn(n, device="cuda") for n in sizes]
    params = [mw.to(torch.bfloat16) for mw in masters]
    grads = [torch.randn(n, device="cuda") for n in sizes]
    ms = [torch.zeros(n, device="cuda") for n in sizes]
    vs = [torch.zeros(n, device="cuda") for n in sizes]
    ref = [(mw.clone(), torch.zeros_like(mw), torch.zeros_like(mw)) for mw in masters]
    tab = native.TensorTable(params, grads, masters, ms, vs)
    lr, b1, b2, eps, wd = 1e-3, 0.9, 0.95, 1e-8, 0.1
    scale = torch.tensor([0.5], device="cuda")
    for t in (1, 2, 3):
        tab.adamw(lr, b1, b2, eps, wd, b1 ** t, b2 ** t, grad_scale=scale)
        ref = [_adamw_ref(p, g * 0.5, m, v, lr, b1, b2, eps, wd, t) for (p, m, v), g in zip(ref, grads)]
    for i in range(len(sizes)):
        assert torch.allclose(masters[i], ref[i][0], rtol=1e-5, atol=1e-6)
        assert torch.allclose(ms[i], ref[i][1], rtol=1e-5, atol=1e-7)
        assert torch.allclose(vs[i], ref[i][2], rtol=1e-5, atol=1e-7)
        assert torch.equal(params[i], masters[i].to(torch.bfloat16))
    # skip flag leaves everything untouched
    snap = masters[1].clone()
    skip = torch.ones(1, dtype=torch.int32, device="cuda")
    tab.adamw(lr, b1, b2, eps, wd, b1 ** 4, b2 ** 4, skip=skip)
    assert torch.equal(snap, masters[1])
    # flat variant
    n = 100003
    mw = torch.randn(n, device="cuda"); p16 = mw.to(torch.bfloat16); g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    r = _adamw_ref(mw.clone(), g, m.clone(), v.clone(), lr, b1, b2, eps, wd, 1)
    native.adamw_flat(p16, mw, g, m, v, lr, b1, b2, eps, wd, b1, b2)
    assert torch.allclose(mw, r[0], rtol=1e-5, atol=1e-6)
    assert torch.equal(p16, mw.to(torch.bfloat16))


def test_l2norm_and_unscale():
    from paddle_b200.ops import native
    torch.manual_seed(1)
    sizes = [7, 5000, 33333]
    grads = [torch.randn(n, device="cuda") for n in sizes]
    grads16 = [g.to(torch.bfloat16) for g in grads]
    tab = native.TensorTable(grads, grads)
    out = tab.sq_l2_norm()
    ref = sum((g.double() ** 2).sum() for g in grads)
    assert abs(out.item() - ref.item()) / ref.item() < 1e-5
    tab16 = native.TensorTable(grads16, grads16)
    out16 = tab16.sq_l2_norm()
    ref16 = sum((g.double() ** 2).sum() for g in grads16)
    assert abs(out16.item() - ref16.item()) / ref16.item() < 1e-5
    found = torch.zeros(1, dtype=torch.int32, device="cuda")
    inv = torch.tensor([0.25], device="cuda")
    before = [g.clone() for g in grads]
    tab.unscale_check(inv, found)
    assert found.item() == 0
    assert all(torch.allclose(g, b * 0.25) for g, b in zip(grads, before))
    grads[1][17] = float("inf")
    tab.unscale_check(inv, found)
    assert found.item() == 1
