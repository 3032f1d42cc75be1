"""tcgen05 GEMM vs an fp32 PyTorch reference: every operand-layout combination, ragged edges,
bf16 / fp32 / fp32-accumulate epilogues, for both tile schemes (128 x 256 per SM; 256 x 256 per SM pair with
tcgen05 cta_group::2)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["1cta", "2cta"], autouse=True)
def gemm_impl(request):
    from paddle_b200.ops import native
    prev = native.set_gemm_impl(request.param)
    yield request.param
    native.set_gemm_impl(prev)


def _ref(a, b, ta, tb):
    A = a.float().t() if ta else a.float()
    B = b.float().t() if tb else b.float()
    return A @ B


def _mk(M, N, K, ta, tb, dev="cuda"):
    g = torch.Generator(device=dev).manual_seed(M * 7 + N * 3 + K)
    a = torch.randn((K, M) if ta else (M, K), device=dev, generator=g).to(torch.bfloat16)
    b = torch.randn((N, K) if tb else (K, N), device=dev, generator=g).to(torch.bfloat16)
    return a, b


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 776, 200), (1000, 264, 1032), (136, 144, 72)])
def test_gemm_layouts(ta, tb, M, N, K):
    from paddle_b200.ops import _lib, native
    a, b = _mk(M, N, K, ta, tb)
    out = native.gemm(a, b, ta, tb)
    _lib.check_status()
    ref = _ref(a, b, ta, tb)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-2 * scale + 1e-2, f"max err {err} (scale {scale})"


def test_gemm_fp32_out_and_accumulate():
    from paddle_b200.ops import _lib, native
    M, N, K = 512, 768, 1024
    a, b = _mk(M, N, K, True, False)
    ref = _ref(a, b, True, False)
    out = native.gemm(a, b, True, False, out_dtype=torch.float32)
    _lib.check_status()
    assert torch.allclose(out, ref, rtol=1e-3, atol=1e-2)
    acc = torch.full((M, N), 2.0, device="cuda")
    native.gemm(a, b, True, False, out=acc, accumulate=True)
    native.gemm(a, b, True, False, out=acc, accumulate=True)
    _lib.check_status()
    assert torch.allclose(acc, 2.0 + 2 * ref, rtol=1e-3, atol=2e-2)


def test_gemm_large_and_deterministic():
    from paddle_b200.ops import _lib, native
    M, N, K = 4096, 11008, 4096
    a, b = _mk(M, N, K, False, False)
    o1 = native.gemm(a, b)
    o2 = native.gemm(a, b)
    _lib.check_status()
    assert torch.equal(o1, o2)
    ref = a[:256].float() @ b.float()
    assert torch.allclose(o1[:256].float(), ref, rtol=2e-2, atol=1.0)
    ref2 = a[-128:].float() @ b.float()
    assert torch.allclose(o1[-128:].float(), ref2, rtol=2e-2, atol=1.0)


def test_debug_bounds_build_runs_clean():
    """The -DPD_DEBUG_BOUNDS build of the kernels (every TMA / bulk copy checked before it is issued) computes the same
    results and records no violation for GEMM (all layouts, accumulate), attention forward / backward and RMSNorm."""
    import os
    import subprocess
    import sys
    code = r"""
import math, torch
from paddle_b200.ops import _lib, native, attention
assert hasattr(_lib.kernels(), "pd_debug_bounds_read")
torch.manual_seed(0)
a = torch.randn(300, 520, device="cuda").bfloat16(); b = torch.randn(520, 264, device="cuda").bfloat16()
for impl in ("2cta", "1cta"):
    native.set_gemm_impl(impl)
    y = native.gemm(a, b)
    assert (y.float() - a.float() @ b.float()).abs().max() < 0.5
    acc = torch.zeros(520, 264, device="cuda")
    x2 = torch.randn(300, 264, device="cuda").bfloat16()
    native.gemm(a, x2, trans_a=True, out=acc, accumulate=True)
    assert (acc - a.float().t() @ x2.float()).abs().max() < 0.5
q = torch.randn(1, 300, 2, 128, device="cuda").bfloat16().requires_grad_(True)
k = torch.randn(1, 300, 2, 128, device="cuda").bfloat16().requires_grad_(True)
v = torch.randn(1, 300, 2, 128, device="cuda").bfloat16().requires_grad_(True)
o = attention.flash_attn_func(q, k, v, True, 1 / math.sqrt(128))
o.backward(torch.randn_like(o))
w = torch.ones(512, device="cuda").bfloat16()
native.rms_norm_fwd(torch.randn(64, 512, device="cuda").bfloat16(), w, 1e-6)
torch.cuda.synchronize()
_lib.check_status()
assert _lib.debug_bounds_violation() is None
print("CLEAN")
"""
    env = dict(os.environ, PD_DEBUG_BOUNDS="1", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0 and "CLEAN" in p.stdout, p.stdout[-2000:] + p.stderr[-3000:]
