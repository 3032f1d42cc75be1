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
