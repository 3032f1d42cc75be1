"""The allocation-free RMSNorm backward (``pd_rms_norm_bwd_static``), for callers that cannot allocate device
memory themselves (fixed memory plans, allocator-free callbacks): called through its exported C symbol, twice
in a row, and compared with the regular entry point that takes its scratch buffer from the caller.
This file sorts last on purpose: a run that stops at the first failure has then already run everything else."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "paddle_b200", "lib", "libpd_kernels.so")
    if not os.path.exists(path):
        from paddle_b200.ops import build
        build.build_kernels()
    return ctypes.CDLL(path)


def test_static_scratch_matches_regular_entry_twice():
    from paddle_b200.ops import native
    lib = _lib()
    fn = lib.pd_rms_norm_bwd_static
    fn.restype = ctypes.c_int
    torch.manual_seed(0)
    for call, (rows, H) in enumerate([(300, 4096), (77, 1024)]):
        x = torch.randn(rows, H, device="cuda").to(torch.bfloat16)
        dy = torch.randn(rows, H, device="cuda").to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
        inv = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
        ref_dx, ref_dw = native.rms_norm_bwd(dy, x, w, inv)
        dx = torch.empty_like(x)
        dw = torch.empty(H, dtype=torch.float32, device="cuda")
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = fn(ctypes.c_void_p(dy.data_ptr()), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                ctypes.c_int(0), ctypes.c_void_p(inv.data_ptr()), ctypes.c_void_p(dx.data_ptr()), ctypes.c_void_p(0),
                ctypes.c_void_p(dw.data_ptr()), ctypes.c_int(0), ctypes.c_int64(rows), ctypes.c_int(H), stream)
        assert rc == 0, f"call {call}: launcher returned {rc}"
        torch.cuda.synchronize()
        assert torch.equal(dx, ref_dx), f"call {call}: dx differs"
        assert torch.allclose(dw, ref_dw, rtol=2e-2, atol=5e-2), f"call {call}: dw differs"


@pytest.mark.parametrize("w_f32,accumulate,with_add", [(True, False, False), (False, True, False), (False, False, True),
                                                       (True, True, True)])
def test_static_scratch_variants(w_f32, accumulate, with_add):
    """fp32 weights, accumulation into an existing dw and the fused ``dx_add`` input, each against the regular entry
    point (``native.rms_norm_bwd``, itself checked against an fp32 PyTorch reference in test_fused_ops_gpu.py)."""
    from paddle_b200.ops import native
    lib = _lib()
    fn = lib.pd_rms_norm_bwd_static
    fn.restype = ctypes.c_int
    torch.manual_seed(1)
    rows, H = 260, 2048
    x = torch.randn(rows, H, device="cuda").to(torch.bfloat16)
    dy = torch.randn(rows, H, device="cuda").to(torch.bfloat16)
    w = 1 + 0.1 * torch.randn(H, device="cuda")
    w = w if w_f32 else w.to(torch.bfloat16)
    inv = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    add = torch.randn(rows, H, device="cuda").to(torch.bfloat16) if with_add else None
    base = torch.randn(H, device="cuda") if accumulate else None
    ref_dw_out = base.clone() if accumulate else None
    ref_dx, ref_dw = native.rms_norm_bwd(dy, x, w, inv, dx_add=add, dw_out=ref_dw_out)
    dx = torch.empty_like(x)
    dw = base.clone() if accumulate else torch.empty(H, dtype=torch.float32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = fn(ctypes.c_void_p(dy.data_ptr()), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
            ctypes.c_int(1 if w_f32 else 0), ctypes.c_void_p(inv.data_ptr()), ctypes.c_void_p(dx.data_ptr()),
            ctypes.c_void_p(add.data_ptr() if with_add else 0), ctypes.c_void_p(dw.data_ptr()),
            ctypes.c_int(1 if accumulate else 0), ctypes.c_int64(rows), ctypes.c_int(H), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(dx, ref_dx)
    assert torch.allclose(dw, ref_dw, rtol=2e-2, atol=5e-2)


def test_static_scratch_rejects_oversize():
    lib = _lib()
    fn = lib.pd_rms_norm_bwd_static
    fn.restype = ctypes.c_int
    z = ctypes.c_void_p(0)
    rc = fn(z, z, z, ctypes.c_int(0), z, z, z, z, ctypes.c_int(0), ctypes.c_int64(4), ctypes.c_int(16384), z)
    assert rc == -5
    rc = fn(z, z, z, ctypes.c_int(0), z, z, z, z, ctypes.c_int(0), ctypes.c_int64(2 ** 31), ctypes.c_int(1024), z)
    assert rc == -5
