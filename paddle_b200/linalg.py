"""``paddle.linalg`` namespace (python/paddle/linalg.py): re-exports of the tensor linear-algebra functions plus
decompositions expressed with torch.linalg under Paddle's names and return conventions."""
from __future__ import annotations

import torch

from ._core.tensor import as_tensor
from .tensor.linalg import *  # noqa: F401,F403
from .tensor import linalg as _tl


def _wrap(fn):
    def f(*a, name=None, **k):
        out = fn(*a, **k)
        if isinstance(out, tuple):
            return tuple(as_tensor(o) if isinstance(o, torch.Tensor) else o for o in out)
        return as_tensor(out) if isinstance(out, torch.Tensor) else out
    return f


def _missing(name, impl):
    if not hasattr(_tl, name):
        globals()[name] = impl


_missing("cholesky", lambda x, upper=False, name=None: as_tensor(torch.linalg.cholesky(x, upper=upper)))
_missing("cholesky_solve", lambda x, y, upper=False, name=None: as_tensor(torch.cholesky_solve(x, y, upper=upper)))
_missing("cholesky_inverse", lambda x, upper=False, name=None: as_tensor(torch.cholesky_inverse(x, upper=upper)))
_missing("inv", _wrap(torch.linalg.inv))
_missing("pinv", lambda x, rcond=1e-15, hermitian=False, name=None: as_tensor(torch.linalg.pinv(x, rtol=rcond, hermitian=hermitian)))
_missing("det", _wrap(torch.linalg.det))
_missing("slogdet", lambda x, name=None: as_tensor(torch.stack(list(torch.linalg.slogdet(x)))))
_missing("eig", _wrap(torch.linalg.eig))
_missing("eigh", lambda x, UPLO="L", name=None: tuple(as_tensor(t) for t in torch.linalg.eigh(x, UPLO=UPLO)))
_missing("eigvals", _wrap(torch.linalg.eigvals))
_missing("eigvalsh", lambda x, UPLO="L", name=None: as_tensor(torch.linalg.eigvalsh(x, UPLO=UPLO)))
_missing("svd", lambda x, full_matrices=False, name=None: tuple(as_tensor(t) for t in torch.linalg.svd(x, full_matrices=full_matrices)))
_missing("svdvals", _wrap(torch.linalg.svdvals))
_missing("qr", lambda x, mode="reduced", name=None: tuple(as_tensor(t) for t in torch.linalg.qr(x, mode=mode)))
_missing("lu", lambda x, pivot=True, get_infos=False, name=None: _lu(x, pivot, get_infos))
_missing("lu_unpack", lambda x, y, unpack_ludata=True, unpack_pivots=True, name=None:
         tuple(as_tensor(t) for t in torch.lu_unpack(x, y.to(torch.int32), unpack_ludata, unpack_pivots)))
_missing("lu_solve", lambda b, lu, pivots, trans="N", name=None: as_tensor(torch.linalg.lu_solve(lu, pivots.to(torch.int32), b, adjoint=trans != "N")))
_missing("solve", lambda x, y, left=True, name=None: as_tensor(torch.linalg.solve(x, y, left=left)))
_missing("triangular_solve", lambda x, y, upper=True, transpose=False, unitriangular=False, name=None:
         as_tensor(torch.linalg.solve_triangular(x.transpose(-1, -2) if transpose else x, y,
                                                 upper=(upper != transpose), unitriangular=unitriangular)))
_missing("lstsq", lambda x, y, rcond=None, driver=None, name=None: _lstsq(x, y, rcond, driver))
_missing("matrix_power", lambda x, n, name=None: as_tensor(torch.linalg.matrix_power(x, n)))
_missing("matrix_rank", lambda x, tol=None, hermitian=False, atol=None, rtol=None, name=None:
         as_tensor(torch.linalg.matrix_rank(x, tol=tol, hermitian=hermitian) if tol is not None else
                   torch.linalg.matrix_rank(x, atol=atol, rtol=rtol, hermitian=hermitian)))
_missing("matrix_exp", _wrap(torch.linalg.matrix_exp))
_missing("matrix_norm", lambda x, p="fro", axis=(-2, -1), keepdim=False, name=None: as_tensor(torch.linalg.matrix_norm(x, p, axis, keepdim)))
_missing("vector_norm", lambda x, p=2.0, axis=None, keepdim=False, name=None: as_tensor(torch.linalg.vector_norm(x, p, axis, keepdim)))
_missing("cond", lambda x, p=None, name=None: as_tensor(torch.linalg.cond(x, p)))
_missing("multi_dot", lambda x, name=None: as_tensor(torch.linalg.multi_dot(list(x))))
_missing("householder_product", lambda x, tau, name=None: as_tensor(torch.linalg.householder_product(x, tau)))
_missing("corrcoef", lambda x, rowvar=True, name=None: as_tensor(torch.corrcoef(x if rowvar else x.t())))
_missing("cov", lambda x, rowvar=True, ddof=True, fweights=None, aweights=None, name=None:
         as_tensor(torch.cov(x if rowvar else x.t(), correction=int(ddof), fweights=fweights, aweights=aweights)))
_missing("pca_lowrank", lambda x, q=None, center=True, niter=2, name=None: tuple(as_tensor(t) for t in torch.pca_lowrank(x, q, center, niter)))
_missing("svd_lowrank", lambda x, q=6, niter=2, M=None, name=None: tuple(as_tensor(t) for t in torch.svd_lowrank(x, q, niter, M)))
_missing("ormqr", lambda x, tau, other, left=True, transpose=False, name=None: as_tensor(torch.ormqr(x, tau, other, left, transpose)))
_missing("cdist", lambda x, y, p=2.0, compute_mode="use_mm_for_euclid_dist_if_necessary", name=None: as_tensor(torch.cdist(x, y, p)))


def _lu(x, pivot, get_infos):
    LU, piv, info = torch.linalg.lu_factor_ex(x, pivot=pivot)
    out = (as_tensor(LU), as_tensor(piv))
    return out + (as_tensor(info),) if get_infos else out


def _lstsq(x, y, rcond, driver):
    r = torch.linalg.lstsq(x, y, rcond=rcond, driver=driver)
    return as_tensor(r.solution), as_tensor(r.residuals), as_tensor(r.rank), as_tensor(r.singular_values)


def vecdot(x, y, axis=-1, name=None):
    return as_tensor(torch.linalg.vecdot(x.as_subclass(torch.Tensor), y.as_subclass(torch.Tensor), dim=axis))


def matrix_transpose(x, name=None):
    return as_tensor(x.as_subclass(torch.Tensor).transpose(-1, -2))


def diagonal(x, offset=0, axis1=0, axis2=1, name=None):
    return as_tensor(torch.diagonal(x.as_subclass(torch.Tensor), offset, axis1, axis2))


def fp8_fp8_half_gemm_fused(x, y, transpose_x=False, transpose_y=False, bias=None, scale=1.0, output_dtype="float16",
                            activation_type="identity", name=None):
    """``act(scale * op(x) @ op(y) + bias)`` for fp8 (e4m3 / e5m2) operands with a bf16 / fp16 result
    (python/paddle/tensor/linalg.py ``fp8_fp8_half_gemm_fused``).  On a GPU the product runs on the fp8 tensor-core
    path (per-tensor scale folded into the epilogue); on CPU the operands are widened first."""
    from ._core import dtype as _dt
    a, b = x.as_subclass(torch.Tensor), y.as_subclass(torch.Tensor)
    od = _dt.to_torch(output_dtype)
    a2 = a.transpose(-1, -2) if transpose_x else a
    b2 = b.transpose(-1, -2) if transpose_y else b
    if a.is_cuda and a.dim() == 2 and b.dim() == 2 and a2.shape[1] % 16 == 0 and b2.shape[1] % 16 == 0:
        one = torch.ones((), device=a.device)
        # _scaled_mm wants a row-major and b column-major
        out = torch._scaled_mm(a2.contiguous(), b2.t().contiguous().t(), scale_a=one, scale_b=one * scale, out_dtype=od)
    else:
        out = (a2.float() @ b2.float() * scale).to(od)
    if bias is not None:
        out = out + bias.as_subclass(torch.Tensor).to(od)
    if activation_type == "gelu":
        out = torch.nn.functional.gelu(out)
    elif activation_type == "relu":
        out = torch.relu(out)
    return as_tensor(out)
