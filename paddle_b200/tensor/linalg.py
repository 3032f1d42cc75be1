"""Linear-algebra API (python/paddle/tensor/linalg.py:220 ``matmul`` and python/paddle/linalg.py)."""
from __future__ import annotations

import torch

from .._core.tensor import as_tensor


def matmul(x, y, transpose_x=False, transpose_y=False, name=None):
    """``paddle.matmul``.  2-D (or flattenable) bf16 CUDA operands run on this library's tcgen05
    GEMM; everything else goes to torch."""
    from ..ops import functional as F_ops
    return F_ops.matmul(x, y, transpose_x, transpose_y)


def mm(input, mat2, name=None):
    return matmul(input, mat2)


def bmm(x, y, name=None):
    return torch.bmm(x, y)


def dot(x, y, name=None):
    return (x * y).sum(-1)


def mv(x, vec, name=None):
    return torch.mv(x, vec)


def cross(x, y, axis=9, name=None):
    if axis == 9:
        axis = next(i for i, s in enumerate(x.shape) if s == 3)
    return torch.cross(x, y, dim=axis)


def norm(x, p=None, axis=None, keepdim=False, name=None):
    if p is None:
        p = "fro" if (axis is None or isinstance(axis, (list, tuple))) else 2
    if p == "fro":
        return torch.linalg.vector_norm(x, 2, dim=tuple(axis) if isinstance(axis, list) else axis, keepdim=keepdim)
    if p == "nuc":
        return torch.linalg.matrix_norm(x, "nuc", dim=tuple(axis), keepdim=keepdim)
    if isinstance(axis, (list, tuple)) and len(axis) == 2:
        return torch.linalg.matrix_norm(x, p, dim=tuple(axis), keepdim=keepdim)
    return torch.linalg.vector_norm(x, p, dim=axis, keepdim=keepdim)


def vector_norm(x, p=2.0, axis=None, keepdim=False, name=None):
    return torch.linalg.vector_norm(x, p, dim=axis, keepdim=keepdim)


def matrix_norm(x, p="fro", axis=(-2, -1), keepdim=False, name=None):
    return torch.linalg.matrix_norm(x, p, dim=tuple(axis), keepdim=keepdim)


def dist(x, y, p=2, name=None):
    return torch.dist(x, y, p)


def cholesky(x, upper=False, name=None):
    return torch.linalg.cholesky(x, upper=upper)


def cholesky_solve(x, y, upper=False, name=None):
    return torch.cholesky_solve(x, y, upper)


def inv(x, name=None):
    return torch.linalg.inv(x)


inverse = inv


def pinv(x, rcond=1e-15, hermitian=False, name=None):
    return torch.linalg.pinv(x, rcond=rcond, hermitian=hermitian)


def det(x, name=None):
    return torch.linalg.det(x)


def slogdet(x, name=None):
    s, l = torch.linalg.slogdet(x)
    return torch.stack([s, l])


def svd(x, full_matrices=False, name=None):
    return torch.linalg.svd(x, full_matrices=full_matrices)


def qr(x, mode="reduced", name=None):
    return torch.linalg.qr(x, mode)


def lu(x, pivot=True, get_infos=False, name=None):
    lu_, piv, info = torch.linalg.lu_factor_ex(x, pivot=pivot)
    return (lu_, piv.to(torch.int32) , info) if get_infos else (lu_, piv.to(torch.int32))


def lu_unpack(x, y, unpack_ludata=True, unpack_pivots=True, name=None):
    return torch.lu_unpack(x, y.to(torch.int32), unpack_ludata, unpack_pivots)


def eig(x, name=None):
    return torch.linalg.eig(x)


def eigvals(x, name=None):
    return torch.linalg.eigvals(x)


def eigh(x, UPLO="L", name=None):
    return torch.linalg.eigh(x, UPLO)


def eigvalsh(x, UPLO="L", name=None):
    return torch.linalg.eigvalsh(x, UPLO)


def solve(x, y, name=None):
    return torch.linalg.solve(x, y)


def triangular_solve(x, y, upper=True, transpose=False, unitriangular=False, name=None):
    return torch.linalg.solve_triangular(x.mT if transpose else x, y, upper=(upper != transpose), unitriangular=unitriangular)


def lstsq(x, y, rcond=None, driver=None, name=None):
    r = torch.linalg.lstsq(x, y, rcond=rcond, driver=driver)
    return r.solution, r.residuals, r.rank, r.singular_values


def matrix_power(x, n, name=None):
    return torch.linalg.matrix_power(x, n)


def matrix_rank(x, tol=None, hermitian=False, name=None):
    return torch.linalg.matrix_rank(x, tol=tol, hermitian=hermitian)


def multi_dot(x, name=None):
    return torch.linalg.multi_dot(list(x))


def cond(x, p=None, name=None):
    return torch.linalg.cond(x, p)


def cov(x, rowvar=True, ddof=True, fweights=None, aweights=None, name=None):
    return torch.cov(x if rowvar else x.T, correction=1 if ddof else 0, fweights=fweights, aweights=aweights)


def corrcoef(x, rowvar=True, name=None):
    return torch.corrcoef(x if rowvar else x.T)


def householder_product(x, tau, name=None):
    return torch.linalg.householder_product(x, tau)


def matrix_exp(x, name=None):
    return torch.linalg.matrix_exp(x)


def einsum(equation, *operands):
    if len(operands) == 1 and isinstance(operands[0], (list, tuple)):
        operands = tuple(operands[0])
    return torch.einsum(equation, *operands)


def tensordot(x, y, axes=2, name=None):
    return torch.tensordot(x, y, dims=axes)


def cdist(x, y, p=2.0, compute_mode="use_mm_for_euclid_dist_if_necessary", name=None):
    return torch.cdist(x, y, p)


def bincount(x, weights=None, minlength=0, name=None):
    return torch.bincount(x, weights, minlength)


def histogramdd(x, bins=10, ranges=None, density=False, weights=None, name=None):
    return torch.histogramdd(x.cpu(), bins, range=ranges, weight=weights, density=density)
