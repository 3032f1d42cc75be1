"""``minimize_bfgs`` / ``minimize_lbfgs`` (python/paddle/incubate/optimizer/functional/{bfgs,lbfgs}.py):
quasi-Newton minimisation of a scalar function of one tensor with a strong-Wolfe line search.
Returns ``(is_converge, num_func_calls, position, objective_value, objective_gradient[, inverse_hessian])``."""
from __future__ import annotations

import torch

from ...._core.tensor import as_tensor


def _value_and_grad(f, x, counter):
    x = x.detach().requires_grad_(True)
    y = f(as_tensor(x))
    y = y.as_subclass(torch.Tensor) if isinstance(y, torch.Tensor) else torch.as_tensor(y)
    g, = torch.autograd.grad(y, x)
    counter[0] += 1
    return y.detach(), g


def _strong_wolfe(f, x, d, f0, g0, counter, alpha=1.0, c1=1e-4, c2=0.9, max_iters=50):
    """Bracketing + zoom line search (Nocedal & Wright, algorithms 3.5 / 3.6)."""
    dg0 = torch.dot(g0, d)
    a_prev, f_prev = 0.0, f0
    a = alpha
    phi = lambda t: _value_and_grad(f, x + t * d, counter)     # noqa: E731

    def zoom(lo, hi, f_lo):
        fa, ga, a_ = f_lo, g0, lo
        for _ in range(max_iters):
            a_ = 0.5 * (lo + hi)
            fa, ga = phi(a_)
            if fa > f0 + c1 * a_ * dg0 or fa >= f_lo:
                hi = a_
            else:
                dga = torch.dot(ga, d)
                if abs(dga) <= -c2 * dg0:
                    return a_, fa, ga
                if dga * (hi - lo) >= 0:
                    hi = lo
                lo, f_lo = a_, fa
            if abs(hi - lo) < 1e-12:
                break
        return a_, fa, ga
    fa, ga = f0, g0
    for i in range(max_iters):
        fa, ga = phi(a)
        if fa > f0 + c1 * a * dg0 or (i > 0 and fa >= f_prev):
            return zoom(a_prev, a, f_prev)
        dga = torch.dot(ga, d)
        if abs(dga) <= -c2 * dg0:
            return a, fa, ga
        if dga >= 0:
            return zoom(a, a_prev, fa)
        a_prev, f_prev = a, fa
        a = a * 2.0
    return a, fa, ga


def _minimize(objective_func, initial_position, max_iters, tolerance_grad, tolerance_change, initial_inverse_hessian_estimate,
              line_search_fn, max_line_search_iters, initial_step_length, dtype, history_size):
    if line_search_fn != "strong_wolfe":
        raise NotImplementedError(f"Currently only support line_search_fn = 'strong_wolfe', but the specified is '{line_search_fn}'")
    td = torch.float64 if dtype == "float64" else torch.float32
    x = initial_position.as_subclass(torch.Tensor).detach().to(td).reshape(-1)
    n = x.numel()
    counter = [0]
    fx, g = _value_and_grad(objective_func, x, counter)
    H = None
    if history_size is None:
        H = torch.eye(n, dtype=td) if initial_inverse_hessian_estimate is None else \
            initial_inverse_hessian_estimate.as_subclass(torch.Tensor).to(td).clone()
    S, Y = [], []
    converged = False
    for _ in range(max_iters):
        if g.abs().max() < tolerance_grad:
            converged = True
            break
        if H is not None:
            d = -(H @ g)
        else:                                   # two-loop recursion
            q = g.clone()
            al = []
            for s, y in zip(reversed(S), reversed(Y)):
                a_i = torch.dot(s, q) / torch.dot(y, s)
                al.append(a_i)
                q -= a_i * y
            gamma = torch.dot(S[-1], Y[-1]) / torch.dot(Y[-1], Y[-1]) if S else 1.0
            r = gamma * q
            for (s, y), a_i in zip(zip(S, Y), reversed(al)):
                b = torch.dot(y, r) / torch.dot(y, s)
                r += s * (a_i - b)
            d = -r
        a, f_new, g_new = _strong_wolfe(objective_func, x, d, fx, g, counter, initial_step_length,
                                        max_iters=max_line_search_iters)
        s, y = a * d, g_new - g
        x, change = x + s, abs(float(f_new - fx))
        fx, g = f_new, g_new
        sy = torch.dot(s, y)
        if sy > 1e-10:
            if H is not None:
                rho = 1.0 / sy
                I = torch.eye(n, dtype=td)
                H = (I - rho * torch.outer(s, y)) @ H @ (I - rho * torch.outer(y, s)) + rho * torch.outer(s, s)
            else:
                S.append(s), Y.append(y)
                if len(S) > history_size:
                    S.pop(0), Y.pop(0)
        if change < tolerance_change or s.abs().max() < tolerance_change:
            converged = bool(g.abs().max() < tolerance_grad) or True
            break
    shape = initial_position.shape
    out = [as_tensor(torch.tensor(converged)), as_tensor(torch.tensor(counter[0])), as_tensor(x.reshape(list(shape))),
           as_tensor(fx), as_tensor(g.reshape(list(shape)))]
    if H is not None:
        out.append(as_tensor(H))
    return tuple(out)


def minimize_bfgs(objective_func, initial_position, max_iters=50, tolerance_grad=1e-7, tolerance_change=1e-9,
                  initial_inverse_hessian_estimate=None, line_search_fn="strong_wolfe", max_line_search_iters=50,
                  initial_step_length=1.0, dtype="float32", name=None):
    return _minimize(objective_func, initial_position, max_iters, tolerance_grad, tolerance_change,
                     initial_inverse_hessian_estimate, line_search_fn, max_line_search_iters, initial_step_length, dtype, None)


def minimize_lbfgs(objective_func, initial_position, history_size=100, max_iters=50, tolerance_grad=1e-8,
                   tolerance_change=1e-8, initial_inverse_hessian_estimate=None, line_search_fn="strong_wolfe",
                   max_line_search_iters=50, initial_step_length=1.0, dtype="float32", name=None):
    return _minimize(objective_func, initial_position, max_iters, tolerance_grad, tolerance_change,
                     initial_inverse_hessian_estimate, line_search_fn, max_line_search_iters, initial_step_length, dtype,
                     history_size)
