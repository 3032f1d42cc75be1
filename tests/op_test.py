"""Operator test harness in the style of the reference's ``OpTest`` (test/legacy_test/op_test.py:418): an operator
case gives NumPy inputs, a NumPy reference of the forward, and the names of the inputs to differentiate;
``check_output`` compares the framework's forward with the reference, ``check_grad`` compares autograd with a
central-difference numeric gradient of the framework's own forward (``get_numeric_gradient`` :148)."""
import numpy as np

import paddle_b200 as paddle


def _to_tensors(inputs, grad_names=()):
    out = {}
    for k, v in inputs.items():
        if isinstance(v, np.ndarray):
            t = paddle.to_tensor(v)
            t.stop_gradient = k not in grad_names
            out[k] = t
        else:
            out[k] = v
    return out


def _first(out):
    return out[0] if isinstance(out, (tuple, list)) else out


def check_output(fn, inputs, expect, rtol=1e-5, atol=1e-6):
    got = fn(**_to_tensors(inputs))
    gots = got if isinstance(got, (tuple, list)) else [got]
    exps = expect if isinstance(expect, (tuple, list)) else [expect]
    assert len(gots) >= len(exps)
    for g, e in zip(gots, exps):
        g = g.numpy() if hasattr(g, "numpy") else np.asarray(g)
        assert tuple(g.shape) == tuple(np.shape(e)), f"shape {g.shape} vs {np.shape(e)}"
        np.testing.assert_allclose(g.astype(np.float64) if g.dtype != bool else g, e, rtol=rtol, atol=atol)


def numeric_grad(fn, inputs, name, weights, delta=1e-3):
    base = {k: (v.astype(np.float64) if isinstance(v, np.ndarray) and v.dtype.kind == "f" else v) for k, v in inputs.items()}
    x = base[name]
    g = np.zeros_like(x)
    flat, gf = x.reshape(-1), g.reshape(-1)

    def loss():
        out = _first(fn(**_to_tensors(base)))
        return float((out.numpy().astype(np.float64) * weights).sum())
    for i in range(flat.size):
        old = flat[i]
        flat[i] = old + delta
        hi = loss()
        flat[i] = old - delta
        lo = loss()
        flat[i] = old
        gf[i] = (hi - lo) / (2 * delta)
    return g


def check_grad(fn, inputs, names, max_rel=5e-3, delta=1e-3):
    """Analytic gradient of ``sum(out * w)`` (w fixed, random) against the numeric one, in float64."""
    inputs64 = {k: (v.astype(np.float64) if isinstance(v, np.ndarray) and v.dtype.kind == "f" else v) for k, v in inputs.items()}
    ts = _to_tensors(inputs64, names)
    out = _first(fn(**ts))
    w = np.random.RandomState(7).uniform(0.5, 1.5, size=tuple(out.shape))
    (out * paddle.to_tensor(w)).sum().backward()
    for n in names:
        ana = ts[n].grad.numpy()
        num = numeric_grad(fn, inputs64, n, w, delta)
        denom = np.maximum(np.abs(num), 1e-3)
        rel = np.abs(ana - num) / denom
        assert rel.max() < max_rel, f"grad of {n}: max rel err {rel.max():.3e} at {np.unravel_index(rel.argmax(), rel.shape)}"
