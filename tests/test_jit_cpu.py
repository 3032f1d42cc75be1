"""``jit.to_static(full_graph=True)``: Python control flow on tensors becomes cond / while_loop nodes of a recorded
program (test/dygraph_to_static/test_ifelse.py, test_loop.py, test_logical.py patterns): one program serves inputs that
take different branches, results and gradients match eager execution."""
import numpy as np

import paddle_b200 as paddle


def _branchy(x, y):
    if x.sum() > 0:
        z = x + y
        w = z * 2
    else:
        z = x - y
        w = z * 3
    return w + z


def _loop(x, n):
    i = 0
    s = paddle.zeros([1])
    while i < n:
        s = s + x * i
        i = i + 1
    return s


def _logical(x):
    if x.mean() > 0 and not (x.max() > 10):
        y = x * 2
    else:
        y = x * 0
    return y


def _nested(x):
    if x.sum() > 0:
        if x.max() > 5:
            y = x * 10
        else:
            y = x + 1
    else:
        y = -x
    return y


def test_if_else_one_program_both_branches():
    sf = paddle.jit.to_static(_branchy, full_graph=True)
    y = paddle.to_tensor(np.full((2, 3), 0.5, "float32"))
    for v in (1.0, -1.0, 2.0):
        x = paddle.to_tensor(np.full((2, 3), v, "float32"))
        np.testing.assert_allclose(sf(x, y).numpy(), _branchy(x, y).numpy())
    assert len(sf._programs) == 1
    names = [n.name for n in sf.concrete_program(x, y)[0]._nodes]
    assert "cond" in names


def test_while_loop_on_tensor_bound():
    sf = paddle.jit.to_static(_loop, full_graph=True)
    x = paddle.to_tensor([2.0])
    for n in (0, 1, 5):
        nt = paddle.to_tensor([n], dtype="int64")
        assert float(sf(x, nt)) == float(_loop(x, nt)) == 2.0 * sum(range(n))
    assert len(sf._programs) == 1


def test_logical_operators_and_nested_if():
    sl, sn = paddle.jit.to_static(_logical, full_graph=True), paddle.jit.to_static(_nested, full_graph=True)
    for v in ([1.0, 2.0], [1.0, 20.0], [-1.0, -2.0]):
        t = paddle.to_tensor(v)
        np.testing.assert_allclose(sl(t).numpy(), _logical(t).numpy())
        np.testing.assert_allclose(sn(t).numpy(), _nested(t).numpy())
    assert len(sl._programs) == 1 and len(sn._programs) == 1


class _Net(paddle.nn.Layer):
    def __init__(self):
        super().__init__()
        self.a = paddle.nn.Linear(4, 4)
        self.b = paddle.nn.Linear(4, 4)

    def forward(self, x):
        if x.sum() > 0:
            h = self.a(x)
        else:
            h = self.b(x)
        return h.sum()


def test_layer_gradients_flow_through_the_replayed_program():
    net, ref = _Net(), _Net()
    ref.set_state_dict(net.state_dict())
    net = paddle.jit.to_static(net, full_graph=True)
    for sign in (1.0, -1.0, 1.0):
        x = paddle.to_tensor(np.full((2, 4), sign, "float32"))
        x.stop_gradient = False
        xr = paddle.to_tensor(np.full((2, 4), sign, "float32"))
        xr.stop_gradient = False
        l1, l2 = net(x), ref(xr)
        l1.backward()
        l2.backward()
        np.testing.assert_allclose(float(l1), float(l2), rtol=1e-6)
        np.testing.assert_allclose(x.grad.numpy(), xr.grad.numpy(), rtol=1e-6)
    for (_, p1), (_, p2) in zip(net.named_parameters(), ref.named_parameters()):
        np.testing.assert_allclose(p1.grad.numpy(), p2.grad.numpy(), rtol=1e-6)


def test_python_conditions_keep_python_semantics():
    def f(x, flag):
        if flag:
            y = x + 1
        else:
            y = x - 1
        k = 0
        while k < 3:
            y = y * 2
            k += 1
        return y
    sf = paddle.jit.to_static(f, full_graph=True)
    x = paddle.to_tensor([1.0])
    assert float(sf(x, True)) == 16.0 and float(sf(x, False)) == 0.0
    assert len(sf._programs) == 2                      # Python values are part of the signature


def test_for_range_with_tensor_bound():
    def f(x, n):
        acc = paddle.zeros([1])
        for i in range(n):
            acc = acc + x * (i + 1)
        return acc
    sf = paddle.jit.to_static(f, full_graph=True)
    x = paddle.to_tensor([3.0])
    for n in (0, 2, 4):
        nt = paddle.to_tensor([n], dtype="int64")
        assert float(sf(x, nt)) == 3.0 * sum(range(1, n + 1))
    assert len(sf._programs) == 1
    assert float(sf(x, 3)) == 18.0 and float(f(x, 3)) == 18.0         # Python bound: unrolled at trace time


def test_early_return_in_tensor_dependent_if():
    def f(x):
        y = x * 2
        if y.sum() > 10:
            return y - 10
        z = y + 1
        if z.max() < 0:
            return z * 0
        return z

    sf = paddle.jit.to_static(f, full_graph=True)
    for v in ([10.0, 10.0], [1.0, 2.0], [-3.0, -4.0]):
        t = paddle.to_tensor(v)
        np.testing.assert_allclose(sf(t).numpy(), f(t).numpy())
    assert len(sf._programs) == 1
