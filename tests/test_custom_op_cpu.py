"""Custom C++ operators: a source written against ``paddle/extension.h`` is built just in time and its operators
become Python functions with autograd, list / optional inputs, attribute conversion and shape / dtype inference
(reference behaviour: python/paddle/utils/cpp_extension/, test/custom_op/test_custom_relu_op_jit.py)."""
import os

import numpy as np
import pytest

import paddle_b200 as paddle
from paddle_b200.utils import cpp_extension

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def ops(tmp_path_factory):
    build = os.environ.get("PD_TEST_EXT_DIR") or str(tmp_path_factory.mktemp("ext"))
    return cpp_extension.load("pd_test_ops", [os.path.join(HERE, "custom_op", "relu_scale_op.cc")], build_directory=build)


@pytest.mark.timeout(600)
def test_custom_operator_forward_backward_and_metadata(ops):
    assert sorted(ops.__all__) == ["relu_scale", "sum_list"] and not hasattr(ops, "relu_scale_grad")
    assert ops.relu_scale.meta["inputs"] == ["X"] and ops.relu_scale.meta["attrs"] == ["scale: float"]
    x = paddle.to_tensor(np.array([[-1.0, 2.0], [3.0, -4.0]], "float32"), stop_gradient=False)
    y = ops.relu_scale(x, 2.5)
    assert isinstance(y, paddle.Tensor) and y.numpy().tolist() == [[0.0, 5.0], [7.5, 0.0]]
    (y * paddle.to_tensor([[1.0, 2.0], [3.0, 4.0]])).sum().backward()
    assert x.grad.numpy().tolist() == [[0.0, 5.0], [7.5, 0.0]]                  # the custom backward kernel: g * scale where out > 0
    x64 = paddle.to_tensor(np.array([1.0, -1.0]), stop_gradient=False)           # float64 dispatch
    assert ops.relu_scale(x64, scale=3).dtype == paddle.float64
    with pytest.raises(RuntimeError, match="not implemented for this data type"):
        ops.relu_scale(paddle.to_tensor([1, 2]), 1.0)
    with pytest.raises(TypeError, match="missing attribute"):
        ops.relu_scale(x)
    with pytest.raises(TypeError, match="unexpected"):
        ops.relu_scale(x, 1.0, slope=2)
    # through a Layer and an optimizer step
    lin = paddle.nn.Linear(2, 2)
    opt = paddle.optimizer.SGD(0.1, parameters=lin.parameters())
    before = lin.weight.numpy().copy()
    ops.relu_scale(lin(paddle.ones([3, 2])), 1.0).sum().backward()
    opt.step()
    assert not np.allclose(before, lin.weight.numpy()) or float(np.abs(before).sum()) == 0.0
    # list + optional inputs, vector and bool attributes, two outputs
    s, c = ops.sum_list([paddle.ones([2]), paddle.ones([2]) * 2], None, [1, 3], True)
    assert s.numpy().tolist() == [-7.0, -7.0] and c.numpy().tolist() == [2]
    s, _ = ops.sum_list([paddle.ones([2])], Bias=paddle.full([2], 0.5), repeat=[], negate=False)
    assert s.numpy().tolist() == [1.5, 1.5]
    with pytest.raises(RuntimeError, match="at least one tensor"):
        ops.sum_list([], None, [], False)
    assert ops.infer_shape("relu_scale", [4, 5]) == [[4, 5]] and ops.infer_dtype("relu_scale", 9) == [9]
    assert os.path.exists(os.path.join(cpp_extension.get_include(), "paddle", "extension.h"))


def test_extension_factories_carry_include_path_and_arch(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    ext = cpp_extension.CppExtension(sources=["a.cc"], name="my_ops")
    assert ext.name == "my_ops" and cpp_extension.get_include() in ext.include_dirs
    assert any(s.endswith("my_ops_pd_bind.cc") for s in ext.sources) and "a.cc" in ext.sources
    monkeypatch.setenv("PADDLE_EXTENSION_DIR", str(tmp_path / "cache"))
    assert cpp_extension.get_build_directory() == str(tmp_path / "cache") and os.path.isdir(tmp_path / "cache")
    assert "arch=compute_100a,code=sm_100a" in cpp_extension.SM100_FLAGS


@pytest.mark.gpu
@pytest.mark.timeout(900)
@pytest.mark.skipif(not os.environ.get("PD_TEST_CUSTOM_CUDA_OP"), reason="builds a CUDA extension (minutes); set PD_TEST_CUSTOM_CUDA_OP=1")
def test_custom_cuda_operator(tmp_path):
    """A ``.cu`` operator compiled for sm_100a runs on the tensor's stream; checked against a * x + y in fp32."""
    m = cpp_extension.load("pd_test_cuda_ops", [os.path.join(HERE, "custom_op", "axpy_op.cu")], build_directory=str(tmp_path))
    x = paddle.randn([1000], dtype="float32").cuda()
    y = paddle.randn([1000], dtype="float32").cuda()
    x.stop_gradient = False
    out = m.axpy(x, y, 2.0)
    assert np.allclose(out.numpy(), 2.0 * x.numpy() + y.numpy(), atol=1e-6)
    out.sum().backward()
    assert np.allclose(x.grad.numpy(), 2.0)
