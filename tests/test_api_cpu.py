"""API surface on CPU: Tensor semantics, Layer naming/state dict, optimizers vs formulas, save/load format,
amp scaler, jit cache, profiler scheduler, io, hapi."""
import os
import pickle

import numpy as np
import pytest
import torch

import paddle_b200 as paddle


def test_tensor_paddle_semantics():
    x = paddle.to_tensor([[1., 2., 3.], [4., 5., 6.]])
    assert x.shape == [2, 3] and x.stop_gradient
    assert x.transpose([1, 0]).shape == [3, 2]
    assert [t.shape for t in x.split(3, axis=1)] == [[2, 1]] * 3
    assert np.allclose(x.max(axis=1).numpy(), [3, 6])
    assert x.astype("int64").dtype == paddle.int64
    y = paddle.matmul(x, x, transpose_y=True)
    assert y.shape == [2, 2]
    x.stop_gradient = False
    (x * x).sum().backward()
    assert np.allclose(x.grad.numpy(), 2 * x.numpy())
    x.clear_gradient()
    assert float(x.grad.sum()) == 0.0
    assert isinstance(paddle.concat([x, x], axis=0), paddle.Tensor)
    assert paddle.arange(5).dtype == paddle.int64 and paddle.full([2], 1.5).dtype == paddle.float32


def test_layer_naming_and_state_dict():
    with paddle.utils.unique_name.guard():
        net = paddle.nn.Sequential(paddle.nn.Linear(4, 8), paddle.nn.ReLU(), paddle.nn.Linear(8, 2))
    names = [p.name for p in net.parameters()]
    assert names == ["linear_0.w_0", "linear_0.b_0", "linear_1.w_0", "linear_1.b_0"]
    assert list(net.state_dict().keys()) == ["0.weight", "0.bias", "2.weight", "2.bias"]
    assert net[0].weight.shape == [4, 8]          # [in, out]
    seen = []
    h = net.register_forward_post_hook(lambda l, i, o: seen.append(o.shape))
    net(paddle.ones([3, 4]))
    h.remove()
    assert seen == [[3, 2]]


def test_adamw_matches_formula_and_state_keys():
    with paddle.utils.unique_name.guard():
        l = paddle.nn.Linear(3, 2)
    w0 = l.weight.detach().clone()
    opt = paddle.optimizer.AdamW(0.1, parameters=l.parameters(), weight_decay=0.01, beta1=0.9, beta2=0.99)
    l(paddle.ones([1, 3])).sum().backward()
    g = l.weight.grad.clone()
    opt.step()
    m = 0.1 * g
    v = 0.01 * g * g
    ref = w0 * (1 - 0.1 * 0.01) - 0.1 / (1 - 0.9) * m / (v.sqrt() / (1 - 0.99) ** 0.5 + 1e-8)
    assert torch.allclose(l.weight.detach(), ref, atol=1e-6)
    sd = opt.state_dict()
    assert {"linear_0.w_0_moment1_0", "linear_0.w_0_moment2_0", "linear_0.w_0_beta1_pow_acc_0",
            "linear_0.b_0_beta2_pow_acc_0"} <= set(sd)
    assert abs(float(sd["linear_0.w_0_beta1_pow_acc_0"]) - 0.81) < 1e-6


def test_save_load_format(tmp_path):
    with paddle.utils.unique_name.guard():
        l = paddle.nn.Linear(3, 2)
    l.to(dtype="bfloat16")
    opt = paddle.optimizer.AdamW(0.1, parameters=l.parameters(), multi_precision=True)
    l(paddle.ones([1, 3]).astype("bfloat16")).sum().backward()
    opt.step()
    p = str(tmp_path / "m.pdparams")
    paddle.save(l.state_dict(), p)
    raw = pickle.load(open(p, "rb"))
    assert raw["StructuredToParameterName@@"] == {"weight": "linear_0.w_0", "bias": "linear_0.b_0"}
    assert isinstance(raw["weight"], np.ndarray) and raw["weight"].dtype == np.uint16     # bf16 bit pattern
    back = paddle.load(p)
    assert back["weight"].dtype == paddle.bfloat16 and torch.equal(back["weight"], l.weight.detach())
    po = str(tmp_path / "m.pdopt")
    paddle.save(opt.state_dict(), po)
    rawo = pickle.load(open(po, "rb"))
    assert isinstance(rawo["master_weights"]["linear_0.w_0"], tuple)          # (name, ndarray)
    assert rawo["master_weights"]["linear_0.w_0"][0] == "linear_0.w_0_fp32_master_0"
    opt2 = paddle.optimizer.AdamW(0.1, parameters=l.parameters(), multi_precision=True)
    opt2.set_state_dict(paddle.load(po))
    l(paddle.ones([1, 3]).astype("bfloat16")).sum().backward()
    opt2.step()
    assert torch.allclose(opt2._master_weights["linear_0.w_0"], opt2._master_weights["linear_0.w_0"])
    # protocol 2 big-array split
    big = {"w": paddle.zeros([10])}
    paddle.save(big, str(tmp_path / "b.pdparams"), protocol=2)
    assert paddle.load(str(tmp_path / "b.pdparams"))["w"].shape == [10]


def test_grad_scaler_skips_on_inf():
    l = paddle.nn.Linear(2, 2)
    opt = paddle.optimizer.SGD(0.1, parameters=l.parameters())
    sc = paddle.amp.GradScaler(init_loss_scaling=4.0, decr_every_n_nan_or_inf=1)
    w0 = l.weight.detach().clone()
    loss = l(paddle.ones([1, 2])).sum() * float("inf")
    sc.scale(loss).backward()
    sc.step(opt); sc.update()
    assert torch.equal(l.weight.detach(), w0) and sc.state_dict()["scale"] == 2.0
    opt.clear_grad()
    sc.scale(l(paddle.ones([1, 2])).sum()).backward()
    sc.step(opt); sc.update()
    assert not torch.equal(l.weight.detach(), w0)


def test_lr_schedulers_and_profiler_states():
    s = paddle.optimizer.lr.CosineAnnealingDecay(1.0, T_max=10)
    vals = []
    for _ in range(3):
        vals.append(s()); s.step()
    assert vals[0] == 1.0 and vals[1] < 1.0
    w = paddle.optimizer.lr.LinearWarmup(paddle.optimizer.lr.StepDecay(0.5, 2), 3, 0.0, 0.5)
    seq = []
    for _ in range(6):
        seq.append(round(w(), 4)); w.step()
    assert seq[:3] == [0.0, 0.1667, 0.3333] and seq[3] == 0.5
    sched = paddle.profiler.make_scheduler(closed=1, ready=1, record=2, repeat=1)
    S = paddle.profiler.ProfilerState
    assert [sched(i) for i in range(5)] == [S.CLOSED, S.READY, S.RECORD, S.RECORD_AND_RETURN, S.CLOSED]


def test_to_static_cache_and_jit_save_load(tmp_path):
    net = paddle.nn.Linear(4, 2)
    calls = []

    @paddle.jit.to_static
    def f(x):
        calls.append(1)
        return net(x) * 2
    a = f(paddle.ones([3, 4])); b = f(paddle.ones([3, 4])); c = f(paddle.ones([5, 4]))
    assert len(f.program_cache) == 2 and a.shape == [3, 2] and c.shape == [5, 2]
    paddle.jit.save(net, str(tmp_path / "inf"), input_spec=[paddle.static.InputSpec([None, 4], "float32")])
    loaded = paddle.jit.load(str(tmp_path / "inf"))
    assert torch.allclose(loaded(paddle.ones([3, 4])), net(paddle.ones([3, 4])))


def test_dataloader_and_distributed_batch_sampler():
    ds = paddle.io.TensorDataset([paddle.arange(10).astype("float32").reshape([10, 1]), paddle.arange(10)])
    dl = paddle.io.DataLoader(ds, batch_size=4)
    shapes = [b[0].shape for b in dl]
    assert shapes == [[4, 1], [4, 1], [2, 1]]
    s0 = list(paddle.io.DistributedBatchSampler(ds, 2, num_replicas=2, rank=0))
    s1 = list(paddle.io.DistributedBatchSampler(ds, 2, num_replicas=2, rank=1))
    assert sorted(sum(s0 + s1, [])) == list(range(10))


def test_hapi_fit():
    x = np.random.RandomState(0).randn(64, 4).astype(np.float32)
    y = (x.sum(1) > 0).astype(np.int64)
    ds = paddle.io.TensorDataset([paddle.to_tensor(x), paddle.to_tensor(y)])
    net = paddle.nn.Sequential(paddle.nn.Linear(4, 16), paddle.nn.ReLU(), paddle.nn.Linear(16, 2))
    m = paddle.Model(net)
    m.prepare(paddle.optimizer.Adam(0.05, parameters=net.parameters()), paddle.nn.CrossEntropyLoss(),
              paddle.metric.Accuracy())
    m.fit(ds, batch_size=16, epochs=8, verbose=0)
    assert m.evaluate(ds, batch_size=16, verbose=0)["acc"] > 0.8


def test_flags_and_clip():
    assert paddle.get_flags("FLAGS_check_nan_inf")["FLAGS_check_nan_inf"] is False
    with pytest.raises(ValueError):
        paddle.set_flags({"FLAGS_nope": 1})
    l = paddle.nn.Linear(2, 2)
    (l(paddle.ones([1, 2])).sum() * 100).backward()
    clip = paddle.nn.ClipGradByGlobalNorm(1.0)
    out = clip([(p, p.grad) for p in l.parameters()])
    tot = sum(float((g ** 2).sum()) for _, g in out) ** 0.5
    assert abs(tot - 1.0) < 1e-4


def test_tensor_semantics_table():
    """Paddle-specific conventions of creation, dtype promotion, indexing, autograd switches and persistence."""
    import os
    import tempfile

    import numpy as np

    import paddle_b200 as paddle
    assert paddle.to_tensor(1.5).dtype == paddle.float32 and paddle.to_tensor([1, 2]).dtype == paddle.int64
    assert paddle.to_tensor(np.ones(2)).dtype == paddle.float64 and paddle.to_tensor([True]).dtype == paddle.bool
    x = paddle.ones([2, 3])
    assert x.stop_gradient and x.shape == [2, 3] and isinstance(x.shape, list)
    assert (paddle.to_tensor([1]) + 1.5).dtype == paddle.float32 and (paddle.to_tensor([3]) / 2).dtype == paddle.float32
    w = paddle.create_parameter([2], "float32")
    assert not w.stop_gradient
    (w * 2).sum().backward()
    (w * 3).sum().backward()
    assert np.allclose(w.grad.numpy(), 5)                 # gradients accumulate until cleared
    w.clear_grad()
    assert w.grad is None or np.allclose(w.grad.numpy(), 0)
    a = paddle.arange(12).reshape([3, 4])
    assert a[..., 1].tolist() == [1, 5, 9] and a[a > 9].tolist() == [10, 11]
    assert a[[0, 2]].shape == [2, 4] and a[None, 1].shape == [1, 4] and a.T.shape == [4, 3]
    b = paddle.zeros([3, 4])
    b[1] = 1.0
    b[:, 0] = paddle.to_tensor([7.0, 8.0, 9.0])
    assert b.numpy()[1].tolist() == [8, 1, 1, 1]
    assert a.ndim == 2 and a.dim() == 2 and int(a.numel()) == 12 and len(a) == 3
    assert a.astype("float16").dtype == paddle.float16 and paddle.to_tensor(3.5).item() == 3.5
    g = paddle.grad((w * w).sum(), w)[0]
    assert np.allclose(g.numpy(), 2 * w.numpy())
    with paddle.no_grad():
        assert (w * 2).stop_gradient
    assert (w * 2).detach().stop_gradient and not (w * 1).clone().stop_gradient
    d = tempfile.mkdtemp()
    lin = paddle.nn.Linear(3, 2)
    paddle.save(lin.state_dict(), os.path.join(d, "m.pdparams"))
    sd = paddle.load(os.path.join(d, "m.pdparams"))
    assert set(sd) == {"weight", "bias"} and sd["weight"].shape == [3, 2] and lin.weight.shape == [3, 2]
    assert paddle.argmax(a, axis=1).tolist() == [3, 3, 3] and paddle.unique(paddle.to_tensor([3, 1, 3, 2])).tolist() == [1, 2, 3]
    assert paddle.nonzero(paddle.to_tensor([0, 1, 0, 2])).tolist() == [[1], [3]] and paddle.shape(a).tolist() == [3, 4]
    paddle.seed(1)
    r1 = paddle.rand([3]).tolist()
    paddle.seed(1)
    assert paddle.rand([3]).tolist() == r1
    assert paddle.matmul(paddle.ones([2, 2], "bfloat16"), paddle.ones([2, 2], "bfloat16")).dtype == paddle.bfloat16


def test_typed_errors_follow_the_reference_mapping():
    """Error codes map onto the built-in exception classes the reference raises for them, share EnforceNotMet as base,
    and the native launcher codes arrive as typed errors that are still RuntimeErrors."""
    import pytest

    import paddle_b200 as paddle
    from paddle_b200.framework import errors
    from paddle_b200.ops import _lib
    pairs = {errors.InvalidArgumentError: ValueError, errors.OutOfRangeError: IndexError,
             errors.ResourceExhaustedError: MemoryError, errors.UnimplementedError: NotImplementedError,
             errors.FatalError: SystemError, errors.ExternalError: OSError, errors.InvalidTypeError: TypeError,
             errors.NotFoundError: RuntimeError, errors.ExecutionTimeoutError: RuntimeError}
    for cls, builtin in pairs.items():
        assert issubclass(cls, builtin) and issubclass(cls, errors.EnforceNotMet)
        assert errors.BY_CODE[cls.code] is cls
    assert paddle.base.core.EnforceNotMet is errors.EnforceNotMet
    with pytest.raises(ValueError, match=r"\(InvalidArgumentError\).*bad shape"):
        _lib.check(-1, "pd_some_kernel")
    with pytest.raises(RuntimeError):
        _lib.check(-2, "pd_some_kernel")
    with pytest.raises(IndexError):
        _lib.check(-5, "pd_some_kernel")
    with pytest.raises(OSError):
        _lib.check(-4, "pd_some_kernel")
    assert issubclass(_lib.KernelStatusError, errors.ExecutionTimeoutError)
    with pytest.raises(errors.PreconditionNotMetError):
        errors.enforce(False, message="state")
    errors.enforce(True)


def test_flag_registry_covers_the_reference_and_effects_apply(tmp_path):
    """Every flag the reference exports is registered with a type, a kind and a note; ``set_flags`` converts and
    checks types, runs the effect handlers and mirrors values into the native runtime."""
    import re
    import subprocess
    import sys

    import torch

    from paddle_b200.framework import flags as F
    info = F.flag_info()
    assert len(info) >= 185 and all(v["kind"] in ("effect", "read", "inert") for v in info.values())
    assert all(v["note"] for v in info.values() if v["kind"] == "inert")
    ref_root = os.environ.get("PADDLE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                                                                       "reference")
    ref = os.path.join(ref_root, "paddle", "common", "flags.cc")
    if os.path.exists(ref):
        names = set(re.findall(r"PHI_DEFINE_EXPORTED_\w+\(\s*(?://[^\n]*\n\s*)?(\w+)\s*,", open(ref).read()))
        assert len(names) > 150 and not {n for n in names if "FLAGS_" + n not in info}
    # conversion and type checks
    paddle.set_flags({"FLAGS_cudnn_exhaustive_search": "true", "paddle_num_threads": 2, "FLAGS_fraction_of_gpu_memory_to_use": 1})
    assert torch.backends.cudnn.benchmark is True and torch.get_num_threads() == 2
    assert paddle.get_flags("FLAGS_fraction_of_gpu_memory_to_use")["FLAGS_fraction_of_gpu_memory_to_use"] == 1.0
    paddle.set_flags({"FLAGS_cudnn_exhaustive_search": False})
    with pytest.raises(TypeError):
        paddle.set_flags({"FLAGS_paddle_num_threads": 1.5})
    with pytest.raises(TypeError):
        paddle.set_flags({"FLAGS_check_nan_inf": "yes" and [1]})
    # tensor checker level: 1 = report and continue
    paddle.set_flags({"FLAGS_check_nan_inf_level": 1, "FLAGS_check_nan_inf": True})
    try:
        out = paddle.to_tensor([1.0, 0.0]) / paddle.to_tensor([0.0, 0.0])
        assert not bool(torch.isfinite(out).all())
    finally:
        paddle.set_flags({"FLAGS_check_nan_inf": False, "FLAGS_check_nan_inf_level": 0})
    paddle.set_flags({"FLAGS_check_nan_inf": True})
    try:
        with pytest.raises(RuntimeError, match="nan/inf"):
            paddle.to_tensor([1.0]) / paddle.to_tensor([0.0])
    finally:
        paddle.set_flags({"FLAGS_check_nan_inf": False})
    # accuracy_check reads its default tolerances from the flags
    from paddle_b200 import _C_ops
    a = paddle.ones([4])
    with pytest.raises(AssertionError):
        _C_ops.accuracy_check(a, a + 1e-4, "f")
    paddle.set_flags({"FLAGS_accuracy_check_atol_fp32": 1e-3})
    try:
        assert bool(_C_ops.accuracy_check(a, a + 1e-4, "f"))
    finally:
        paddle.set_flags({"FLAGS_accuracy_check_atol_fp32": 1e-6})
    # native mirror
    from paddle_b200.ops import _lib
    import ctypes
    rt = _lib.runtime()
    paddle.set_flags({"FLAGS_async_trace_count": 9})
    buf = ctypes.create_string_buffer(32)
    assert rt.pd_flag_get(b"FLAGS_async_trace_count", buf, 32) == 1 and buf.value == b"9"
    paddle.set_flags({"FLAGS_async_trace_count": 5})
    # the API tracer through FLAGS_trace_api, and flags from the environment acting at import
    apis = tmp_path / "apis.txt"
    apis.write_text("paddle.nn.functional.relu\n")
    paddle.set_flags({"FLAGS_trace_api": f"{apis},{tmp_path / 'trace.txt'}"})
    try:
        paddle.nn.functional.relu(paddle.to_tensor([-1.0, 1.0]))
    finally:
        paddle.set_flags({"FLAGS_trace_api": ""})
    assert "relu(" in (tmp_path / "trace.txt").read_text()
    code = "import torch, paddle_b200; print(torch.backends.cudnn.deterministic, paddle_b200.get_flags('FLAGS_use_autotune'))"
    env = dict(os.environ, FLAGS_cudnn_deterministic="1", FLAGS_use_autotune="true", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120).stdout
    assert out.strip() == "True {'FLAGS_use_autotune': True}"
