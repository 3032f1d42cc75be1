"""Static-graph mode (record and replay): programs, executor, backward, control flow, persistence.
Modelled on test/legacy_test/test_executor_*.py, test_cond.py, test_while_loop_op.py, test_inference_model_io.py."""
import numpy as np
import pytest
import torch

import paddle_b200 as paddle
from paddle_b200 import static


@pytest.fixture(autouse=True)
def _static_mode():
    paddle.enable_static()
    yield
    paddle.disable_static()


def _regression_program(opt_cls=None, **opt_kw):
    main, startup = static.Program(), static.Program()
    with static.program_guard(main, startup):
        x = static.data("x", [None, 8], "float32")
        y = static.data("y", [None, 1], "float32")
        h = static.nn.fc(x, 16, activation="relu")
        pred = static.nn.fc(h, 1)
        loss = paddle.mean(paddle.nn.functional.square_error_cost(pred, y))
        test_prog = main.clone(for_test=True)
        if opt_cls is not None:
            opt_cls(**opt_kw).minimize(loss)
    return main, startup, test_prog, pred, loss


def test_train_loop_converges_and_batch_size_is_free():
    main, startup, test_prog, pred, loss = _regression_program(paddle.optimizer.Adam, learning_rate=0.02)
    exe = static.Executor()
    exe.run(startup)
    rng = np.random.RandomState(0)
    W = rng.randn(8, 1).astype("float32")
    first = last = None
    for i in range(150):
        xb = rng.randn(32, 8).astype("float32")
        last, = exe.run(main, feed={"x": xb, "y": xb @ W}, fetch_list=[loss])
        first = last if first is None else first
    assert float(last) < 0.05 * float(first)
    xb = rng.randn(5, 8).astype("float32")
    before = [p.numpy().copy() for p in main.all_parameters()]
    p, = exe.run(test_prog, feed={"x": xb, "y": xb @ W}, fetch_list=[pred])
    assert p.shape == (5, 1)
    for b, q in zip(before, main.all_parameters()):          # the test clone does not train
        np.testing.assert_array_equal(b, q.numpy())


def test_append_backward_matches_eager_autograd():
    main, startup, _, pred, loss = _regression_program()
    with static.program_guard(main, startup):
        pg = static.append_backward(loss)
    assert len(pg) == 4 and all(g.name == p.name + "@GRAD" for p, g in pg)
    xb = np.random.RandomState(1).randn(6, 8).astype("float32")
    yb = np.ones((6, 1), "float32")
    outs = static.Executor().run(main, feed={"x": xb, "y": yb}, fetch_list=[loss] + [g for _, g in pg])
    paddle.disable_static()                     # the reference below is plain eager autograd
    params = [p.as_subclass(torch.Tensor).detach().clone().requires_grad_(True) for p, _ in pg]
    w1, w2 = [p for p in params if p.dim() == 2]
    b1, b2 = [p for p in params if p.dim() == 1]
    ref = ((torch.relu(torch.tensor(xb) @ w1 + b1) @ w2 + b2 - torch.tensor(yb)) ** 2).mean()
    ref.backward()
    np.testing.assert_allclose(outs[0], ref.item(), rtol=1e-5)
    for got, p in zip(outs[1:], params):
        np.testing.assert_allclose(got, p.grad.numpy(), rtol=1e-4, atol=1e-6)


def test_gradients_wrt_input():
    main = static.Program()
    with static.program_guard(main):
        x = static.data("x", [None, 3], "float32")
        x.stop_gradient = False
        y = paddle.sum(paddle.tanh(x) * 2.0)
        gx, = static.gradients(y, x)
    xb = np.random.RandomState(2).randn(4, 3).astype("float32")
    g, = static.Executor().run(main, feed={"x": xb}, fetch_list=[gx])
    np.testing.assert_allclose(g, 2 * (1 - np.tanh(xb) ** 2), rtol=1e-5)


def test_cond_selects_branch_at_run_time():
    main = static.Program()
    with static.program_guard(main):
        a = static.data("a", [1], "float32")
        b = static.data("b", [1], "float32")
        out = static.nn.cond(a < b, lambda: a + b, lambda: a * b)
    exe = static.Executor()
    r, = exe.run(main, feed={"a": np.array([2.0], "float32"), "b": np.array([5.0], "float32")}, fetch_list=[out])
    assert r.item() == 7.0
    r, = exe.run(main, feed={"a": np.array([6.0], "float32"), "b": np.array([5.0], "float32")}, fetch_list=[out])
    assert r.item() == 30.0


def test_switch_case_and_case():
    main = static.Program()
    with static.program_guard(main):
        idx = static.data("idx", [1], "int32")
        v = static.data("v", [2], "float32")
        out = static.nn.switch_case(idx, {0: lambda: v + 1.0, 1: lambda: v * 10.0}, default=lambda: v - 1.0)
    exe = static.Executor()
    vb = np.array([1.0, 2.0], "float32")
    for i, want in [(0, vb + 1), (1, vb * 10), (7, vb - 1)]:
        r, = exe.run(main, feed={"idx": np.array([i], "int32"), "v": vb}, fetch_list=[out])
        np.testing.assert_allclose(r, want)


def test_while_loop_iterates_on_fed_bound():
    main = static.Program()
    with static.program_guard(main):
        n = static.data("n", [1], "int64")
        i = paddle.zeros([1], "int64")
        acc = paddle.zeros([1], "float32")
        i2, acc2 = static.nn.while_loop(lambda i, acc: i < n, lambda i, acc: [i + 1, acc + 1.5], [i, acc])
    exe = static.Executor()
    for bound in (0, 1, 7):
        ri, ra = exe.run(main, feed={"n": np.array([bound], "int64")}, fetch_list=[i2, acc2])
        assert ri.item() == bound and ra.item() == pytest.approx(1.5 * bound)


def test_for_test_clone_disables_dropout_and_freezes_batch_norm():
    main = static.Program()
    with static.program_guard(main):
        x = static.data("x", [None, 4, 3, 3], "float32")
        h = static.nn.batch_norm(x)
        out = paddle.nn.functional.dropout(h, 0.5, training=True)
        test_prog = main.clone(for_test=True)
    xb = np.random.RandomState(3).randn(8, 4, 3, 3).astype("float32") * 3 + 1
    exe = static.Executor()
    a, = exe.run(test_prog, feed={"x": xb}, fetch_list=[out])
    b, = exe.run(test_prog, feed={"x": xb}, fetch_list=[out])
    np.testing.assert_array_equal(a, b)
    np.testing.assert_allclose(a, xb / np.sqrt(1 + 1e-5), rtol=1e-4, atol=1e-5)     # running stats are still (0, 1)
    c, = exe.run(main, feed={"x": xb}, fetch_list=[out])
    assert (c == 0).mean() > 0.2                                                     # train program drops


def test_save_load_params_and_inference_model(tmp_path):
    main, startup, test_prog, pred, loss = _regression_program(paddle.optimizer.SGD, learning_rate=0.1)
    exe = static.Executor()
    xb = np.random.RandomState(4).randn(3, 8).astype("float32")
    want, = exe.run(test_prog, feed={"x": xb, "y": np.zeros((3, 1), "float32")}, fetch_list=[pred])
    static.save(main, str(tmp_path / "ckpt"))
    saved = static.load_program_state(str(tmp_path / "ckpt"))
    assert set(saved) == {p.name for p in main.all_parameters()}
    x_var = main.global_block().var("x")
    static.save_inference_model(str(tmp_path / "infer"), [x_var], [pred], exe, program=test_prog)
    for p in main.all_parameters():
        with torch.no_grad():
            p.as_subclass(torch.Tensor).zero_()
    static.load(main, str(tmp_path / "ckpt"), exe)
    got, = exe.run(test_prog, feed={"x": xb, "y": np.zeros((3, 1), "float32")}, fetch_list=[pred])
    np.testing.assert_allclose(got, want, rtol=1e-6)
    prog, feed_names, fetch_targets = static.load_inference_model(str(tmp_path / "infer"), exe)
    assert feed_names == ["x"]
    got2, = exe.run(prog, feed={"x": xb}, fetch_list=fetch_targets)
    np.testing.assert_allclose(got2, want, rtol=1e-6)
    # the same files serve the inference API
    from paddle_b200 import inference
    pred = inference.create_predictor(inference.Config(str(tmp_path / "infer.pdmodel"), str(tmp_path / "infer.pdiparams")))
    assert pred.get_input_names() == ["x"]
    pred.get_input_handle("x").copy_from_cpu(xb)
    pred.run()
    np.testing.assert_allclose(pred.get_output_handle(pred.get_output_names()[0]).copy_to_cpu(), want, rtol=1e-6)


def test_scope_and_ema():
    main, startup, _, pred, loss = _regression_program(paddle.optimizer.SGD, learning_rate=0.1)
    with static.program_guard(main, startup):
        ema = static.ExponentialMovingAverage(0.5)
        ema.update()
    exe = static.Executor()
    name = main.all_parameters()[0].name
    t = static.global_scope().find_var(name).get_tensor()
    assert t is main.all_parameters()[0]
    xb = np.ones((4, 8), "float32")
    for _ in range(3):
        exe.run(main, feed={"x": xb, "y": np.ones((4, 1), "float32")}, fetch_list=[loss])
    raw = t.numpy().copy()
    with ema.apply(exe):
        assert not np.allclose(t.numpy(), raw)
    np.testing.assert_array_equal(t.numpy(), raw)


def test_unrecorded_autograd_history_is_rejected():
    main = static.Program()
    with static.program_guard(main):
        w = paddle.create_parameter([3], "float32")
        from paddle_b200.static import graph
        with graph.suspend():
            hidden = w * 2.0
        with pytest.raises(RuntimeError, match="autograd history"):
            paddle.sum(hidden)


def test_conv_net_trains_with_batch_sizes_other_than_the_traced_one():
    """conv + batch-norm + pool + dropout + fc + cross-entropy + accuracy; the program is traced with batch 1 (sizes that
    Python code baked into view / reshape calls are repaired at replay) and run with batches of 32 and 96."""
    main, startup = static.Program(), static.Program()
    with static.program_guard(main, startup):
        img = static.data("img", [None, 1, 8, 8], "float32")
        lab = static.data("lab", [None, 1], "int64")
        h = static.nn.conv2d(img, 4, 3, padding=1, act="relu")
        h = static.nn.batch_norm(h)
        h = paddle.flatten(paddle.nn.functional.max_pool2d(h, 2), 1)
        logits = static.nn.fc(paddle.nn.functional.dropout(h, 0.1), 3)
        loss = paddle.nn.functional.cross_entropy(logits, lab)
        acc = static.accuracy(paddle.nn.functional.softmax(logits), lab)
        test_prog = main.clone(for_test=True)
        paddle.optimizer.Adam(0.01).minimize(loss)
    exe = static.Executor()
    rng = np.random.RandomState(0)
    X = rng.randn(96, 1, 8, 8).astype("float32")
    Y = ((X.mean((1, 2, 3)) > 0).astype("int64") + (X[:, 0, 0, 0] > 1).astype("int64")).reshape(-1, 1)
    first = None
    for _ in range(25):
        for i in range(0, 96, 32):
            l, a = exe.run(main, feed={"img": X[i:i + 32], "lab": Y[i:i + 32]}, fetch_list=[loss, acc])
            first = float(l) if first is None else first
    l2, a2 = exe.run(test_prog, feed={"img": X, "lab": Y}, fetch_list=[loss, acc])
    assert float(l2) < 0.6 * first and float(a2) > 0.8
    out, = exe.run(static.CompiledProgram(test_prog), feed={"img": X[:5], "lab": Y[:5]}, fetch_list=[logits])
    assert out.shape == (5, 3) and len(main.all_parameters()) == 6


def test_transformer_layer_program_matches_eager_at_another_batch_size():
    emb = paddle.nn.Embedding(50, 16)
    enc = paddle.nn.TransformerEncoderLayer(16, 4, 32, dropout=0.0)
    enc.eval()
    x = np.random.RandomState(0).randint(0, 50, (7, 10))
    paddle.disable_static()
    ref = enc(emb(paddle.to_tensor(x))).mean(1).numpy()
    paddle.enable_static()
    main = static.Program()
    with static.program_guard(main):
        ids = static.data("ids", [None, 10], "int64")
        out = enc(emb(ids)).mean(1)
    got, = static.Executor().run(main, feed={"ids": x}, fetch_list=[out])
    np.testing.assert_allclose(got, ref, rtol=1e-6, atol=1e-7)


def test_decomposition_rules_match_composites_eagerly():
    """Every registered rule equals the composite operator it replaces (values and input gradient)."""
    import torch
    import torch.nn.functional as TF

    from paddle_b200.decomposition import get_decomp_rule, registered_ops
    paddle.disable_static()                 # plain eager comparison; the fixture's teardown tolerates the early switch
    torch.manual_seed(0)
    x = torch.randn(6, 10, dtype=torch.float64)
    t = torch.randn(6, 10, dtype=torch.float64)
    w, b = torch.randn(10, dtype=torch.float64), torch.randn(10, dtype=torch.float64)
    cases = {
        "relu": (TF.relu, (x,), {}), "relu6": (TF.relu6, (x * 4,), {}), "leaky_relu": (TF.leaky_relu, (x, 0.1), {}),
        "sigmoid": (torch.sigmoid, (x,), {}), "silu": (TF.silu, (x,), {}), "gelu": (TF.gelu, (x,), {}),
        "hardswish": (TF.hardswish, (x * 3,), {}), "hardsigmoid": (TF.hardsigmoid, (x * 3,), {}),
        "hardtanh": (TF.hardtanh, (x,), {}), "softplus": (TF.softplus, (x * 10,), {}), "softsign": (TF.softsign, (x,), {}),
        "mish": (TF.mish, (x,), {}), "elu": (TF.elu, (x,), {}), "selu": (TF.selu, (x,), {}),
        "softmax": (TF.softmax, (x,), {"dim": 1}), "log_softmax": (TF.log_softmax, (x,), {"dim": 0}),
        "logsumexp": (torch.logsumexp, (x, 1), {}), "layer_norm": (TF.layer_norm, (x, [10], w, b), {}),
        "rms_norm": (TF.rms_norm, (x, [10], w, 1e-6), {}),
        "batch_norm": (TF.batch_norm, (x, w * 0.1, w.abs() + 0.5, w, b), {}),
        "group_norm": (TF.group_norm, (x.reshape(6, 10, 1), 5, w, b), {}),
        "instance_norm": (TF.instance_norm, (x.reshape(2, 3, 10),), {}),
        "normalize": (TF.normalize, (x,), {}), "var": (torch.var, (x, 1), {}), "std": (torch.std, (x, 0), {}),
        "square": (torch.square, (x,), {}), "linear": (TF.linear, (x, torch.randn(4, 10, dtype=torch.float64), None), {}),
        "addmm": (torch.addmm, (torch.randn(6, 6, dtype=torch.float64), x, x.t()), {"beta": 0.5, "alpha": 2.0}),
        "addcmul": (torch.addcmul, (x, t, t), {"value": 0.3}), "addcdiv": (torch.addcdiv, (x, t, t.abs() + 1), {"value": 0.3}),
        "lerp": (torch.lerp, (x, t, 0.3), {}), "mse_loss": (TF.mse_loss, (x, t), {}), "l1_loss": (TF.l1_loss, (x, t), {}),
        "smooth_l1_loss": (TF.smooth_l1_loss, (x, t), {}),
        "binary_cross_entropy_with_logits": (TF.binary_cross_entropy_with_logits, (x, torch.sigmoid(t)), {}),
        "cross_entropy": (TF.cross_entropy, (x, torch.tensor([1, 2, -100, 0, 9, 3])), {}),
        "dropout": (TF.dropout, (x, 0.5, False), {}),
    }
    untested = set(registered_ops()) - set(cases) - {"swiglu", "squared_l2_norm", "baddbmm"}
    assert not untested, untested
    for name, (fn, args, kwargs) in cases.items():
        a1 = [a.clone().requires_grad_(True) if isinstance(a, torch.Tensor) and a.is_floating_point() and i == 0 else a
              for i, a in enumerate(args)]
        a2 = [a.clone().requires_grad_(True) if isinstance(a, torch.Tensor) and a.is_floating_point() and i == 0 else a
              for i, a in enumerate(args)]
        want, got = fn(*a1, **kwargs), get_decomp_rule(name)(*a2, **kwargs)
        assert torch.allclose(want, got, atol=1e-9), name
        want.sum().backward()
        got.sum().backward()
        assert torch.allclose(a1[0].grad, a2[0].grad, atol=1e-9), name


def test_decompose_program_to_primitives_and_train():
    """decompose() rewrites a recorded program into primitive nodes only; outputs, black / white lists and a training
    step through the decomposed program (append_backward on primitives) are unchanged."""
    from paddle_b200.decomposition import PRIMITIVES, decompose, is_primitive_program

    def build():
        main, startup = static.Program(), static.Program()
        with static.program_guard(main, startup):
            paddle.seed(5)
            x = static.data("x", [-1, 16], "float32")
            lab = static.data("lab", [-1], "int64")
            fc1 = paddle.nn.Linear(16, 32)
            fc2 = paddle.nn.Linear(32, 8)
            h = paddle.nn.functional.gelu(fc1(x))
            h = paddle.nn.functional.layer_norm(h, [32])
            logits = fc2(h)
            prob = paddle.nn.functional.softmax(logits, axis=-1)
            loss = paddle.nn.functional.cross_entropy(logits, lab)
        return main, startup, x, lab, prob, loss, [fc1, fc2]

    rng = np.random.RandomState(0)
    xv, lv = rng.randn(12, 16).astype("float32"), rng.randint(0, 8, (12,)).astype("int64")
    exe = static.Executor()
    main, startup, x, lab, prob, loss, _ = build()
    base = exe.run(main, feed={"x": xv, "lab": lv}, fetch_list=[prob, loss])
    types_before = {n.type for n in main._nodes}
    assert {"gelu", "layer_norm", "softmax"} <= types_before
    decompose(main, [prob, loss], blacklist={"pd_op.softmax"})
    assert "softmax" in {n.type for n in main._nodes} and "gelu" not in {n.type for n in main._nodes}
    decompose(main, [prob, loss])
    assert is_primitive_program(main), sorted({n.type for n in main._nodes} - PRIMITIVES)
    after = exe.run(main, feed={"x": xv, "lab": lv}, fetch_list=[prob, loss])
    for a, b in zip(base, after):
        assert np.allclose(a, b, atol=1e-5)
    # whitelist
    main2, _, _, _, prob2, loss2, _ = build()
    decompose(main2, [prob2], whitelist={"gelu"})
    t2 = {n.type for n in main2._nodes}
    assert "gelu" not in t2 and "layer_norm" in t2
    # training through the decomposed program equals training through the composite one
    losses = []
    for dec in (False, True):
        main3, startup3, _, _, _, loss3, fcs = build()
        if dec:
            decompose(main3, [loss3])
        with static.program_guard(main3, startup3):
            opt = paddle.optimizer.SGD(learning_rate=0.1, parameters=[p for f in fcs for p in f.parameters()])
            opt.minimize(loss3)
        exe.run(startup3)
        losses.append([float(exe.run(main3, feed={"x": xv, "lab": lv}, fetch_list=[loss3])[0]) for _ in range(4)])
    assert losses[0][-1] < losses[0][0]
    assert np.allclose(losses[0], losses[1], atol=1e-5), losses
