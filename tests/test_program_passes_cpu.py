"""Passes that rewrite recorded programs: recomputation between checkpoints and mixed-precision regions."""
import numpy as np
import pytest
import torch

import paddle_b200 as paddle
import paddle_b200.nn as nn
import paddle_b200.nn.functional as F
from paddle_b200.distributed.passes import PassContext, PassManager, SegmentNode, new_pass


@pytest.fixture(autouse=True)
def _dynamic_mode_after():
    yield
    paddle.disable_static()


def _program():
    paddle.seed(2)
    paddle.enable_static()
    main, start = paddle.static.Program(), paddle.static.Program()
    with paddle.static.program_guard(main, start):
        x = paddle.static.data("x", [16, 32], "float32")
        y = paddle.static.data("y", [16, 1], "float32")
        l1, l2, l3 = nn.Linear(32, 64), nn.Linear(64, 64), nn.Linear(64, 1)
        h1 = F.gelu(l1(x))
        h2 = F.gelu(l2(h1)) + h1
        pred = l3(h2)
        loss = F.mse_loss(pred, y)
        pg = paddle.static.append_backward(loss)
    paddle.disable_static()
    return main, start, (h1, h2, pred, loss), pg


def _run(main, fetch):
    g = torch.Generator().manual_seed(1)
    feed = {"x": torch.randn(16, 32, generator=g).numpy(), "y": torch.randn(16, 1, generator=g).numpy()}
    paddle.enable_static()
    try:
        exe = paddle.static.Executor()
        return [np.asarray(v) for v in exe.run(main, feed=feed, fetch_list=fetch)]
    finally:
        paddle.disable_static()


def test_recompute_pass_keeps_values_and_gradients_and_runs_segments_twice():
    main, start, (h1, h2, pred, loss), pg = _program()
    fetch = [loss, pred] + [g for _, g in pg]
    before = _run(main, fetch)
    n_before = len(main._nodes)
    ctx = new_pass("auto_parallel_recompute", {"checkpoints": [h1, h2]}).apply([main], [start], PassContext())
    assert ctx.get_attr("recompute_segments") == 2
    segs = [n for n in main._nodes if isinstance(n, SegmentNode)]
    assert len(segs) == 2 and all(s.mode == "recompute" for s in segs) and len(main._nodes) < n_before
    assert main._nodes[-1].name == "backward"
    after = _run(main, fetch)
    for a, b in zip(before, after):
        np.testing.assert_allclose(a, b, rtol=1e-6, atol=1e-7)
    assert [s.runs for s in segs] == [2, 2]                     # once forward, once in the backward pass
    # without checkpoints the pass declines
    main2, start2, _, _ = _program()
    n2 = len(main2._nodes)
    new_pass("auto_parallel_recompute").apply([main2], [start2], PassContext())
    assert len(main2._nodes) == n2


def test_amp_pass_runs_the_forward_in_low_precision():
    main, start, (h1, h2, pred, loss), pg = _program()
    want = _run(main, [loss, pred])
    mgr = PassManager([new_pass("auto_parallel_amp", {"dtype": "bfloat16", "keep": [pred]})])
    mgr.apply([main], [start])
    assert mgr.names == ["auto_parallel_amp"]
    region = main._nodes[0]
    assert isinstance(region, SegmentNode) and region.mode == "autocast" and region.dtype == torch.bfloat16
    got = _run(main, [loss, pred] + [g for _, g in pg])
    assert got[1].dtype != np.float32 or not np.array_equal(got[1], want[1])      # matmuls ran in bfloat16
    np.testing.assert_allclose(got[0].astype(np.float32), want[0], rtol=5e-2, atol=5e-3)
    assert all(np.isfinite(g.astype(np.float32)).all() for g in got[2:])
    assert new_pass("auto_parallel_fp16").default_dtype == "float16"


def test_planner_sees_through_segments():
    from paddle_b200.distributed.auto_parallel.static import Completer
    main, start, (h1, h2, pred, loss), pg = _program()
    plain = Completer(main, [2, 2]).annotate("x", [0, -1]).complete_forward_annotation()
    new_pass("auto_parallel_recompute", {"checkpoints": [h1, h2]}).apply([main], [start], PassContext())
    wrapped = Completer(main, [2, 2]).annotate("x", [0, -1]).complete_forward_annotation()
    assert [op.name for op in wrapped.dist_ops] == [op.name for op in plain.dist_ops]
    assert wrapped.get_tensor_dist_attr(h2).dims_mapping == [0, -1]


def test_gradient_merge_pass_updates_every_k_runs_with_the_mean_gradient():
    paddle.seed(4)
    paddle.enable_static()
    main, start = paddle.static.Program(), paddle.static.Program()
    with paddle.static.program_guard(main, start):
        x = paddle.static.data("x", [4, 8], "float32")
        y = paddle.static.data("y", [4, 1], "float32")
        lin = nn.Linear(8, 1)
        loss = F.mse_loss(lin(x), y)
        paddle.optimizer.SGD(learning_rate=0.1).minimize(loss)
    paddle.disable_static()
    new_pass("auto_parallel_gradient_merge", {"k_steps": 2, "avg": True}).apply([main], [start], PassContext())
    g = torch.Generator().manual_seed(0)
    batches = [(torch.randn(4, 8, generator=g), torch.randn(4, 1, generator=g)) for _ in range(2)]
    w0, b0 = torch.from_numpy(lin.weight.numpy().copy()), torch.from_numpy(lin.bias.numpy().copy())
    grads = []
    for xb, yb in batches:                                       # the gradients both runs see, at the unchanged weights
        w, b = w0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
        torch.nn.functional.mse_loss(xb @ w + b, yb).backward()
        grads.append((w.grad, b.grad))
    paddle.enable_static()
    exe = paddle.static.Executor()
    exe.run(main, feed={"x": batches[0][0].numpy(), "y": batches[0][1].numpy()}, fetch_list=[loss])
    assert torch.equal(torch.as_tensor(lin.weight.numpy()), w0)                 # nothing moves on the first run
    exe.run(main, feed={"x": batches[1][0].numpy(), "y": batches[1][1].numpy()}, fetch_list=[loss])
    want_w = w0 - 0.1 * (grads[0][0] + grads[1][0]) / 2
    want_b = b0 - 0.1 * (grads[0][1] + grads[1][1]) / 2
    np.testing.assert_allclose(lin.weight.numpy(), want_w.numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(lin.bias.numpy(), want_b.numpy(), rtol=1e-5, atol=1e-6)
