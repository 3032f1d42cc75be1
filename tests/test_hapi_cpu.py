"""High-level API: callback protocol and default callback set, progress bar, accumulation, AMP configuration,
early stopping / plateau decay / checkpoints, predict, save / load with mismatch skipping, summary and flops tables
(reference behaviour: python/paddle/hapi/, test/legacy_test/test_model.py, test_callbacks.py)."""
import io
import json
import os

import numpy as np
import pytest

import paddle_b200 as paddle
from paddle_b200.hapi.callbacks import config_callbacks
from paddle_b200.hapi.progressbar import ProgressBar


def _data(n=64, seed=0):
    x = np.random.RandomState(seed).randn(n, 4).astype(np.float32)
    y = (x.sum(1) > 0).astype(np.int64)
    return paddle.io.TensorDataset([paddle.to_tensor(x), paddle.to_tensor(y)])


def _net():
    paddle.seed(1)
    return paddle.nn.Sequential(paddle.nn.Linear(4, 16), paddle.nn.ReLU(), paddle.nn.Linear(16, 2))


class Recorder(paddle.callbacks.Callback):
    def __init__(self):
        super().__init__()
        self.calls = []

    def __getattribute__(self, name):
        if name.startswith("on_"):
            def rec(*a, **k):
                object.__getattribute__(self, "calls").append(name)
            return rec
        return object.__getattribute__(self, name)


def test_fit_callback_protocol_and_defaults(tmp_path, capsys):
    net = _net()
    m = paddle.Model(net)
    m.prepare(paddle.optimizer.Adam(0.05, parameters=net.parameters()), paddle.nn.CrossEntropyLoss(), paddle.metric.Accuracy())
    rec = Recorder()
    m.fit(_data(), _data(32, 1), batch_size=16, epochs=2, verbose=2, log_freq=2, save_dir=str(tmp_path / "ck"), callbacks=[rec])
    out = capsys.readouterr().out
    assert "Epoch 1/2" in out and "step 2/4 - loss:" in out and "acc:" in out and "Eval begin..." in out and "Eval samples: 32" in out
    c = rec.calls
    assert c[0] == "on_train_begin" and c[-1] == "on_train_end" and c.count("on_epoch_begin") == 2
    assert c.count("on_train_batch_begin") == c.count("on_train_batch_end") == 8
    assert c.count("on_eval_begin") == c.count("on_eval_end") == 2 and c.count("on_eval_batch_end") == 4
    assert c.index("on_eval_begin") > c.index("on_epoch_end")
    assert sorted(os.listdir(tmp_path / "ck")) == ["0.pdopt", "0.pdparams", "1.pdopt", "1.pdparams", "final.pdopt", "final.pdparams"]
    res = m.evaluate(_data(32, 1), batch_size=16, verbose=0)
    assert set(res) == {"loss", "acc"} and isinstance(res["loss"], list)
    lst = config_callbacks(None, model=m, epochs=1, steps=3, verbose=0, save_dir=None)
    assert [type(x).__name__ for x in lst] == ["LRScheduler"] and lst.params["steps"] == 3
    lst = config_callbacks([paddle.callbacks.LRScheduler(by_step=False, by_epoch=True)], model=m, verbose=1, save_dir="x")
    assert [type(x).__name__ for x in lst] == ["ProgBarLogger", "LRScheduler", "ModelCheckpoint"]
    with pytest.raises(ValueError):
        paddle.callbacks.LRScheduler(by_step=True, by_epoch=True)


def test_accumulation_matches_large_batch_and_scheduler_steps_on_updates():
    ds = _data(32)
    results = []
    for bs, acc in ((16, 1), (4, 4)):
        net = _net()
        sched = paddle.optimizer.lr.StepDecay(0.1, step_size=1, gamma=0.5)
        m = paddle.Model(net)
        m.prepare(paddle.optimizer.SGD(sched, parameters=net.parameters()), paddle.nn.CrossEntropyLoss())
        m.fit(ds, batch_size=bs, epochs=1, shuffle=False, verbose=0, accumulate_grad_batches=acc)
        results.append((np.concatenate([p.numpy().ravel() for p in net.parameters()]), sched.last_epoch))
    assert np.allclose(results[0][0], results[1][0], atol=1e-5)            # 2 updates of 16 samples either way
    assert results[0][1] == results[1][1] == 2                             # the scheduler stepped once per update


def test_amp_configs_and_errors():
    net = _net()
    m = paddle.Model(net)
    opt = paddle.optimizer.Adam(0.05, parameters=net.parameters())
    m.prepare(opt, paddle.nn.CrossEntropyLoss(), amp_configs={"level": "O1", "dtype": "bfloat16", "custom_white_list": {"matmul"}})
    assert m._amp_level == "O1" and m._scaler is None
    m.fit(_data(), batch_size=16, epochs=3, verbose=0)
    assert m.evaluate(_data(), batch_size=16, verbose=0)["loss"][0] < 0.69
    m.prepare(opt, paddle.nn.CrossEntropyLoss(), amp_configs={"level": "O1", "init_loss_scaling": 128.0})
    assert m._scaler is not None
    with pytest.raises(ValueError):
        m.prepare(opt, paddle.nn.CrossEntropyLoss(), amp_configs={"level": "O3"})
    with pytest.raises(ValueError):
        m.prepare(opt, paddle.nn.CrossEntropyLoss(), amp_configs={"level": "O1", "loss_scale": 2})
    with pytest.raises(TypeError):
        m.prepare(opt, paddle.nn.CrossEntropyLoss(), metrics=[object()])
    with pytest.raises(TypeError):
        m.prepare(opt, loss=3)


def test_early_stopping_plateau_and_scalar_log(tmp_path):
    net = _net()
    m = paddle.Model(net)
    opt = paddle.optimizer.SGD(0.0, parameters=net.parameters())             # nothing improves
    m.prepare(opt, paddle.nn.CrossEntropyLoss(), paddle.metric.Accuracy())
    rec = Recorder()
    es = paddle.callbacks.EarlyStopping(monitor="loss", patience=1, verbose=0, save_best_model=True)
    m.fit(_data(), _data(16, 2), batch_size=32, epochs=10, verbose=0, save_dir=str(tmp_path / "es"),
          callbacks=[es, rec, paddle.callbacks.VisualDL(str(tmp_path / "vdl"))])
    assert rec.calls.count("on_epoch_begin") == 3 and m.stop_training            # best at eval 1, waits 2 > patience 1
    assert os.path.exists(tmp_path / "es" / "best_model.pdparams")
    rows = [json.loads(l) for l in open(tmp_path / "vdl" / "scalars.jsonl")]
    assert sum(r["mode"] == "train" for r in rows) == 6 and sum(r["mode"] == "eval" for r in rows) == 3 and "acc" in rows[0]
    opt.set_lr(1.0)
    red = paddle.callbacks.ReduceLROnPlateau(monitor="loss", factor=0.5, patience=2, verbose=0, min_lr=0.2)
    red.set_model(m)
    red.on_train_begin()
    for v in (1.0, 1.0, 1.0, 1.0, 1.0, 1.0):
        red.on_eval_end({"loss": [v]})
    assert opt.get_lr() == 0.25                                                   # halved after evaluations 3 and 5
    red.on_eval_end({"loss": [1.0]})
    red.on_eval_end({"loss": [1.0]})
    assert opt.get_lr() == 0.2                                                    # the floor
    with pytest.raises(ValueError):
        paddle.callbacks.ReduceLROnPlateau(factor=1.5)


def test_predict_save_load_and_skip_mismatch(tmp_path):
    net = _net()
    m = paddle.Model(net, inputs=[paddle.static.InputSpec([None, 4], "float32", "x")])
    m.prepare(paddle.optimizer.Adam(0.05, parameters=net.parameters()), paddle.nn.CrossEntropyLoss())
    ds = _data(20)
    rec = Recorder()
    out = m.predict(ds, batch_size=8, stack_outputs=True, verbose=0, callbacks=[rec])
    assert len(out) == 1 and out[0].shape == (20, 2) and rec.calls.count("on_predict_batch_end") == 3
    assert len(m.predict(ds, batch_size=8, verbose=0)[0]) == 3
    m.save(str(tmp_path / "a" / "model"))
    net2 = paddle.nn.Sequential(paddle.nn.Linear(4, 16), paddle.nn.ReLU(), paddle.nn.Linear(16, 3))
    m2 = paddle.Model(net2)
    with pytest.warns(UserWarning, match="skip loading"):
        m2.load(str(tmp_path / "a" / "model"), skip_mismatch=True)
    assert np.allclose(net2[0].weight.numpy(), net[0].weight.numpy()) and net2[2].weight.shape[1] == 3
    m3 = paddle.Model(_net())
    m3.prepare(paddle.optimizer.Adam(0.05, parameters=m3.network.parameters()), paddle.nn.CrossEntropyLoss())
    m3.load(str(tmp_path / "a" / "model.pdparams"))
    assert np.allclose(m3.predict(ds, batch_size=20, stack_outputs=True, verbose=0)[0], out[0], atol=1e-6)


def test_progress_bar_summary_and_flops(capsys):
    buf = io.StringIO()
    bar = ProgressBar(num=4, verbose=1, file=buf, name="step")
    for i in range(4):
        bar.update(i + 1, [("loss", 0.5 / (i + 1)), ("acc", [0.25, 0.5])])
    lines = buf.getvalue().strip().split("\n")
    assert len(lines) == 4 and lines[0].startswith("step 1/4 [") and "ETA" in lines[0] and "ETA" not in lines[-1]
    assert "loss: 0.1250" in lines[-1] and "acc: 0.2500 0.5000" in lines[-1] and "==]" in lines[-1]
    buf = io.StringIO()
    ProgressBar(num=None, verbose=2, file=buf).update(3, [("loss", 1e-5)])
    assert buf.getvalue().startswith("step 3 - loss: 1.0000e-05")

    lenet = paddle.nn.Sequential(paddle.nn.Conv2D(1, 6, 3, stride=1, padding=1), paddle.nn.ReLU(), paddle.nn.MaxPool2D(2, 2),
                                 paddle.nn.Conv2D(6, 16, 5, stride=1, padding=0), paddle.nn.ReLU(), paddle.nn.MaxPool2D(2, 2),
                                 paddle.nn.Flatten(), paddle.nn.Linear(400, 120), paddle.nn.Linear(120, 84), paddle.nn.Linear(84, 10))
    info = paddle.summary(lenet, (1, 1, 28, 28))
    text = capsys.readouterr().out
    assert info == {"total_params": 61610, "trainable_params": 61610}
    assert "Conv2D-1" in text and "[1, 6, 28, 28]" in text and "Linear-10" in text and "Total params: 61,610" in text
    assert "Estimated Total Size (MB)" in text
    info = paddle.summary(lenet, input=paddle.zeros([2, 1, 28, 28]))
    assert info["total_params"] == 61610
    # multiply-accumulates: conv1 28*28*6*(9+1), conv2 10*10*16*(150+1), linears 400*120 + 120*84 + 84*10
    want = 28 * 28 * 6 * 10 + 10 * 10 * 16 * 151 + 400 * 120 + 120 * 84 + 84 * 10
    assert paddle.flops(lenet, [1, 1, 28, 28], print_detail=True) == want
    text = capsys.readouterr().out
    assert "Layer Name" in text and f"Total Flops: {want}" in text
    assert paddle.flops(lenet, [1, 1, 28, 28], custom_ops={paddle.nn.ReLU: lambda l, x, y: int(np.prod(y.shape))}) > want
    assert paddle.Model(lenet, inputs=[paddle.static.InputSpec([None, 1, 28, 28], "float32")]).summary()["total_params"] == 61610
