"""Domain libraries: vision ops against torchvision, models / transforms shapes, fft / signal / linalg / distribution /
sparse / geometric / text / audio / quantization semantics against plain formulas."""
import itertools

import numpy as np
import pytest
import torch

import paddle_b200 as paddle
from paddle_b200 import nn

tv = pytest.importorskip("torchvision")


def test_vision_ops_match_torchvision():
    from paddle_b200.vision import ops
    torch.manual_seed(0)
    b = torch.rand(20, 2) * 50
    boxes, sc = torch.cat([b, b + torch.rand(20, 2) * 30 + 1], 1), torch.rand(20)
    assert ops.nms(paddle.to_tensor(boxes.numpy()), 0.4, paddle.to_tensor(sc.numpy())).tolist() == tv.ops.nms(boxes, sc, 0.4).tolist()
    x = torch.randn(2, 4, 16, 16)
    rois = torch.tensor([[1., 2, 9, 12], [0, 0, 15, 15], [3, 3, 7, 9]])
    ra = ops.roi_align(paddle.to_tensor(x.numpy()), paddle.to_tensor(rois.numpy()),
                       paddle.to_tensor(np.array([2, 1], dtype=np.int32)), 4, 0.5, 2, True)
    assert float((ra - tv.ops.roi_align(x, [rois[:2], rois[2:]], 4, 0.5, 2, True)).abs().max()) < 1e-5
    rp = ops.roi_pool(paddle.to_tensor(x.numpy()), paddle.to_tensor(rois.numpy()),
                      paddle.to_tensor(np.array([2, 1], dtype=np.int32)), 3, 1.0)
    assert float((rp - tv.ops.roi_pool(x, [rois[:2], rois[2:]], 3, 1.0)).abs().max()) < 1e-5
    w, off, m = torch.randn(6, 4, 3, 3), torch.randn(2, 18, 16, 16) * 0.5, torch.rand(2, 9, 16, 16)
    dc = ops.deform_conv2d(paddle.to_tensor(x.numpy()), paddle.to_tensor(off.numpy()), paddle.to_tensor(w.numpy()),
                           padding=1, mask=paddle.to_tensor(m.numpy()))
    assert float((dc - tv.ops.deform_conv2d(x, off, w, padding=1, mask=m)).abs().max()) < 1e-4


def test_vision_models_and_transforms():
    from paddle_b200.vision import models, transforms as T
    x = paddle.randn([2, 3, 64, 64])
    assert models.resnet18(num_classes=10)(x).shape == [2, 10]
    assert models.mobilenet_v2(num_classes=5)(x).shape == [2, 5]
    assert models.LeNet()(paddle.randn([2, 1, 28, 28])).shape == [2, 10]
    assert sum(p.numel() for p in models.resnet50().parameters()) == 25557032
    with pytest.raises(RuntimeError):
        models.resnet18(pretrained=True)
    img = (np.random.rand(40, 60, 3) * 255).astype(np.uint8)
    out = T.Compose([T.Resize(32), T.CenterCrop(28), T.RandomHorizontalFlip(), T.ToTensor(),
                     T.Normalize([0.5] * 3, [0.5] * 3)])(img)
    assert out.shape == [3, 28, 28] and float(out.min()) >= -1.001 and float(out.max()) <= 1.001


def test_fft_signal_linalg():
    x = paddle.randn([4, 16])
    assert np.allclose(paddle.fft.fft(x).numpy(), np.fft.fft(x.numpy()), atol=1e-4)
    assert paddle.fft.rfft2(paddle.randn([4, 8])).shape == [4, 5]
    w = paddle.ones([16])
    s = paddle.signal.stft(paddle.randn([2, 64]), 16, window=w)
    assert s.shape == [2, 9, 17] and paddle.signal.istft(s, 16, window=w).shape == [2, 64]
    a = paddle.randn([4, 4])
    spd = a @ a.T + paddle.eye(4)
    L = paddle.linalg.cholesky(spd)
    assert np.allclose((L @ L.T).numpy(), spd.numpy(), atol=1e-4)
    assert np.allclose(paddle.linalg.det(spd).numpy(), np.linalg.det(spd.numpy()), rtol=1e-3)
    assert np.allclose((paddle.linalg.inv(spd) @ spd).numpy(), np.eye(4), atol=1e-3)


def test_distribution():
    from paddle_b200.distribution import AffineTransform, Categorical, Normal, TransformedDistribution, kl_divergence
    n = Normal(0.0, 1.0)
    assert abs(float(n.log_prob(paddle.to_tensor(0.0))) + 0.918938) < 1e-5 and n.sample([3]).shape == [3]
    assert abs(float(kl_divergence(Normal(0., 1.), Normal(1., 2.))) - 0.443147) < 1e-5
    c = Categorical(paddle.to_tensor([1., 2., 1.]))
    assert abs(float(c.entropy()) - 1.0397207) < 1e-5
    td = TransformedDistribution(Normal(0., 1.), [AffineTransform(paddle.to_tensor(1.), paddle.to_tensor(2.))])
    assert abs(float(td.log_prob(paddle.to_tensor(1.0))) + 1.612086) < 1e-4


def test_sparse_and_geometric():
    import paddle_b200.geometric as G
    import paddle_b200.sparse as sp
    s = sp.sparse_coo_tensor([[0, 1, 2], [1, 2, 0]], [1., 2., 3.], [3, 3])
    assert sp.matmul(s, paddle.ones([3, 2])).numpy().tolist() == [[1.0, 1.0], [2.0, 2.0], [3.0, 3.0]]
    assert sp.add(s, s).to_dense().sum().item() == 12.0 and sp.nn.functional.relu(sp.neg(s)).to_dense().sum().item() == 0
    x = paddle.to_tensor(np.array([[0., 2, 3], [1, 4, 5], [2, 6, 7]], dtype="float32"))
    out = G.send_u_recv(x, paddle.to_tensor([0, 1, 2, 0]), paddle.to_tensor([1, 2, 1, 0]), "sum")
    assert out.numpy().tolist() == [[0.0, 2.0, 3.0], [2.0, 8.0, 10.0], [1.0, 4.0, 5.0]]
    assert G.segment_mean(x, paddle.to_tensor([0, 0, 1])).numpy().tolist() == [[0.5, 3.0, 4.0], [2.0, 6.0, 7.0]]


def test_text_audio_quantization():
    from paddle_b200.audio import features
    from paddle_b200.quantization import QAT, FakeQuanterWithAbsMaxObserver, QuantConfig
    from paddle_b200.text import viterbi_decode
    pot, tr = paddle.randn([2, 5, 4]), paddle.randn([4, 4])
    _, p = viterbi_decode(pot, tr, paddle.to_tensor([5, 3]), False)
    best = max(itertools.product(range(4), repeat=5),
               key=lambda q: sum(float(pot[0, t, q[t]]) for t in range(5)) + sum(float(tr[q[t], q[t + 1]]) for t in range(4)))
    assert list(best) == p[0].tolist()
    assert features.MFCC(sr=16000, n_fft=256, n_mels=20, n_mfcc=8)(paddle.randn([2, 4000])).shape == [2, 8, 63]
    net = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 2))
    q = FakeQuanterWithAbsMaxObserver(moving_rate=0.9)
    qat = QAT(QuantConfig(activation=q, weight=q))
    qnet = qat.quantize(net)
    y = qnet(paddle.randn([4, 8]))
    y.sum().backward()
    assert type(qnet[0]).__name__ == "QuantedLayer" and qnet[0].inner.weight.grad is not None
    conv = qat.convert(qnet)
    assert type(conv[0]).__name__ == "Linear" and float(conv[0].weight_scale) > 0
