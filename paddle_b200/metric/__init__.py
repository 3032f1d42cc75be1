"""``paddle.metric`` (python/paddle/metric/metrics.py)."""
from __future__ import annotations

import numpy as np
import torch


class Metric:
    def reset(self):
        raise NotImplementedError

    def update(self, *a):
        raise NotImplementedError

    def accumulate(self):
        raise NotImplementedError

    def name(self):
        return self._name

    def compute(self, *args):
        return args


class Accuracy(Metric):
    def __init__(self, topk=(1,), name=None):
        self.topk = (topk,) if isinstance(topk, int) else tuple(topk)
        self.maxk = max(self.topk)
        self._name = [name or "acc"] if len(self.topk) == 1 else [f"{name or 'acc'}_top{k}" for k in self.topk]
        self.reset()

    def compute(self, pred, label, *args):
        idx = torch.topk(pred, self.maxk, dim=-1).indices
        label = label.reshape(-1, 1) if label.dim() == 1 or label.shape[-1] == 1 else label.argmax(-1, keepdim=True)
        return (idx == label.reshape(-1, 1)).float()

    def update(self, correct, *args):
        c = correct.detach().cpu().numpy() if isinstance(correct, torch.Tensor) else np.asarray(correct)
        res = []
        for i, k in enumerate(self.topk):
            n = c[:, :k].sum()
            self.total[i] += n
            self.count[i] += c.shape[0]
            res.append(float(n) / max(c.shape[0], 1))
        return res[0] if len(res) == 1 else res

    def reset(self):
        self.total = [0.0] * len(self.topk)
        self.count = [0] * len(self.topk)

    def accumulate(self):
        r = [t / c if c else 0.0 for t, c in zip(self.total, self.count)]
        return r[0] if len(r) == 1 else r


class Precision(Metric):
    def __init__(self, name="precision"):
        self._name = name
        self.reset()

    def update(self, preds, labels):
        p = (np.asarray(preds.cpu() if isinstance(preds, torch.Tensor) else preds).reshape(-1) > 0.5)
        l = np.asarray(labels.cpu() if isinstance(labels, torch.Tensor) else labels).reshape(-1).astype(bool)
        self.tp += int((p & l).sum())
        self.fp += int((p & ~l).sum())

    def reset(self):
        self.tp = self.fp = 0

    def accumulate(self):
        return self.tp / (self.tp + self.fp) if (self.tp + self.fp) else 0.0


class Recall(Precision):
    def __init__(self, name="recall"):
        self._name = name
        self.reset()

    def update(self, preds, labels):
        p = (np.asarray(preds.cpu() if isinstance(preds, torch.Tensor) else preds).reshape(-1) > 0.5)
        l = np.asarray(labels.cpu() if isinstance(labels, torch.Tensor) else labels).reshape(-1).astype(bool)
        self.tp += int((p & l).sum())
        self.fn += int((~p & l).sum())

    def reset(self):
        self.tp = self.fn = 0

    def accumulate(self):
        return self.tp / (self.tp + self.fn) if (self.tp + self.fn) else 0.0


class Auc(Metric):
    def __init__(self, curve="ROC", num_thresholds=4095, name="auc"):
        self._name, self.n = name, num_thresholds
        self.reset()

    def update(self, preds, labels):
        p = np.asarray(preds.cpu() if isinstance(preds, torch.Tensor) else preds)
        p = p[:, 1] if p.ndim == 2 and p.shape[1] == 2 else p.reshape(-1)
        l = np.asarray(labels.cpu() if isinstance(labels, torch.Tensor) else labels).reshape(-1)
        b = np.clip((p * self.n).astype(int), 0, self.n)
        np.add.at(self.pos, b[l == 1], 1)
        np.add.at(self.neg, b[l == 0], 1)

    def reset(self):
        self.pos = np.zeros(self.n + 1)
        self.neg = np.zeros(self.n + 1)

    def accumulate(self):
        tp = np.cumsum(self.pos[::-1])
        fp = np.cumsum(self.neg[::-1])
        if tp[-1] == 0 or fp[-1] == 0:
            return 0.0
        return float(np.trapz(tp / tp[-1], fp / fp[-1]))


def accuracy(input, label, k=1, correct=None, total=None, name=None):
    idx = torch.topk(input, k, dim=-1).indices
    return (idx == label.reshape(-1, 1)).any(-1).float().mean()
