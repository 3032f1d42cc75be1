"""auto.Engine on 2 data-parallel ranks: fit with gradient merge, evaluate, save / load; dumps the loss history, a
checksum of the parameters (must agree between ranks: gradients are averaged) and the files written."""
import os
import sys

import _common
import numpy as np

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200 import nn
from paddle_b200.distributed import auto_parallel as auto
from paddle_b200.io import Dataset

dist.init_parallel_env()
rank = dist.get_rank()


class Toy(Dataset):
    def __init__(self, n):
        g = np.random.RandomState(0)
        self.x = g.randn(n, 8).astype("float32")
        self.y = (self.x @ g.randn(8, 3).astype("float32")).argmax(-1).astype("int64")

    def __len__(self):
        return len(self.x)

    def __getitem__(self, i):
        return self.x[i], self.y[i]


paddle.seed(1)
model = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 3))
strategy = auto.Strategy()
strategy.gradient_merge.enable = True
strategy.gradient_merge.k_steps = 2
engine = auto.Engine(model, nn.CrossEntropyLoss(), paddle.optimizer.Adam(0.05, parameters=model.parameters()),
                     metrics=paddle.metric.Accuracy(), strategy=strategy)
hist = engine.fit(Toy(64), batch_size=8, epochs=5, verbose=0)
ev = engine.evaluate(Toy(64), batch_size=8, verbose=0)
base = os.path.join(sys.argv[1], "ck")
engine.save(base)
before = float(sum(p.abs().sum() for p in model.parameters()))
for p in model.parameters():
    p.set_value(p * 0)
engine.load(base)
after = float(sum(p.abs().sum() for p in model.parameters()))
_common.dump({"first": hist["loss"][0], "last": hist["loss"][-1], "steps": len(hist["loss"]), "checksum": before,
              "restored": after, "eval": ev, "files": sorted(os.listdir(sys.argv[1]))})
