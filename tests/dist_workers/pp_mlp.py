"""Pipeline parallel vs single-rank twin (pattern of test/collective/fleet/hybrid_parallel_pp_layer.py and
hybrid_parallel_shared_weight.py): the same stack of layers, built from one seed, trained for three steps
with 1F1B (argv[1] == "1f1b"), interleaved virtual stages ("vpp"), the zero-bubble H1 order ("zbh1") or the zero-bubble V
schedule over a zigzag placement ("zbvpp"); dumps per-step losses of
both and the final parameters of this stage next to the twin's."""
import os
import sys

import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200 import nn
from paddle_b200.distributed import fleet
from paddle_b200.distributed.fleet.meta_parallel import LayerDesc, PipelineLayer, SharedLayerDesc

mode = sys.argv[1] if len(sys.argv) > 1 else "1f1b"
n = int(os.environ["PADDLE_TRAINERS_NUM"])
H, VOC, MB, ACC = 16, 32, 2, 4
strategy = fleet.DistributedStrategy()
strategy.hybrid_configs = {"dp_degree": 1, "mp_degree": 1, "pp_degree": n}
strategy.pipeline_configs = {"accumulate_steps": ACC, "micro_batch_size": MB}
if mode == "zbh1":          # zero-bubble H1: weight gradients of the first backwards are postponed to the end
    strategy.pipeline_configs["schedule_mode"] = "ZBH1"
if mode == "zbvpp":         # zero-bubble V: two chunks per rank in zigzag placement, Bx / W split
    strategy.pipeline_configs["schedule_mode"] = "ZBVPP"
fleet.init(is_collective=True, strategy=strategy)
rank = dist.get_rank()


class Emb(nn.Layer):
    def __init__(self):
        super().__init__()
        self.weight = self.create_parameter([VOC, H])

    def forward(self, ids):
        return paddle.nn.functional.embedding(ids, self.weight)


def head(layer, x):
    return paddle.matmul(x, layer.weight, transpose_y=True)


class Block(nn.Layer):
    def __init__(self):
        super().__init__()
        self.fc = nn.Linear(H, H)

    def forward(self, x):
        return x + paddle.tanh(self.fc(x))


def loss_fn(logits, labels):
    return paddle.nn.functional.cross_entropy(logits.reshape([-1, VOC]), labels.reshape([-1]))


descs = [SharedLayerDesc("emb", Emb)] + [LayerDesc(Block) for _ in range(6)] + [SharedLayerDesc("emb", Emb, forward_func=head)]
V = 2 if mode in ("vpp", "zbvpp") else None
placement = "zigzag" if mode == "zbvpp" else "interleaved"
paddle.seed(11)
# twin: all layers on this rank, built in description order from the same seed
twin_layers = []
shared = {}
for d in descs:
    if isinstance(d, SharedLayerDesc):
        if d.layer_name not in shared:
            shared[d.layer_name] = d.build_layer()
        twin_layers.append((shared[d.layer_name], d.forward_func))
    else:
        twin_layers.append((d.build_layer(), None))
pipe = PipelineLayer(descs, loss_fn=loss_fn, num_virtual_pipeline_stages=V, virtual_placement=placement)
# copy the twin's weights into the stage-local layers
parts = pipe.segment_parts
with torch.no_grad():
    if V:
        for c, chunk in enumerate(pipe.get_model_chunks()):
            lo = parts[c * n + (rank if (placement == "interleaved" or c % 2 == 0) else n - 1 - rank)]
            for i, f in enumerate(chunk.run_function):
                src = twin_layers[lo + i][0]
                if isinstance(f, nn.Layer):
                    for (k, p), (_, q) in zip(f.state_dict().items(), src.state_dict().items()):
                        p.copy_(q)
    else:
        for i, f in enumerate(pipe.run_function):
            if isinstance(f, nn.Layer):
                for (k, p), (_, q) in zip(f.state_dict().items(), twin_layers[parts[rank] + i][0].state_dict().items()):
                    p.copy_(q)
    for key, l in pipe.shared_layers.items():
        l.weight.copy_(shared[key].weight)

twin_params = []
seen = set()
for l, _ in twin_layers:
    for p in l.parameters():
        if id(p) not in seen:
            seen.add(id(p)); twin_params.append(p)
opt_t = paddle.optimizer.SGD(0.1, parameters=twin_params)
opt_p = paddle.optimizer.SGD(0.1, parameters=pipe.parameters())
model = fleet.distributed_model(pipe)
opt_p = fleet.distributed_optimizer(opt_p)
gen = torch.Generator().manual_seed(5)
lt, lp = [], []
for step in range(3):
    ids = torch.randint(0, VOC, (MB * ACC, 8), generator=gen)
    lab = torch.randint(0, VOC, (MB * ACC, 8), generator=gen)
    x = paddle.to_tensor(ids.numpy())
    for l, f in twin_layers:
        x = f(l, x) if f is not None else l(x)
    a = loss_fn(x, paddle.to_tensor(lab.numpy()))
    a.backward(); opt_t.step(); opt_t.clear_grad(); lt.append(float(a))
    b = model.train_batch((paddle.to_tensor(ids.numpy()), paddle.to_tensor(lab.numpy())), opt_p)
    lp.append(float(b))
ev = float(model.eval_batch((paddle.to_tensor(ids.numpy()), paddle.to_tensor(lab.numpy())), compute_loss=True))
maxdiff = 0.0
for key, l in pipe.shared_layers.items():
    maxdiff = max(maxdiff, float((l.weight - shared[key].weight).abs().max()))
if not V:
    for i, f in enumerate(pipe.run_function):
        if isinstance(f, nn.Layer):
            for (k, p), (_, q) in zip(f.state_dict().items(), twin_layers[parts[rank] + i][0].state_dict().items()):
                maxdiff = max(maxdiff, float((p - q).abs().max()))
_common.dump({"twin": lt, "pipe": lp, "maxdiff": maxdiff, "eval": ev, "parts": parts, "wrapper": type(model).__name__})
