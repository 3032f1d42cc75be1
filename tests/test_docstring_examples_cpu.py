"""The worked examples in the reference's docstrings, run against this package (``tests/docstring_harness.py``).

Each example block is executed with ``paddle`` bound to this package and what it prints is compared with the printed
results in the docstring: numbers with a tolerance, the remaining text (shape, dtype, layout of the print-out)
literally.  Blocks that need a GPU, the network, distributed launch, static-graph mode or the reference's own random
stream are skipped by the harness.  The floor per group is set just under the pass count at the time of writing, so a
regression in semantics or in the printed form of tensors fails here.  The examples are read from the reference's
source tree; without it the test skips."""
import glob
import os

import pytest

# the reference's source tree: $PADDLE_REFERENCE_ROOT, else a directory named ``reference`` beside this repository
_ROOT = os.environ.get("PADDLE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
REF = os.path.join(_ROOT, "python", "paddle")
pytestmark = pytest.mark.skipif(not os.path.isdir(REF), reason="the reference source tree is not present")

GROUPS = {
    # group: (file globs relative to the reference's python/paddle, minimum passing blocks, maximum failing + erroring blocks)
    "tensor": (["tensor/*.py"], 338, 4),
    "nn_functional": (["nn/functional/*.py"], 115, 5),
    "nn_layer": (["nn/layer/*.py"], 164, 4),
    "optimizer_autograd_amp": (["optimizer/*.py", "autograd/*.py", "amp/*.py", "metric/*.py", "framework/*.py", "fft.py", "signal.py",
                                "regularizer.py", "io/dataloader/*.py"], 143, 4),
    "sparse_quant_init": (["sparse/*.py", "sparse/nn/functional/*.py", "sparse/nn/layer/*.py", "quantization/*.py", "nn/initializer/*.py",
                          "nn/utils/*.py", "nn/clip.py", "nn/decode.py"], 82, 8),
    "incubate_vision_hapi_misc": (["incubate/asp/*.py", "incubate/optimizer/*.py", "incubate/autograd/*.py", "incubate/nn/layer/*.py",
                                  "incubate/tensor/*.py", "incubate/operators/*.py", "reader/*.py", "hapi/*.py", "vision/ops.py",
                                  "vision/transforms/*.py", "base/dygraph/base.py", "base/dygraph/tensor_patch_methods.py", "utils/*.py", "device/__init__.py", "profiler/*.py"],
                                 130, 16),
    # single-process examples of the distributed package (strategy objects, meshes, role makers)
    "distributed_single_process": (["distributed/fleet/base/distributed_strategy.py", "distributed/auto_parallel/process_mesh.py",
                                   "distributed/fleet/base/role_maker.py"], 47, 6, ("distributed",)),
    "distribution_audio_geometric_text": (["distribution/*.py", "audio/*/*.py", "geometric/*.py", "geometric/*/*.py", "text/*.py"], 86, 8),
}


@pytest.mark.timeout(900)
@pytest.mark.parametrize("group", sorted(GROUPS))
def test_reference_docstring_examples(group):
    import paddle
    from docstring_harness import run_file
    patterns, min_pass, max_bad, *rest = GROUPS[group]
    allow = rest[0] if rest else ()
    files = sorted(f for p in patterns for f in glob.glob(os.path.join(REF, p)))
    assert files
    passed, bad = 0, []
    for f in files:
        res = run_file(f, paddle, allow=allow)
        passed += len(res["pass"])
        bad += [(os.path.relpath(f, REF), name, detail.splitlines()[0] if detail else "") for name, detail in
                res["fail"] + res["error"] + res["timeout"]]
    summary = "\n".join(f"{f}::{n}: {d}" for f, n, d in bad)
    assert passed >= min_pass, f"{group}: only {passed} example blocks pass (floor {min_pass})\n{summary}"
    assert len(bad) <= max_bad, f"{group}: {len(bad)} example blocks fail (ceiling {max_bad})\n{summary}"


def test_harness_comparator():
    from docstring_harness import outputs_match
    want = "Tensor(shape=[2], dtype=float32, place=Place(gpu:0), stop_gradient=False,\n[1.50000000, 2.        ])"
    got = "Tensor(shape=[2], dtype=float32, place=Place(cpu), stop_gradient=True,\n       [1.50000012, 2.        ])"
    assert outputs_match(want, got)
    assert not outputs_match(want, got.replace("float32", "float64"))
    assert not outputs_match(want, got.replace("1.50000012", "1.60000000"))
    assert not outputs_match(want, got.replace("shape=[2]", "shape=[1, 2]"))
    assert outputs_match("[nan, inf]", "[nan, inf]") and not outputs_match("[1., inf]", "[1., -inf]")
