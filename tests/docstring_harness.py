"""Run the ``>>>`` examples of the reference's docstrings against this package.

The reference's Python sources carry thousands of worked examples with printed results.  Read as text they are a large
table of golden vectors: this harness extracts them (``doctest`` parser), runs each example block in a fresh namespace
where ``paddle`` is this package, and compares what it prints with what the docstring shows - numbers with a tolerance,
everything else literally after whitespace normalisation.  Blocks that need a GPU, a network, other hardware or
randomness that is tied to the reference's generator are classified as skipped, not failed."""
from __future__ import annotations

import contextlib
import doctest
import io
import math
import re
import signal
import traceback

_NUM = re.compile(r"[-+]?(?:\d+\.\d*|\.\d+|\d+)(?:[eE][-+]?\d+)?|[-+]?(?:inf|nan)\b")
_SKIP_DIRECTIVES = ("+SKIP", "+REQUIRES(env:GPU", "+REQUIRES(env: GPU", "+REQUIRES(env:XPU", "+REQUIRES(env:DISTRIBUTED", "+REQUIRES(env: DISTRIBUTED",
                    "+REQUIRES(env:CUSTOM", "+TIMEOUT", "+REQUIRES(env:CPU, env:GPU")
_RANDOM_HINTS = ("paddle.rand", "paddle.randn", "paddle.randint", "paddle.uniform", "paddle.normal", "paddle.randperm", "np.random", "random.",
                 "paddle.bernoulli", "paddle.multinomial", "paddle.poisson", "paddle.standard_normal", "paddle.empty", "dropout", "Dropout",
                 "paddle.seed", "sample(", "rsample(", "initializer", "nn.Linear", "nn.Conv", "nn.Embedding", "create_parameter", "nn.LSTM", "nn.GRU",
                 "nn.SimpleRNN", "nn.Bilinear", "nn.MultiHeadAttention", "nn.Transformer", "nn.LayerNorm", "nn.BatchNorm", "shuffle", "XavierUniform",
                 "paddle.binomial", "exponential_", "uniform_", "normal_", "bernoulli_", "cauchy_", "geometric_", "log_normal", "gumbel_softmax",
                 "rrelu", "RReLU", "nn.PReLU", "spectral_norm", "weight_norm", "paddle.standard_gamma", "paddle.vision.models", "nn.GroupNorm",
                 "nn.InstanceNorm", "nn.SpectralNorm", "fractional_max_pool", "FractionalMaxPool")


class _Timeout(Exception):
    pass


def extract_blocks(path):
    """[(qualified name, [doctest.Example])] - one entry per ``code-block`` of each docstring in the file."""
    import ast
    src = open(path, encoding="utf-8").read()
    tree = ast.parse(src)
    parser = doctest.DocTestParser()
    out = []

    def visit(node, prefix):
        for child in ast.iter_child_nodes(node):
            if isinstance(child, (ast.FunctionDef, ast.ClassDef, ast.AsyncFunctionDef)):
                name = f"{prefix}{child.name}"
                doc = ast.get_docstring(child, clean=True)
                if doc and ">>>" in doc:
                    chunks = re.split(r"\.\.\s+code-block::\s*python[^\n]*\n", doc)
                    for ci, chunk in enumerate(chunks[1:] if len(chunks) > 1 else chunks):
                        try:
                            ex = parser.get_examples(chunk)
                        except ValueError:
                            continue
                        if ex:
                            out.append((f"{name}#{ci}" if ci else name, ex))
                # methods of classes, and functions defined inside functions (the reference patches Tensor methods
                # from inside ``monkey_patch_tensor``)
                visit(child, name + ".")
    visit(tree, "")
    return out


def classify_skip(examples, allow=()):
    """Why a block is not run, or None.  ``allow`` lists categories to run anyway (``"static"``)."""
    text = "\n".join(e.source for e in examples)
    for d in _SKIP_DIRECTIVES:
        if d in text:
            return "directive"
    if "distributed" not in allow and ("paddle.distributed" in text or "fleet" in text or "dist." in text):
        return "distributed"
    if "static" not in allow and ("paddle.static" in text or "enable_static" in text or "static." in text or "paddle.base" in text
                                  or "fluid" in text):
        return "static"
    if "cuda" in text or "gpu" in text.lower() and "place" in text.lower():
        return "gpu"
    if "download" in text or "http" in text or "datasets." in text:
        return "network"
    return None


def uses_randomness(examples):
    text = "\n".join(e.source for e in examples)
    return any(h in text for h in _RANDOM_HINTS)


def _strip_meta(s):
    s = re.sub(r"Place\([^)]*\)", "Place()", s)
    return re.sub(r"stop_gradient=(True|False)", "stop_gradient=", s)


def _numbers(s):
    s = _strip_meta(s)
    out = []
    for m in _NUM.finditer(s):
        t = m.group(0).lower()
        try:
            out.append(float(t))
        except ValueError:
            pass
    return out


def _skeleton(s):
    s = _NUM.sub("#", _strip_meta(s))
    s = re.sub(r"\s+", "", s)
    s = s.replace("#.", "#").replace(",]", "]")
    return s


def outputs_match(want, got, rtol=2e-3, atol=2e-5):
    """Numbers are compared with a tolerance, the text around them after removing whitespace and device names."""
    if want.strip() == got.strip():
        return True
    w, g = _numbers(want), _numbers(got)
    if len(w) != len(g):
        return False
    for a, b in zip(w, g):
        if math.isnan(a) and math.isnan(b):
            continue
        if math.isinf(a) or math.isinf(b):
            if a != b:
                return False
            continue
        if abs(a - b) > atol + rtol * max(abs(a), abs(b)):
            return False
    return _skeleton(want) == _skeleton(got)


def _reset_global_state(paddle_module):
    """Examples switch global modes (grad mode, default dtype, print options, device, lazy init) and do not always
    switch them back; every block starts from the defaults."""
    import torch
    torch.set_grad_enabled(True)
    try:
        paddle_module.set_default_dtype("float32")
        paddle_module.set_printoptions(precision=8, threshold=1000, edgeitems=3, linewidth=80, sci_mode=False)
        paddle_module.set_device("cpu")
        paddle_module.disable_static()
    except Exception:  # noqa: BLE001
        pass


def run_block(examples, paddle_module, timeout_s=20, check_values=True):
    """-> ("pass" | "fail" | "error" | "timeout", detail)."""
    ns = {"paddle": paddle_module, "__name__": "__main__"}
    _reset_global_state(paddle_module)

    def on_alarm(signum, frame):
        raise _Timeout()
    old = signal.signal(signal.SIGALRM, on_alarm)
    signal.alarm(timeout_s)
    try:
        for ex in examples:
            src = ex.source
            if "doctest: +SKIP" in src:
                continue
            buf = io.StringIO()
            try:
                with contextlib.redirect_stdout(buf):
                    try:
                        code = compile(src, "<example>", "single")
                    except SyntaxError:
                        try:
                            code = compile(src, "<example>", "exec")
                        except SyntaxError:
                            return "skip", "the docstring's continuation lines do not parse"
                    exec(code, ns)                      # noqa: S102 - the examples are the test input
            except _Timeout:
                return "timeout", src.strip()
            except Exception as e:  # noqa: BLE001
                if ex.exc_msg is not None:
                    continue                             # the example documents an exception
                return "error", f"{src.strip()}\n  -> {type(e).__name__}: {e}\n{traceback.format_exc(limit=3)}"
            want = ex.want
            if check_values and want.strip() and "..." not in want and "doctest: +SKIP" not in want:
                got = buf.getvalue()
                if not outputs_match(want, got):
                    return "fail", f"{src.strip()}\n  want: {want.strip()[:400]}\n  got:  {got.strip()[:400]}"
        return "pass", ""
    finally:
        signal.alarm(0)
        signal.signal(signal.SIGALRM, old)


def run_file(path, paddle_module, only=None, allow=()):
    """-> {"pass": [...], "fail": [(name, detail)], "error": [...], "skip": [(name, why)]}."""
    res = {"pass": [], "fail": [], "error": [], "timeout": [], "skip": []}
    for name, examples in extract_blocks(path):
        if only and not any(o in name for o in only):
            continue
        why = classify_skip(examples, allow)
        if why:
            res["skip"].append((name, why))
            continue
        status, detail = run_block(examples, paddle_module, check_values=not uses_randomness(examples))
        if status == "pass":
            res["pass"].append(name)
        elif status == "skip":
            res["skip"].append((name, detail))
        else:
            res[status].append((name, detail))
    return res
