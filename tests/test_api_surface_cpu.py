"""Every public name of the reference's Python packages (their ``__all__`` lists, stored in ``api_surface.json``)
must resolve in the corresponding ``paddle_b200`` module."""
import importlib
import json
import os

import pytest

with open(os.path.join(os.path.dirname(__file__), "api_surface.json")) as f:
    SURFACE = json.load(f)


@pytest.mark.parametrize("module", sorted(SURFACE))
def test_module_exports(module):
    mod = importlib.import_module("paddle_b200" + ("." + module if module else ""))
    missing = []
    for name in SURFACE[module]:
        try:
            getattr(mod, name)
        except Exception:
            missing.append(name)
    assert not missing, f"paddle.{module} lacks: {missing}"
