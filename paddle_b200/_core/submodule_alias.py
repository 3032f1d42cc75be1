"""The reference splits some namespaces over many files (``paddle.nn.functional.loss``, ``paddle.nn.layer.conv`` ...)
that this package keeps in one module.  ``alias_submodules`` registers those dotted paths as thin module objects that
resolve every attribute in the module that really holds it, so imports and attribute paths written for the
reference's layout keep working."""
from __future__ import annotations

import sys
import types


def alias_submodules(parent_name, names):
    parent = sys.modules[parent_name]
    if not hasattr(parent, "__path__"):
        parent.__path__ = []          # lets ``import parent.child`` find the registered child in sys.modules
    for n in names:
        full = f"{parent_name}.{n}"
        if full in sys.modules or isinstance(getattr(parent, n, None), types.ModuleType):
            continue
        existing = getattr(parent, n, None)
        if existing is not None and callable(existing):
            # a function of the same name (``F.flash_attention``): give the function the parent's names as attributes
            for k in dir(parent):
                if not k.startswith("_") and not hasattr(existing, k):
                    try:
                        setattr(existing, k, getattr(parent, k))
                    except (AttributeError, TypeError):
                        pass
            continue
        mod = types.ModuleType(full, f"Alias of {parent_name} under the reference's file layout.")

        def _getattr(attr, _parent=parent, _full=full):
            try:
                return getattr(_parent, attr)
            except AttributeError:
                raise AttributeError(f"module {_full!r} has no attribute {attr!r}") from None
        mod.__getattr__ = _getattr
        mod.__dir__ = lambda _parent=parent: dir(_parent)
        sys.modules[full] = mod
        setattr(parent, n, mod)
