"""``import paddle`` alias: every ``paddle[.x.y]`` module IS the ``paddle_b200[.x.y]`` module object
(no second copy is executed), so user code and pickles that name ``paddle.*`` paths resolve here."""
import importlib
import importlib.abc
import importlib.machinery
import sys

import paddle_b200 as _real

_PREFIX, _REAL = "paddle", "paddle_b200"


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if fullname != _PREFIX and not fullname.startswith(_PREFIX + "."):
            return None
        real = _REAL + fullname[len(_PREFIX):]
        try:
            importlib.import_module(real)
        except ModuleNotFoundError as e:
            if e.name == real:
                return None
            raise
        return importlib.machinery.ModuleSpec(fullname, self, is_package=hasattr(sys.modules[real], "__path__"))

    def create_module(self, spec):
        return sys.modules[_REAL + spec.name[len(_PREFIX):]]

    def exec_module(self, module):
        pass


sys.meta_path.insert(0, _AliasFinder())
sys.modules[__name__] = _real
