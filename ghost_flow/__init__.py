"""``ghost_flow``: the reference's package name, served by :mod:`ghost_flow_b200`.

``import ghost_flow as gf`` gives the same namespace, and every submodule is importable under the alias
(``import ghost_flow.models``, ``from ghost_flow.ml import RandomForestClassifier``): a finder on ``sys.meta_path``
resolves ``ghost_flow.x.y`` to the module object of ``ghost_flow_b200.x.y``, so both names share one module.
"""
import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys

import ghost_flow_b200 as _impl
from ghost_flow_b200 import *  # noqa: F401,F403
from ghost_flow_b200 import DType, Tensor, nn, optim, ops, __version__  # noqa: F401

_PREFIX, _REAL = __name__ + ".", _impl.__name__ + "."


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        try:
            real = importlib.util.find_spec(_REAL + fullname[len(_PREFIX):])
        except (ImportError, ValueError):
            return None
        if real is None:
            return None
        return importlib.machinery.ModuleSpec(fullname, self, is_package=real.submodule_search_locations is not None)

    def create_module(self, spec):
        return importlib.import_module(_REAL + spec.name[len(_PREFIX):])

    def exec_module(self, module):
        pass


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())


def __getattr__(name):
    return getattr(_impl, name)
