"""Run scripts written against the reference's package name unchanged.

    import flextrain_b200.compat          # once, before the script's own imports
    import flextrain
    from flextrain.config import init_flextrain_config
    from flextrain.ops.adam import FlexTrainAdam

Importing this module installs a finder that resolves ``flextrain`` and every
``flextrain.<sub>`` to the module of the same path in this package (the very same
module objects, so singletons such as the config are shared).  Nothing is installed
unless this module is imported, and a real ``flextrain`` that is already imported is
left alone.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

_ALIAS, _TARGET = "flextrain", "flextrain_b200"


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self._target = target

    def create_module(self, spec):
        return importlib.import_module(self._target)

    def exec_module(self, module):          # already executed under its own name
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if fullname != _ALIAS and not fullname.startswith(_ALIAS + "."):
            return None
        real = _TARGET + fullname[len(_ALIAS):]
        try:
            found = importlib.util.find_spec(real)
        except ModuleNotFoundError:
            return None
        if found is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real),
                                               is_package=found.submodule_search_locations is not None)
        return spec


def install() -> bool:
    """Install the alias (idempotent).  False when a different ``flextrain`` is already loaded."""
    existing = sys.modules.get(_ALIAS)
    if existing is not None and getattr(existing, "__name__", "") != _TARGET:
        return False
    if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
        sys.meta_path.insert(0, _AliasFinder())
    return True


def uninstall():
    sys.meta_path[:] = [f for f in sys.meta_path if not isinstance(f, _AliasFinder)]
    for name in [n for n in sys.modules if n == _ALIAS or n.startswith(_ALIAS + ".")]:
        if getattr(sys.modules[name], "__name__", "").startswith(_TARGET):
            del sys.modules[name]


installed = install()
