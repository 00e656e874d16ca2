"""``import rustorch``: the reference's package name, resolving to :mod:`rustorch_b200` (same objects).

``rustorch`` and every ``rustorch.<sub>`` name are aliases of the ``rustorch_b200`` modules themselves: a finder on
``sys.meta_path`` answers ``import rustorch.nn`` with the already imported ``rustorch_b200.nn`` object, so there is one
copy of every class whichever name it was imported through (two copies would make ``isinstance`` checks between
``rustorch.Variable`` and ``rustorch.nn`` layers fail)."""
import importlib
import importlib.abc
import importlib.machinery
import sys

import rustorch_b200 as _impl

_ALIAS, _REAL = __name__, _impl.__name__


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_ALIAS + "."):
            return None
        try:
            importlib.import_module(_REAL + fullname[len(_ALIAS):])
        except ImportError:
            return None
        return importlib.machinery.ModuleSpec(fullname, self)

    def create_module(self, spec):
        return sys.modules[_REAL + spec.name[len(_ALIAS):]]

    def exec_module(self, module):
        pass


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
for _name, _mod in list(sys.modules.items()):          # submodules that are loaded already
    if _name.startswith(_REAL + "."):
        sys.modules.setdefault(_ALIAS + _name[len(_REAL):], _mod)
sys.modules[__name__] = _impl
sys.modules.setdefault("_rustorch_py", _impl)            # the extension module's own name in the reference's wheel
