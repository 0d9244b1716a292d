"""``lmms_engine`` is the import name users of the reference know
(``python -m lmms_engine.launch.cli``, ``python -m lmms_engine.merger``).  Every submodule
resolves to the same module object as its ``lmms_engine_b200`` counterpart, so registries
and global state are shared whichever name is used."""
import importlib
import importlib.abc
import importlib.util
import sys

import lmms_engine_b200 as _impl

_PREFIX = __name__ + "."


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = "lmms_engine_b200." + fullname[len(_PREFIX):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        return importlib.util.spec_from_loader(fullname, self, is_package=True)

    def create_module(self, spec):
        real = "lmms_engine_b200." + spec.name[len(_PREFIX):]
        return importlib.import_module(real)

    def exec_module(self, module):
        return None


sys.meta_path.insert(0, _AliasFinder())
__version__ = _impl.__version__
