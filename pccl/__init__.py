"""Drop-in names of the reference project: ``import pccl.lang`` / ``import pccl.engine`` resolve to
the B200-native implementation in ``pccl_b200``, and so does every other ``pccl.<module>`` that
exists there (``pccl.synth``, ``pccl.ops.collectives``, ``pccl.engine.elastic``, ...)."""
import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import os
import sys

from pccl_b200 import lang, engine  # noqa: F401

__version__ = "0.1.0"
_HERE = os.path.dirname(os.path.abspath(__file__))


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """First in ``sys.meta_path`` (a path finder would otherwise load a second copy of a file through an aliased
    package's search path): a ``pccl.x.y`` that has no file of its own under this package is the module
    ``pccl_b200.x.y`` itself, the same object."""

    @staticmethod
    def _real(fullname: str) -> str:
        return "pccl_b200." + fullname[len("pccl."):]

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith("pccl."):
            return None
        rel = os.path.join(_HERE, *fullname.split(".")[1:])
        if os.path.isfile(rel + ".py") or os.path.isfile(os.path.join(rel, "__init__.py")):
            return None                                   # this package's own module (the reference's file names)
        try:
            real = importlib.util.find_spec(self._real(fullname))
        except (ImportError, ValueError):
            return None
        if real is None:
            return None
        return importlib.machinery.ModuleSpec(fullname, self, is_package=real.submodule_search_locations is not None)

    _own_spec = {}

    def create_module(self, spec):
        module = importlib.import_module(self._real(spec.name))
        self._own_spec[spec.name] = module.__spec__       # the import machinery is about to overwrite it with the alias's
        return module

    def exec_module(self, module):
        module.__spec__ = self._own_spec.pop(module.__spec__.name, module.__spec__)


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
