"""Alias of ``language_model_saes_b200`` under the import name used by code written for the reference project:
every public name, and every submodule (``<alias>.models.sae`` etc.), resolves to the same objects."""

import importlib
import sys

import language_model_saes_b200 as _impl
from language_model_saes_b200 import *  # noqa: F401,F403
from language_model_saes_b200 import __all__, __version__  # noqa: F401


class _AliasFinder:
    """Resolve ``<alias>.x.y`` to ``language_model_saes_b200.x.y`` (the very same module object)."""

    prefix = __name__ + "."
    _real: dict = {}

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(self.prefix):
            return None
        real = _impl.__name__ + "." + fullname[len(self.prefix):]
        try:
            module = importlib.import_module(real)
        except ImportError:
            return None
        from importlib.machinery import ModuleSpec

        # the import system stamps the spec it was given onto the module it gets back: remember the real one
        self._real[fullname] = (module, module.__spec__)
        return ModuleSpec(fullname, self, origin=getattr(module, "__file__", None))

    def create_module(self, spec):
        return self._real[spec.name][0]

    def exec_module(self, module):
        for name, (mod, real_spec) in list(self._real.items()):
            if mod is module:
                module.__spec__ = real_spec
                del self._real[name]


sys.meta_path.insert(0, _AliasFinder())
