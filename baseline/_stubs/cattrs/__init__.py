"""Stand-in: converters are constructed at import time by the reference but never used by the benchmark arm."""
from . import gen, strategies  # noqa: F401


class Converter:
    def __init__(self, *a, **k):
        pass

    def register_structure_hook(self, *a, **k):
        pass

    def register_unstructure_hook(self, *a, **k):
        pass

    def register_structure_hook_func(self, *a, **k):
        pass

    def register_unstructure_hook_func(self, *a, **k):
        pass

    def register_structure_hook_factory(self, *a, **k):
        return lambda f: f

    def register_unstructure_hook_factory(self, *a, **k):
        return lambda f: f

    def structure(self, obj, cl):
        raise RuntimeError("cattrs is not installed")

    def unstructure(self, obj, *a, **k):
        raise RuntimeError("cattrs is not installed")

    def copy(self):
        return self


BaseConverter = Converter


def structure(obj, cl):
    raise RuntimeError("cattrs is not installed")


def unstructure(obj, *a, **k):
    raise RuntimeError("cattrs is not installed")
