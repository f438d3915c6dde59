"""Stand-in for the parts of transformer_lens the reference imports at module level."""
from . import hook_points, utils  # noqa: F401


class HookedTransformer:  # placeholder type: language-model features are not used by the benchmark arm
    def __init__(self, *a, **k):
        raise RuntimeError("transformer_lens is not installed; only hook_points is provided by this stand-in")
