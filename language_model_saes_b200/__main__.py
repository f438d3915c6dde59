"""``python -m language_model_saes_b200 <command>``."""

from .cli import entrypoint

entrypoint()
