"""Read a settings file into a dict: ``.json``, ``.yaml`` / ``.yml``, ``.toml``, or a ``.py`` file that defines
``config`` (cli/utils.py of the reference project)."""

from __future__ import annotations

import importlib.util
import json
import tomllib
from pathlib import Path
from typing import Any

import typer
import yaml


def load_config(config_file: str | Path) -> dict[str, Any]:
    path = Path(config_file)
    if not path.exists():
        raise typer.BadParameter(f"Configuration file not found: {config_file}")
    suffix = path.suffix
    if suffix == ".json":
        return json.loads(path.read_text())
    if suffix in {".yaml", ".yml"}:
        return yaml.safe_load(path.read_text())
    if suffix == ".toml":
        return tomllib.loads(path.read_text())
    if suffix == ".py":
        spec = importlib.util.spec_from_file_location("__lm_sae_config__", path)
        if spec is None or spec.loader is None:
            raise typer.BadParameter(f"Failed to load configuration file: {config_file}")
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        if not hasattr(module, "config"):
            raise typer.BadParameter(f"{config_file} does not define `config`")
        return module.config
    raise typer.BadParameter(f"Unsupported configuration file format: {suffix}. Supported formats: .json, .yaml, .yml, .toml, .py")
