"""Job commands: ``generate``, ``train``, ``analyze`` as in cli/run.py of the reference project, plus ``evaluate``,
``dla``, ``autointerp`` and ``convert`` for the remaining runners. ``train --kind`` / ``analyze --kind`` /
``evaluate --kind`` select the dictionary family."""

from __future__ import annotations

from enum import Enum
from pathlib import Path
from typing import Annotated

import typer

from .utils import load_config

app = typer.Typer()

ConfigArg = Annotated[Path, typer.Argument(help="Settings file (.json, .yaml, .toml or .py defining `config`).")]


class TrainKind(str, Enum):
    sae = "sae"
    crosscoder = "crosscoder"
    clt = "clt"
    lorsa = "lorsa"
    molt = "molt"
    sweep = "sweep"


class AnalyzeKind(str, Enum):
    sae = "sae"
    crosscoder = "crosscoder"


@app.command("generate")
def generate_activations(config: ConfigArg) -> None:
    """Generate activations from a language model and write them to disk."""
    from ..runners import GenerateActivationsSettings
    from ..runners import generate_activations as run

    run(GenerateActivationsSettings.model_validate(load_config(config)))


@app.command("train")
def train(config: ConfigArg, kind: Annotated[TrainKind, typer.Option("--kind", "-k", help="Dictionary family to train.")] = TrainKind.sae) -> None:
    """Train a sparse dictionary."""
    from .. import runners as R

    table = {
        TrainKind.sae: (R.TrainSAESettings, R.train_sae),
        TrainKind.crosscoder: (R.TrainCrosscoderSettings, R.train_crosscoder),
        TrainKind.clt: (R.TrainCLTSettings, R.train_clt),
        TrainKind.lorsa: (R.TrainLorsaSettings, R.train_lorsa),
        TrainKind.molt: (R.TrainMOLTSettings, R.train_molt),
        TrainKind.sweep: (R.SweepSAESettings, R.sweep_sae),
    }
    settings_cls, fn = table[kind]
    fn(settings_cls.model_validate(load_config(config)))


@app.command("analyze")
def analyze(config: ConfigArg, kind: Annotated[AnalyzeKind, typer.Option("--kind", "-k")] = AnalyzeKind.sae) -> None:
    """Analyze the features of a trained sparse dictionary."""
    from .. import runners as R

    if kind is AnalyzeKind.sae:
        R.analyze_sae(R.AnalyzeSAESettings.model_validate(load_config(config)))
    else:
        R.analyze_crosscoder(R.AnalyzeCrosscoderSettings.model_validate(load_config(config)))


@app.command("evaluate")
def evaluate(config: ConfigArg, kind: Annotated[AnalyzeKind, typer.Option("--kind", "-k")] = AnalyzeKind.sae) -> None:
    """Evaluate a trained sparse dictionary on an activation stream."""
    from .. import runners as R

    if kind is AnalyzeKind.sae:
        R.evaluate_sae(R.EvaluateSAESettings.model_validate(load_config(config)))
    else:
        R.evaluate_crosscoder(R.EvaluateCrosscoderSettings.model_validate(load_config(config)))


@app.command("dla")
def dla(config: ConfigArg) -> None:
    """Direct logit attribution of every feature."""
    from .. import runners as R

    R.direct_logit_attribute(R.DirectLogitAttributeSettings.model_validate(load_config(config)))


@app.command("autointerp")
def autointerp(config: ConfigArg) -> None:
    """Explain features with a chat model."""
    from .. import runners as R

    R.auto_interp(R.AutoInterpSettings.model_validate(load_config(config)))


@app.command("convert")
def convert(config: ConfigArg) -> None:
    """Convert a top-k cross-layer transcoder to JumpReLU."""
    from .. import runners as R

    R.convert_topk_to_jumprelu(R.ConvertTopKToJumpReLUSettings.model_validate(load_config(config)))
