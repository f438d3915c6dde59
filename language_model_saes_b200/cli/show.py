"""``show feature``: print a feature's statistics and its top activating samples with coloured tokens
(cli/show.py of the reference project)."""

from __future__ import annotations

import itertools
from functools import lru_cache
from typing import Annotated, Iterator

import numpy as np
import torch
import typer
from rich.panel import Panel
from rich.text import Text

from ..analysis.samples import TokenizedSample
from ..database import FeatureAnalysisSampling, MongoClient, MongoDBConfig
from ..resource_loaders import load_dataset_shard, load_model
from .common import DEFAULT_MONGO_DB, DEFAULT_MONGO_URI, DEFAULT_SAE_SERIES, MongoDBOption, MongoURIOption, SAESeriesOption, console

app = typer.Typer(help="Display feature activation samples and statistics.")


def activation_color(activation: float, max_activation: float) -> str:
    """white (silent) -> yellow -> orange -> red by the fraction of the feature's maximum."""
    if max_activation <= 0:
        return "white"
    frac = min(activation / max_activation, 1.0)
    return "white" if frac < 0.01 else "yellow" if frac < 0.33 else "orange1" if frac < 0.66 else "red"


def extract_samples(sampling: FeatureAnalysisSampling, client: MongoClient, max_activation: float) -> Iterator[TokenizedSample]:
    idx = torch.as_tensor(np.asarray(sampling.feature_acts_indices)).long()
    val = torch.as_tensor(np.asarray(sampling.feature_acts_values)).float()
    n = len(sampling.context_idx)
    width = int(idx[1].max()) + 1 if idx.numel() else 1
    acts = torch.zeros(n, width)
    if idx.numel():
        acts[idx[0], idx[1]] = val

    @lru_cache(maxsize=8)
    def model_of(name: str):
        cfg = client.get_model_cfg(name=name)
        assert cfg is not None, f"Model {name} not found"
        cfg.backend = "tokenizer_only"
        return load_model(cfg)

    @lru_cache(maxsize=8)
    def shard_of(name: str, shard_idx: int, n_shards: int):
        cfg = client.get_dataset_cfg(name=name)
        assert cfg is not None, f"Dataset {name} not found"
        return load_dataset_shard(cfg, shard_idx, n_shards)

    shard = sampling.shard_idx if sampling.shard_idx is not None else [0] * n
    n_shards = sampling.n_shards if sampling.n_shards is not None else [1] * n
    for i in range(n):
        data = shard_of(sampling.dataset_name[i], int(shard[i]), int(n_shards[i]))[int(sampling.context_idx[i])]
        origins = model_of(sampling.model_name[i]).trace({k: [v] for k, v in data.items()}, n_context=2048)[0]
        row = torch.nn.functional.pad(acts[i], (0, max(0, len(origins) - width)))
        yield TokenizedSample.construct(data["text"], row[: len(origins)], origins, max_activation)


def render_sample(sample: TokenizedSample) -> Text:
    out = Text()
    for seg in sample.segments:
        if seg.activation > 0.01:
            out.append(seg.text, style=f"bold {activation_color(seg.activation, sample.max_activation)} on grey23")
        else:
            out.append(seg.text)
    return out


@app.command("feature")
def show_feature(sae_name: Annotated[str, typer.Argument(help="Name of the SAE.")],
                 feature_index: Annotated[int, typer.Argument(help="Index of the feature to display.")],
                 sae_series: SAESeriesOption = DEFAULT_SAE_SERIES,
                 analysis_name: Annotated[str | None, typer.Option("--analysis", "-a", help="Name of the analysis.")] = None,
                 num_samples: Annotated[int, typer.Option("--num-samples", "-n", help="Number of samples to display.")] = 5,
                 visible_range: Annotated[int, typer.Option("--visible-range", "-r", help="Tokens shown around the strongest token.")] = 20,
                 mongo_uri: MongoURIOption = DEFAULT_MONGO_URI, mongo_db: MongoDBOption = DEFAULT_MONGO_DB) -> None:  # fmt: skip
    """Display top activation samples for a feature with highlighted tokens."""
    client = MongoClient(MongoDBConfig(mongo_uri=mongo_uri, mongo_db=mongo_db))
    features = client.list_features(sae_name=sae_name, sae_series=sae_series, indices=[feature_index])
    if not features:
        console.print(f"[red]Feature {feature_index} not found in SAE '{sae_name}'[/red]")
        raise typer.Exit(1)
    feature = features[0]
    wanted = analysis_name or "default"
    analysis = next((a for a in feature.analyses if a.name == wanted), None)
    if analysis is None and analysis_name is None:
        analysis = next(iter(feature.analyses), None)
    if analysis is None:
        console.print(f"[red]No analysis found for feature {feature_index}[/red]")
        raise typer.Exit(1)

    header = Text()
    header.append(f"Feature #{feature_index}", style="bold cyan")
    header.append(f" @ {sae_name}", style="dim")
    if feature.interpretation:
        header.append(f"\n{feature.interpretation.get('text', '')}", style="italic")
    console.print()
    console.print(Panel(header, title="Feature Info", border_style="cyan"))
    stats = Text()
    stats.append("Activation Times: ", style="bold")
    stats.append(f"{analysis.act_times:,}\n")
    stats.append("Max Activation: ", style="bold")
    stats.append(f"{analysis.max_feature_acts:.4f}")
    if analysis.n_analyzed_tokens:
        stats.append("\nAnalyzed Tokens: ", style="bold")
        stats.append(f"{analysis.n_analyzed_tokens:,}")
    console.print(Panel(stats, title="Statistics", border_style="green"))

    sampling = next((s for s in analysis.samplings if s.name == "top_activations"), None)
    if sampling is None:
        console.print("[yellow]No top activation samples available.[/yellow]")
        raise typer.Exit(0)
    legend = Text()
    legend.append(f"Top {num_samples} Activation Samples", style="bold")
    legend.append("  (")
    for label, color, sep in (("Weak", "yellow", " | "), ("Medium", "orange1", " | "), ("Strong", "red", ")")):
        legend.append(label, style=f"{color} on grey23")
        legend.append(sep)
    console.print()
    console.print(legend)
    console.print()
    for i, sample in enumerate(itertools.islice(extract_samples(sampling, client, analysis.max_feature_acts), num_samples)):
        window = sample.to_max_activation_surrounding(visible_range)
        console.print(Panel(render_sample(window), title=f"Sample {i + 1}  (max {sample.sample_max_activation:.3f})", border_style="blue"))
