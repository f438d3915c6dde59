"""``create dataset|model|sae``: register records in the database (cli/create.py of the reference project)."""

from pathlib import Path
from typing import Annotated

import typer

from ..backend.language_model import LanguageModelConfig
from ..config import DatasetConfig
from ..database import MongoClient, MongoDBConfig
from ..models.sparse_dictionary import SparseDictionaryConfig
from .common import DEFAULT_MONGO_DB, DEFAULT_MONGO_URI, DEFAULT_SAE_SERIES, MongoDBOption, MongoURIOption, SAESeriesOption
from .utils import load_config

app = typer.Typer(help="Create database records for datasets, models, or SAEs.")


def _client(uri: str, db: str) -> MongoClient:
    return MongoClient(MongoDBConfig(mongo_uri=uri, mongo_db=db))


@app.command("dataset")
def create_dataset(name: Annotated[str, typer.Argument(help="Name of the dataset.")],
                   config: Annotated[Path, typer.Argument(help="Path to a DatasetConfig file.")],
                   mongo_uri: MongoURIOption = DEFAULT_MONGO_URI, mongo_db: MongoDBOption = DEFAULT_MONGO_DB) -> None:  # fmt: skip
    """Create a dataset record."""
    _client(mongo_uri, mongo_db).add_dataset(name=name, cfg=DatasetConfig.model_validate(load_config(config)))
    typer.echo(f"Dataset '{name}' created successfully.")


@app.command("model")
def create_model(name: Annotated[str, typer.Argument(help="Name of the model.")],
                 config: Annotated[Path, typer.Argument(help="Path to a LanguageModelConfig file.")],
                 mongo_uri: MongoURIOption = DEFAULT_MONGO_URI, mongo_db: MongoDBOption = DEFAULT_MONGO_DB) -> None:  # fmt: skip
    """Create a model record."""
    _client(mongo_uri, mongo_db).add_model(name=name, cfg=LanguageModelConfig.model_validate(load_config(config)))
    typer.echo(f"Model '{name}' created successfully.")


@app.command("sae")
def create_sae(name: Annotated[str, typer.Argument(help="Name of the SAE.")],
               path: Annotated[Path, typer.Argument(help="Directory of the pretrained SAE.")],
               series: SAESeriesOption = DEFAULT_SAE_SERIES,
               mongo_uri: MongoURIOption = DEFAULT_MONGO_URI, mongo_db: MongoDBOption = DEFAULT_MONGO_DB) -> None:  # fmt: skip
    """Create an SAE record (any registered dictionary type; the type is read from its config.json)."""
    cfg = SparseDictionaryConfig.from_pretrained(str(path))
    _client(mongo_uri, mongo_db).create_sae(name=name, series=series, path=str(path), cfg=cfg)
    typer.echo(f"SAE '{name}' (series: {series}) created successfully.")
