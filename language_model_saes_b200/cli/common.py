"""Options shared by the command groups; defaults come from ``MONGO_URI``, ``MONGO_DB`` and ``SAE_SERIES``
(cli/common.py of the reference project)."""

import os
from typing import Annotated

import typer
from rich.console import Console

DEFAULT_MONGO_URI = os.environ.get("MONGO_URI", "mongodb://localhost:27017/")
DEFAULT_MONGO_DB = os.environ.get("MONGO_DB", "mechinterp")
DEFAULT_SAE_SERIES = os.environ.get("SAE_SERIES", "default")

console = Console()

MongoURIOption = Annotated[str, typer.Option("--mongo-uri", envvar="MONGO_URI", help="Database URI (mongodb://... or file://<dir> for the local store).")]
MongoDBOption = Annotated[str, typer.Option("--mongo-db", envvar="MONGO_DB", help="Database name.")]
SAESeriesOption = Annotated[str, typer.Option("--series", "-s", envvar="SAE_SERIES", help="SAE series identifier.")]
