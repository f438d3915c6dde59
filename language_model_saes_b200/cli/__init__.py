"""Command line: ``generate | train | analyze | evaluate | dla | autointerp | convert`` and the groups
``create``, ``remove``, ``show`` (cli/__init__.py of the reference project)."""

import typer

from . import create, remove, run, show
from .common import DEFAULT_MONGO_DB, DEFAULT_MONGO_URI, DEFAULT_SAE_SERIES, MongoDBOption, MongoURIOption, SAESeriesOption, console
from .utils import load_config

app = typer.Typer(name="lmsaes-b200", help="Sparse dictionary training, analysis and database management on B200.", no_args_is_help=True)
for _cmd in run.app.registered_commands:
    app.registered_commands.append(_cmd)
app.add_typer(create.app, name="create")
app.add_typer(remove.app, name="remove")
app.add_typer(show.app, name="show")


def entrypoint() -> None:
    import torch

    try:
        import datasets

        datasets.disable_progress_bar()
    except ImportError:
        pass
    try:
        app()
    finally:
        if torch.distributed.is_initialized():
            torch.distributed.destroy_process_group()


__all__ = ["app", "console", "entrypoint", "load_config", "DEFAULT_MONGO_URI", "DEFAULT_MONGO_DB", "DEFAULT_SAE_SERIES",
           "MongoURIOption", "MongoDBOption", "SAESeriesOption"]  # fmt: skip
