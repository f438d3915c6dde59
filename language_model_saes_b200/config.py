"""Base configuration classes (pydantic v2).

Mirrors the configuration surface of the reference project's ``config.py`` (BaseConfig, BaseModelConfig
with ``device`` / ``dtype`` excluded from dumps, DatasetConfig; config.py:19-51 there). Unknown fields are
ignored on validation, as pydantic does by default, because user configs rely on that.
"""

from __future__ import annotations

from typing import Annotated

import torch
from pydantic import BaseModel, BeforeValidator, ConfigDict, Field, PlainSerializer, WithJsonSchema

from .utils.misc import convert_str_to_torch_dtype, convert_torch_dtype_to_str

TorchDType = Annotated[
    torch.dtype,
    BeforeValidator(lambda v: convert_str_to_torch_dtype(v) if isinstance(v, str) else v),
    PlainSerializer(convert_torch_dtype_to_str),
    WithJsonSchema({"type": "string"}, mode="serialization"),
]

OptionalTorchDType = Annotated[
    torch.dtype | None,
    BeforeValidator(lambda v: convert_str_to_torch_dtype(v) if isinstance(v, str) else v),
    PlainSerializer(lambda v: None if v is None else convert_torch_dtype_to_str(v)),
    WithJsonSchema({"type": ["string", "null"]}, mode="serialization"),
]


class BaseConfig(BaseModel):
    """Root of every non-model configuration object."""


class BaseModelConfig(BaseModel):
    """Root of model configurations: carries ``device`` and ``dtype``, neither of which is serialised."""

    model_config = ConfigDict(arbitrary_types_allowed=True)

    device: str = Field(default="cpu", exclude=True)
    dtype: TorchDType = Field(default=torch.float32, exclude=True, validate_default=False)


class DatasetConfig(BaseConfig):
    dataset_name_or_path: str = "openwebtext"
    cache_dir: str | None = None
    is_dataset_on_disk: bool = False
