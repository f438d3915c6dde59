"""Capability protocols that a dictionary class may implement.

Other layers ask ``isinstance(model, NormComputing)`` etc. instead of naming concrete classes
(the same six capabilities as models/protocols.py:14-113 in the reference project).
"""

from __future__ import annotations

from typing import Protocol, runtime_checkable

import torch


@runtime_checkable
class NormComputing(Protocol):
    """Can report encoder / decoder / decoder-bias norms per feature."""

    def encoder_norm(self, keepdim: bool = False) -> torch.Tensor: ...

    def decoder_norm(self, keepdim: bool = False) -> torch.Tensor: ...

    def decoder_bias_norm(self) -> torch.Tensor: ...


@runtime_checkable
class NormConstrainable(Protocol):
    """Can rescale its weights to prescribed norms."""

    def set_decoder_to_fixed_norm(self, value: float, force_exact: bool) -> None: ...

    def set_encoder_to_fixed_norm(self, value: float) -> None: ...

    def transform_to_unit_decoder_norm(self) -> None: ...


@runtime_checkable
class DatasetNormStandardizable(Protocol):
    """Can fold the dataset-wise activation scale into its parameters (switching to inference mode)."""

    def standardize_parameters_of_dataset_norm(self) -> None: ...


@runtime_checkable
class EncoderInitializable(Protocol):
    """Can initialise the encoder as a multiple of the transposed decoder."""

    def init_encoder_with_decoder_transpose(self, factor: float = 1.0) -> None: ...


@runtime_checkable
class ActiveSubspaceInitializable(Protocol):
    """Can project its decoder onto the top principal subspace of a batch of labels."""

    def init_W_D_with_active_subspace(self, batch: dict[str, torch.Tensor], d_active_subspace: int) -> None: ...


@runtime_checkable
class EncoderBiasInitializable(Protocol):
    """Can set the encoder bias so that mean pre-activations over a batch are zero."""

    def init_encoder_bias_with_mean_hidden_pre(self, batch: dict[str, torch.Tensor]) -> None: ...
