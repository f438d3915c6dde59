"""Entry points that take one settings object and run a whole job."""

from .analyze import AnalyzeCrosscoderSettings, AnalyzeSAESettings, DirectLogitAttributeSettings, analyze_crosscoder, analyze_sae, direct_logit_attribute
from .autointerp import AutoInterpSettings, auto_interp
from .eval import EvaluateCrosscoderSettings, EvaluateSAESettings, evaluate_crosscoder, evaluate_sae
from .generate import CheckActivationConsistencySettings, GenerateActivationsSettings, check_activation_consistency, generate_activations
from .topk_to_jumprelu_conversion import ConvertTopKToJumpReLUSettings, convert_topk_to_jumprelu
from .train import (
    SweepingItem,
    SweepSAESettings,
    TrainCLTSettings,
    TrainCrosscoderSettings,
    TrainLorsaSettings,
    TrainMOLTSettings,
    TrainSAESettings,
    sweep_sae,
    train_clt,
    train_crosscoder,
    train_lorsa,
    train_molt,
    train_sae,
)
from .utils import PretrainedSAE, load_config

__all__ = [
    "AnalyzeCrosscoderSettings", "AnalyzeSAESettings", "AutoInterpSettings", "CheckActivationConsistencySettings",
    "ConvertTopKToJumpReLUSettings", "DirectLogitAttributeSettings", "EvaluateCrosscoderSettings", "EvaluateSAESettings",
    "GenerateActivationsSettings", "PretrainedSAE", "SweepSAESettings", "SweepingItem", "TrainCLTSettings",
    "TrainCrosscoderSettings", "TrainLorsaSettings", "TrainMOLTSettings", "TrainSAESettings", "analyze_crosscoder",
    "analyze_sae", "auto_interp", "check_activation_consistency", "convert_topk_to_jumprelu", "direct_logit_attribute",
    "evaluate_crosscoder", "evaluate_sae", "generate_activations", "load_config", "sweep_sae", "train_clt",
    "train_crosscoder", "train_lorsa", "train_molt", "train_sae",
]  # fmt: skip
