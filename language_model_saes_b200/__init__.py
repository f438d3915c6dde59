"""Blackwell-native sparse-dictionary training framework (SAEs, transcoders, crosscoders, CLTs, Lorsa, MOLT).

Top-level names follow the public surface of the reference project (``llamascopium/__init__.py``): configs, models,
runners and their settings, trainer, initializer, activation pipeline, language-model backends, analysis, circuits,
database and loaders. ``TransformerLensLanguageModel`` is the hooked backend of this package (same hook-point names).
"""

from .activation.factory import (
    ActivationFactory,
    ActivationFactoryActivationsSource,
    ActivationFactoryConfig,
    ActivationFactoryDatasetSource,
    ActivationFactoryTarget,
)
from .activation.processors.activation import BufferShuffleConfig
from .activation.writer import ActivationWriter, ActivationWriterConfig
from .activation_functions import JumpReLU
from .analysis.direct_logit_attributor import DirectLogitAttributor, DirectLogitAttributorConfig
from .analysis.feature_analyzer import FeatureAnalyzer, FeatureAnalyzerConfig
from .backend.language_model import (
    HookedLanguageModel,
    HuggingFaceLanguageModel,
    LanguageModel,
    LanguageModelConfig,
    QwenVLLanguageModel,
    TokenizerOnlyLanguageModel,
)
from .circuits import (
    AttributionResult,
    NodeDimension,
    NodeIndexed,
    NodeIndexedMatrix,
    NodeIndexedTensor,
    NodeIndexedVector,
    NodeInfo,
    attribute,
    compute_hessian_matrix,
    prune_attribution,
    qk_trace,
)
from .config import BaseConfig, BaseModelConfig, DatasetConfig
from .database import (
    CircuitConfig,
    CircuitInput,
    CircuitStatus,
    FeatureAnalysisSampling,
    FeatureRecord,
    MongoClient,
    MongoDBConfig,
)
from .evaluator import EvalConfig, Evaluator
from .initializer import Initializer, InitializerConfig
from .models.clt import CLTConfig, CrossLayerTranscoder
from .models.crosscoder import Crosscoder, CrosscoderConfig
from .models.lorsa import LorsaConfig, LowRankSparseAttention
from .models.molt import MixtureOfLinearTransform, MOLTConfig
from .models.protocols import DatasetNormStandardizable, EncoderInitializable, NormComputing, NormConstrainable
from .models.sae import SAEConfig, SparseAutoEncoder
from .models.sparse_dictionary import SparseDictionary, SparseDictionaryConfig
from .resource_loaders import load_dataset, load_dataset_shard, load_model
from .runners import (
    AnalyzeCrosscoderSettings,
    AnalyzeSAESettings,
    AutoInterpSettings,
    CheckActivationConsistencySettings,
    ConvertTopKToJumpReLUSettings,
    DirectLogitAttributeSettings,
    EvaluateCrosscoderSettings,
    EvaluateSAESettings,
    GenerateActivationsSettings,
    PretrainedSAE,
    SweepingItem,
    SweepSAESettings,
    TrainCLTSettings,
    TrainCrosscoderSettings,
    TrainLorsaSettings,
    TrainMOLTSettings,
    TrainSAESettings,
    analyze_crosscoder,
    analyze_sae,
    auto_interp,
    check_activation_consistency,
    convert_topk_to_jumprelu,
    direct_logit_attribute,
    evaluate_crosscoder,
    evaluate_sae,
    generate_activations,
    sweep_sae,
    train_clt,
    train_crosscoder,
    train_lorsa,
    train_molt,
    train_sae,
)
from .trainer import Trainer, TrainerConfig, WandbConfig
from .utils.logging import setup_logging

TransformerLensLanguageModel = HookedLanguageModel

__version__ = "0.1.0"

__all__ = [
    "ActivationFactory", "ActivationFactoryActivationsSource", "ActivationFactoryConfig", "ActivationFactoryDatasetSource",
    "ActivationFactoryTarget", "ActivationWriter", "ActivationWriterConfig", "AnalyzeCrosscoderSettings", "AnalyzeSAESettings",
    "AttributionResult", "AutoInterpSettings", "BaseConfig", "BaseModelConfig", "BufferShuffleConfig", "CLTConfig",
    "CheckActivationConsistencySettings", "CircuitConfig", "CircuitInput", "CircuitStatus", "ConvertTopKToJumpReLUSettings",
    "CrossLayerTranscoder", "Crosscoder", "CrosscoderConfig", "DatasetConfig", "DatasetNormStandardizable",
    "DirectLogitAttributeSettings", "DirectLogitAttributor", "DirectLogitAttributorConfig", "EncoderInitializable", "EvalConfig",
    "EvaluateCrosscoderSettings", "EvaluateSAESettings", "Evaluator", "FeatureAnalysisSampling", "FeatureAnalyzer",
    "FeatureAnalyzerConfig", "FeatureRecord", "GenerateActivationsSettings", "HookedLanguageModel", "HuggingFaceLanguageModel",
    "Initializer", "InitializerConfig", "JumpReLU", "LanguageModel", "LanguageModelConfig", "LorsaConfig", "LowRankSparseAttention",
    "MOLTConfig", "MixtureOfLinearTransform", "MongoClient", "MongoDBConfig", "NodeDimension", "NodeIndexed", "NodeIndexedMatrix",
    "NodeIndexedTensor", "NodeIndexedVector", "NodeInfo", "NormComputing", "NormConstrainable", "PretrainedSAE",
    "QwenVLLanguageModel", "SAEConfig", "SparseAutoEncoder", "SparseDictionary", "SparseDictionaryConfig", "SweepSAESettings",
    "SweepingItem", "TokenizerOnlyLanguageModel", "TrainCLTSettings", "TrainCrosscoderSettings", "TrainLorsaSettings",
    "TrainMOLTSettings", "TrainSAESettings", "Trainer", "TrainerConfig", "TransformerLensLanguageModel", "WandbConfig",
    "analyze_crosscoder", "analyze_sae", "attribute", "auto_interp", "check_activation_consistency", "compute_hessian_matrix",
    "convert_topk_to_jumprelu", "direct_logit_attribute", "evaluate_crosscoder", "evaluate_sae", "generate_activations",
    "load_dataset", "load_dataset_shard", "load_model", "prune_attribution", "qk_trace", "setup_logging", "sweep_sae", "train_clt",
    "train_crosscoder", "train_lorsa", "train_molt", "train_sae",
]  # fmt: skip
