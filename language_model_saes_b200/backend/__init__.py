from .hooked_transformer import HookedTransformer, HookedTransformerConfig, pythia_shaped_config
from .language_model import (
    HookedLanguageModel,
    HuggingFaceLanguageModel,
    LanguageModel,
    LanguageModelConfig,
    QwenVLLanguageModel,
    TokenizerOnlyLanguageModel,
    TransformerLensLanguageModel,
)
