from .factory import (
    ActivationFactory,
    ActivationFactoryActivationsSource,
    ActivationFactoryConfig,
    ActivationFactoryDatasetSource,
    ActivationFactorySource,
    ActivationFactoryTarget,
)
from .processors.activation import (
    ActivationBatchler,
    ActivationBuffer,
    ActivationGenerator,
    ActivationTransformer,
    BufferShuffleConfig,
    OverrideDtypeProcessor,
)
from .processors.cached_activation import CachedActivationLoader, ChunkInfo
from .processors.core import BaseActivationProcessor
from .processors.huggingface import HuggingFaceDatasetLoader
from .processors.token import PadAndTruncateTokensProcessor, RawDatasetTokenProcessor
from .writer import ActivationWriter, ActivationWriterConfig
