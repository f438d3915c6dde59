"""Blackwell-native sparse-dictionary training framework (SAEs, transcoders, crosscoders, CLTs, Lorsa, MOLT)."""

from .config import BaseConfig, BaseModelConfig, DatasetConfig
from .models.sae import SAEConfig, SparseAutoEncoder
from .models.sparse_dictionary import SparseDictionary, SparseDictionaryConfig
from .trainer import Trainer, TrainerConfig, WandbConfig
from .utils.logging import setup_logging

__version__ = "0.1.0"
