import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


TINY_WORDS = ["the", "cat", "sat", "on", "a", "mat", "dog", "ran", "far", "away", "big", "red", "sun", "sky", "is", "blue"]


@pytest.fixture(scope="session")
def tiny_lm_workspace(tmp_path_factory):
    """A directory with ``model/`` (random 2-layer GPT-2, d_model 16, word-level tokenizer: ids 0 bos/eos, 1 pad, 2 unk)
    and ``data/`` (64 texts of 20 words, saved with ``datasets``)."""
    return build_tiny_lm(tmp_path_factory.mktemp("tiny_lm"))


def build_tiny_lm(root):
    """Write the tiny model and dataset under ``root`` (a ``pathlib.Path``) and return it."""
    import datasets
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import GPT2Config, GPT2LMHeadModel, PreTrainedTokenizerFast

    vocab = {"<bos>": 0, "<pad>": 1, "<unk>": 2, **{w: i + 3 for i, w in enumerate(TINY_WORDS)}}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<bos>", eos_token="<bos>", pad_token="<pad>", unk_token="<unk>")
    torch.manual_seed(0)
    hf = GPT2LMHeadModel(GPT2Config(vocab_size=len(vocab), n_positions=32, n_embd=16, n_layer=2, n_head=2))
    hf.save_pretrained(root / "model")
    fast.save_pretrained(root / "model")
    g = torch.Generator().manual_seed(0)
    texts = [" ".join(TINY_WORDS[int(i)] for i in torch.randint(0, len(TINY_WORDS), (20,), generator=g)) for _ in range(64)]
    datasets.Dataset.from_dict({"text": texts}).save_to_disk(str(root / "data"))
    return root


def tiny_lm_config(root, backend: str = "hooked"):
    from language_model_saes_b200.backend.language_model import LanguageModelConfig

    return LanguageModelConfig(model_name="gpt2", model_from_pretrained_path=str(root / "model"), local_files_only=True, backend=backend,
                               device="cpu", dtype=torch.float32, max_length=32, bos_token_id=0, eos_token_id=0, pad_token_id=1)  # fmt: skip
