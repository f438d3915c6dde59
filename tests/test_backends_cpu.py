"""Language-model backends against each other on the tiny model: the plain ``transformers`` backend (residual streams from
``output_hidden_states``) must read the same activations, tokens and origins as the hooked-transformer backend, and
refuse hook points it cannot reach; the tokenizer-only backend traces text without a model; the consistency runner walks
caches of several hook points together."""

import pytest
import torch
from conftest import tiny_lm_config

from language_model_saes_b200.backend.language_model import HookedLanguageModel, HuggingFaceLanguageModel, TokenizerOnlyLanguageModel


def test_transformers_backend_reads_the_same_residual_streams_as_the_hooked_one(tiny_lm_workspace):
    cfg = tiny_lm_config(tiny_lm_workspace)
    hooked, plain = HookedLanguageModel(cfg), HuggingFaceLanguageModel(cfg.model_copy(update={"backend": "huggingface"}))
    raw = {"text": ["the cat sat on a mat", "dog ran far away"]}
    hooks = ["blocks.0.hook_resid_post", "blocks.1.hook_resid_post"]
    a, b = hooked.to_activations(raw, hooks), plain.to_activations(raw, hooks)
    assert torch.equal(a["tokens"], b["tokens"])
    assert torch.equal(a["mask"], b["mask"]) and not a["mask"].all()  # padding of the shorter text is masked on both
    valid = a["mask"]
    # blocks.0 is the stream after the first block on both; the last one differs by the final layer norm, which
    # ``output_hidden_states`` applies to its last entry
    assert torch.allclose(a[hooks[0]][valid], b[hooks[0]][valid], atol=1e-4)
    assert b[hooks[1]].shape == a[hooks[1]].shape
    assert hooked.trace(raw) == plain.trace(raw)
    origins = plain.trace(raw)[1]
    text = raw["text"][1]
    words = [text[o["range"][0] : o["range"][1]] for o in origins if o is not None]
    assert words == text.split() or words[: len(text.split())] == text.split()
    with pytest.raises((ValueError, AssertionError)):
        plain.to_activations(raw, ["blocks.0.attn.hook_q"])  # only residual streams are reachable this way
    assert plain.bos_token_id == hooked.bos_token_id and plain.pad_token_id == hooked.pad_token_id
    short = plain.to_activations(raw, hooks[:1], n_context=3)
    assert short["tokens"].shape == (2, 3) and short[hooks[0]].shape[:2] == (2, 3)


def test_tokenizer_only_backend_traces_text_but_has_no_activations(tiny_lm_workspace):
    cfg = tiny_lm_config(tiny_lm_workspace).model_copy(update={"backend": "tokenizer_only"})
    tok = TokenizerOnlyLanguageModel(cfg)
    raw = {"text": ["big red sun"]}
    origins = tok.trace(raw)[0]
    assert [raw["text"][0][o["range"][0] : o["range"][1]] for o in origins if o is not None] == ["big", "red", "sun"]
    with pytest.raises((NotImplementedError, AttributeError, AssertionError, RuntimeError)):
        tok.to_activations(raw, ["blocks.0.hook_resid_post"])


def test_consistency_runner_walks_caches_together_and_names_a_mismatch(tmp_path):
    from safetensors.torch import save_file

    from language_model_saes_b200.runners.generate import CheckActivationConsistencySettings, check_activation_consistency

    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(3, 50, (4, 6), generator=g)
    for hp in ("h0", "h1"):
        (tmp_path / hp).mkdir()
        for c in range(2):
            save_file({"activation": torch.randn(4, 6, 8, generator=g), "tokens": tokens + c, "mask": torch.ones(4, 6, dtype=torch.bool),
                       "attention_mask": torch.ones(4, 6, dtype=torch.bool)}, str(tmp_path / hp / f"chunk-{c}.safetensors"))  # fmt: skip
    settings = CheckActivationConsistencySettings(paths={"h0": tmp_path / "h0", "h1": tmp_path / "h1"}, device="cpu")
    check_activation_consistency(settings)  # agrees: returns quietly
    save_file({"activation": torch.randn(4, 6, 8, generator=g), "tokens": tokens + 7, "mask": torch.ones(4, 6, dtype=torch.bool),
               "attention_mask": torch.ones(4, 6, dtype=torch.bool)}, str(tmp_path / "h1" / "chunk-1.safetensors"))  # fmt: skip
    with pytest.raises(AssertionError, match="tokens mismatch"):
        check_activation_consistency(settings)
