"""Load published dictionaries and run them on a prompt: a transcoder from a Hugging Face repository in this package's
layout (``<repo>:<folder>``) and a residual-stream SAE from a SAELens release (``<release>:<sae id>``, needs ``sae_lens``).

    python examples/load_pretrained_dictionaries.py hub
    python examples/load_pretrained_dictionaries.py saelens

Both need the model and the dictionary in the local Hugging Face cache (or network access).
"""

import sys

import torch

from language_model_saes_b200 import LanguageModelConfig, SparseDictionary, load_model

SOURCES = {
    # (dictionary, language model): a transcoder reads one hook point and reconstructs another
    "hub": ("OpenMOSS-Team/Llama-Scope-2-Qwen3-1.7B:transcoder/8x/k128/layer12_transcoder_8x_k128", "Qwen/Qwen3-1.7B"),
    "saelens": ("gemma-scope-2-1b-pt-res-all:layer_12_width_16k_l0_small", "google/gemma-3-1b-pt"),
}

if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "hub"
    name, model_name = SOURCES[which]
    device = "cuda" if torch.cuda.is_available() else "cpu"
    # fold_activation_scale=False keeps the stored norm convention: normalize_activations() below applies it to the inputs
    sae = SparseDictionary.from_pretrained(name, fold_activation_scale=False, device=device)
    print(f"{type(sae).__name__}: {sae.cfg.hook_point_in} -> {sae.cfg.hook_point_out}, {sae.cfg.d_sae} features, {sae.cfg.act_fn}")
    lm = load_model(LanguageModelConfig(model_name=model_name, device=device, dtype="bfloat16"))
    prompt = "The capital of France is"
    hooks = sorted({sae.cfg.hook_point_in, sae.cfg.hook_point_out})
    batch = lm.to_activations({"text": [prompt]}, hook_points=hooks)
    with torch.no_grad():
        batch = sae.normalize_activations(batch)
        x, encoder_kwargs, decoder_kwargs = sae.prepare_input(batch)
        feature_acts = sae.encode(x, **encoder_kwargs)
        reconstructed = sae.decode(feature_acts, **decoder_kwargs)
        label = sae.prepare_label(batch)
    l0 = (feature_acts > 0).sum(dim=-1).float().mean()
    err = (label.to(reconstructed.dtype) - reconstructed).pow(2).sum(-1)
    var = (label - label.mean(dim=(0, 1), keepdim=True)).pow(2).sum(-1)
    print(f"prompt: {prompt!r}\nmean L0 {float(l0):.1f}, explained variance {1 - float(err.mean() / var.mean()):.3f}")
    top = feature_acts[0, -1].float().topk(5)
    print("strongest features on the last token:", [(int(i), round(float(v), 3)) for v, i in zip(top.values, top.indices)])
