"""Attribution graph of one prompt through spliced-in dictionaries.

    python examples/attribute_prompt.py "The capital of France is"
"""

import sys

import torch

from language_model_saes_b200 import LanguageModelConfig, SparseDictionary, attribute, load_model, prune_attribution

if __name__ == "__main__":
    prompt = sys.argv[1] if len(sys.argv) > 1 else "The capital of France is"
    lm = load_model(LanguageModelConfig(model_name="EleutherAI/pythia-160m", device="cuda", dtype="bfloat16"))
    # transcoders on every MLP (so that the replaced model is linear in the features) and Lorsa on every attention layer
    dictionaries = [SparseDictionary.from_pretrained(f"results/pythia-160m-L{i}-transcoder", device="cuda") for i in range(12)]
    result = attribute(lm.model, prompt, dictionaries, target_type="logits", max_n_logits=5, desired_logit_prob=0.9,
                       batch_size=256, max_features=4096)  # fmt: skip
    pruned = prune_attribution(result.attribution, result.logit_probs, node_threshold=0.8, edge_threshold=0.98)
    kept = int((pruned.data != 0).sum())
    print(f"{result.attribution.data.shape[0]} target / intermediate rows, {kept} edges after pruning")
    torch.save(result, "attribution.pt")
