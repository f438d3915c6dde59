"""Model configurations of the other dictionary families; each trains with the runner of the same name
(``train_crosscoder``, ``train_clt``, ``train_lorsa``, ``train_molt``) and the same settings layout as ``train_sae``.

    python examples/train_crosscoder_clt_lorsa.py      # prints the parameter counts
"""

import torch

from language_model_saes_b200 import CLTConfig, CrosscoderConfig, LorsaConfig, MOLTConfig
from language_model_saes_b200.models.sparse_dictionary import SparseDictionary

layers = range(12)
configs = {
    # one shared latent for eight training snapshots of a model (heads), JumpReLU; heads can be split over a `head` mesh
    # dimension, where the encoder GEMM sums the pre-activations over heads in its K loop and across ranks in its epilogue
    "crosscoder": CrosscoderConfig(hook_points=[f"step{s}/blocks.6.hook_resid_post" for s in range(8)], d_model=768,
                                   expansion_factor=32, act_fn="jumprelu", dtype=torch.bfloat16, device="cpu"),
    # cross-layer transcoder: features read the residual stream before each MLP and write to this and all later MLP outputs;
    # with `decode_with_csr` the decoder runs as one gather kernel over all (source, target) pairs
    "clt": CLTConfig(hook_points_in=[f"blocks.{i}.ln2.hook_normalized" for i in layers],
                     hook_points_out=[f"blocks.{i}.hook_mlp_out" for i in layers], d_model=768, expansion_factor=8,
                     act_fn="batchtopk", top_k=64, decode_with_csr=True, dtype=torch.bfloat16, device="cpu"),
    # low-rank sparse attention: 64 QK heads of width 64 shared by groups of 128 rank-1 OV heads; attention_kernel selects
    # the library attention or this package's tcgen05 kernels
    "lorsa": LorsaConfig(hook_point_in="blocks.6.ln1.hook_normalized", hook_point_out="blocks.6.hook_attn_out", d_model=768,
                         expansion_factor=8192 / 768, n_qk_heads=64, d_qk_head=64, rotary_dim=64, n_ctx=1024, act_fn="topk",
                         top_k=128, attention_kernel="library", dtype=torch.bfloat16, device="cpu"),
    # mixture of linear transforms: a sparse gate over low-rank maps of several ranks
    "molt": MOLTConfig(hook_point_in="blocks.6.ln2.hook_normalized", hook_point_out="blocks.6.hook_mlp_out", d_model=768,
                       expansion_factor=8, rank_counts={4: 2048, 16: 2048, 64: 2048}, act_fn="relu", dtype=torch.bfloat16, device="cpu"),
}  # fmt: skip

if __name__ == "__main__":
    for name, cfg in configs.items():
        with torch.device("meta"):
            model = SparseDictionary.from_config(cfg.model_copy(update={"device": "meta"}))
        print(f"{name:10s} {type(model).__name__:26s} {sum(p.numel() for p in model.parameters()) / 1e6:8.1f} M parameters")
