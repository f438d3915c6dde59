"""The sparse decode of a mixture of linear transforms (``ops/molt_sparse.py``, opt-in through ``use_triton_kernel``)
against the model's dense decode: outputs and the gradients of gate, input and both factor matrices. On the CPU the torch
statements of the gather kernels run; the operands are rounded to bf16 on both sides of the comparison."""

import copy

import pytest
import torch

from language_model_saes_b200.models.molt import MixtureOfLinearTransform, MOLTConfig
from language_model_saes_b200.ops import molt_sparse
from language_model_saes_b200.ops.molt_sparse import molt_group_decode


def _bf(t):
    return t.to(torch.bfloat16).float()


@pytest.mark.parametrize("r", [1, 4, 16])
def test_group_decode_matches_the_dense_products(r, monkeypatch):
    g = torch.Generator().manual_seed(r)
    B, n, d = 37, 24, 32
    acts = torch.relu(torch.randn(B, n, generator=g) - 1.0)  # a sparse gate, some rows empty
    acts[3] = 0
    x = _bf(torch.randn(B, d, generator=g))
    U = _bf(torch.randn(n, d, r, generator=g) / d**0.5)
    V = _bf(torch.randn(n, r, d, generator=g) / d**0.5)
    leaves = [t.clone().requires_grad_(True) for t in (acts, x, U, V)]
    dense = [t.clone().requires_grad_(True) for t in (acts, x, U, V)]
    if r == 4:  # several launches per row: the codes of a row are split
        monkeypatch.setattr(molt_sparse, "_MAX_CODES", 8)
    out = molt_group_decode(*leaves)
    Vx = torch.einsum("bd,crd->bcr", dense[1], dense[3])
    want = torch.einsum("bcr,cdr->bd", dense[0].unsqueeze(-1) * Vx, dense[2])
    assert torch.allclose(out, want, atol=2e-2, rtol=2e-2)
    go = _bf(torch.randn(B, d, generator=g))
    out.backward(go)
    want.backward(go)
    # the gate's gradient lives on its active entries only (what an activation function's backward keeps anyway)
    assert not leaves[0].grad[acts == 0].any()
    dense[0].grad[acts == 0] = 0
    for name, a, b in zip(("acts", "x", "U", "V"), leaves, dense):
        scale = float(b.grad.abs().max()) + 1e-6
        assert float((a.grad - b.grad).abs().max()) < 3e-2 * scale, name


def test_model_with_the_sparse_decode_trains_like_the_dense_one():
    torch.manual_seed(0)
    cfg = MOLTConfig(hook_point_in="a", hook_point_out="b", d_model=32, expansion_factor=0.75, rank_counts={2: 16, 8: 8}, act_fn="relu",
                     dtype=torch.float32, device="cpu", norm_activation="inference")  # fmt: skip
    dense = MixtureOfLinearTransform(cfg)
    dense.init_parameters()
    with torch.no_grad():
        dense.b_E.sub_(0.3)  # a sparser gate
        for p in list(dense.U_matrices.values()) + list(dense.V_matrices.values()):
            p.copy_(_bf(p * 4))
    sparse = MixtureOfLinearTransform(cfg.model_copy(update={"use_triton_kernel": True}))
    sparse.load_state_dict(copy.deepcopy(dense.state_dict()))
    g = torch.Generator().manual_seed(1)
    x, y = _bf(torch.randn(48, 32, generator=g)), torch.randn(48, 32, generator=g)
    batch = {"a": x, "b": y, "tokens": torch.zeros(48, dtype=torch.long)}
    outs = []
    for m in (dense, sparse):
        res = m.compute_loss(batch, return_aux_data=True)
        res["loss"].backward()
        outs.append(res)
    assert torch.allclose(outs[0]["loss"], outs[1]["loss"], rtol=2e-3)
    assert torch.allclose(outs[0]["reconstructed"], outs[1]["reconstructed"], atol=2e-2)
    for (name, p), (_, q) in zip(dense.named_parameters(), sparse.named_parameters()):
        scale = float(p.grad.abs().max()) + 1e-6
        assert float((p.grad - q.grad).abs().max()) < 4e-2 * scale, name
