"""The bounds-checked debug build of the kernels (``-DLMSAE_BOUNDS_CHECK``, selected with ``LMSAE_NATIVE_CHECKED=1``): an
index beyond its limit is recorded and clamped instead of read out of bounds, and a regular training step records
nothing. Runs in a child process because the build variant is chosen when the extension is first loaded."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

CHILD = r"""
import torch
from language_model_saes_b200.ops import native, sae_kernels as K
from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
from language_model_saes_b200.ops.fused_step import FusedTopKSAEStep

ext = native.load(required=True)
assert ext.bounds_checked_build()
dev = torch.device("cuda")
F, d, B, k = 512, 64, 32, 4
W = torch.randn(F, d, device=dev).to(torch.bfloat16)
idx = torch.randint(0, F, (B, k), device=dev, dtype=torch.int32)
val = torch.randn(B, k, device=dev)
good = K.sparse_decode(idx, val, W, None)
torch.cuda.synchronize()
assert ext.bounds_report()["sparse_ops.cu"][3] == 0
bad = idx.clone()
bad[3, 1] = F + 7          # beyond the dictionary: the checked build records it and reads row F - 1 instead
out = K.sparse_decode(bad, val, W, None)
torch.cuda.synchronize()
line, index, limit, count = ext.bounds_report()["sparse_ops.cu"]
assert count >= 1 and index == F + 7 and limit == F and line > 0, (line, index, limit, count)
assert torch.isfinite(out).all()
assert ext.bounds_report()["sparse_ops.cu"][3] == 0   # reading cleared the record
# a regular fused step stays inside every limit
torch.manual_seed(0)
cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=256, expansion_factor=8, act_fn="topk", top_k=16, device="cuda", dtype=torch.float32)
sae = SparseAutoEncoder(cfg)
sae.init_parameters(encoder_uniform_bound=0.06, decoder_uniform_bound=0.06)
sae.set_decoder_to_fixed_norm(1.0, True)
sae.init_encoder_with_decoder_transpose()
eng = FusedTopKSAEStep(sae)
x = torch.randn(512, 256, device=dev).to(torch.bfloat16)
losses = [float(eng.step(x, x, 16, 1e-3)) for _ in range(3)]
K.check_status(dev)
rep = ext.bounds_report()
assert all(v[3] == 0 for v in rep.values()), rep
assert losses[-1] < losses[0]
print("checked build ok")
"""


def test_checked_build_records_and_clamps_an_out_of_range_index():
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, LMSAE_NATIVE_CHECKED="1", PYTHONPATH=str(root))
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, cwd=str(root), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "checked build ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
