"""Interchange of dictionaries with the outside world, without a network: HuggingFace hub upload / download (through a
directory that plays the hub) and SAELens conversion in both directions (through a minimal stand-in for the ``sae_lens``
package that has the classes and fields the conversion touches). What is checked is OUR side of the contract: which
files are written, how a ``<repo>:<name>`` address is resolved, and that weights and thresholds survive the round trip.
Counterparts in the reference project: models/sparse_dictionary.py:361-455 (hub), models/sae.py:377-470 (SAELens)."""

import shutil
import sys
import types
from dataclasses import dataclass, field

import pytest
import torch

from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
from language_model_saes_b200.models.sparse_dictionary import PretrainedSAEType, SparseDictionary, auto_infer_pretrained_sae_type


def _sae(act_fn: str, **kw) -> SparseAutoEncoder:
    torch.manual_seed(0)
    kw.setdefault("hook_point_out", "blocks.3.hook_resid_post")
    cfg = SAEConfig(hook_point_in="blocks.3.hook_resid_post", d_model=16, expansion_factor=4, act_fn=act_fn, top_k=5, device="cpu",
                    dtype=torch.float32, **kw)  # fmt: skip
    m = SparseAutoEncoder(cfg)
    m.init_parameters(encoder_uniform_bound=0.3, decoder_uniform_bound=0.3, init_log_jumprelu_threshold_value=-1.0)
    with torch.no_grad():
        m.b_E.normal_(std=0.1)
        m.b_D.normal_(std=0.1)
    return m


# ---- a directory that plays the hub -----------------------------------------------------------------------------------
@pytest.fixture
def fake_hub(tmp_path, monkeypatch):
    import huggingface_hub

    root = tmp_path / "hub"
    calls = {"create": [], "upload": [], "download": []}

    def create_repo(repo_id, private=False, exist_ok=False, token=None):
        calls["create"].append((repo_id, private))
        (root / repo_id).mkdir(parents=True, exist_ok=exist_ok)

    def upload_folder(folder_path, repo_id, path_in_repo, commit_message=None, token=None):
        calls["upload"].append((repo_id, path_in_repo, commit_message))
        shutil.copytree(folder_path, root / repo_id / path_in_repo, dirs_exist_ok=True)

    def snapshot_download(repo_id, allow_patterns=None, token=None):
        calls["download"].append((repo_id, tuple(allow_patterns or ())))
        if not (root / repo_id).exists():
            raise FileNotFoundError(repo_id)
        return str(root / repo_id)

    def hf_hub_download(repo_id, filename, token=None):
        return str(root / repo_id / filename)

    for name, fn in (("create_repo", create_repo), ("upload_folder", upload_folder), ("snapshot_download", snapshot_download),
                     ("hf_hub_download", hf_hub_download)):  # fmt: skip
        monkeypatch.setattr(huggingface_hub, name, fn)
    return root, calls


@pytest.mark.parametrize("act_fn", ["topk", "jumprelu"])
def test_hub_round_trip(fake_hub, act_fn):
    root, calls = fake_hub
    m = _sae(act_fn)
    m.set_dataset_average_activation_norm({"blocks.3.hook_resid_post": 3.0})
    m.upload_to_hf("someone/dictionaries", "layer3", private=True)
    assert calls["create"] == [("someone/dictionaries", True)] and calls["upload"][0][:2] == ("someone/dictionaries", "layer3")
    written = {p.name for p in (root / "someone/dictionaries/layer3").iterdir()}
    assert "config.json" in written and any(n.endswith(".safetensors") for n in written)
    address = "someone/dictionaries:layer3"
    assert auto_infer_pretrained_sae_type(address) == PretrainedSAEType.HUGGINGFACE  # not a path, not a SAELens release
    again = SparseDictionary.from_pretrained(address, device="cpu", dtype=torch.float32)
    assert type(again) is SparseAutoEncoder and again.cfg.act_fn == act_fn and calls["download"] == [("someone/dictionaries", ("layer3/*",))]
    for (name, a), (_, b) in zip(m.named_parameters(), again.named_parameters()):
        assert torch.equal(a, b), name
    assert again.dataset_average_activation_norm == {"blocks.3.hook_resid_post": 3.0}
    x = torch.randn(7, 16)
    assert torch.allclose(m.forward(x), again.forward(x))
    cfg = SAEConfig.from_pretrained(address)  # the configuration alone, through hf_hub_download
    assert cfg.d_model == 16 and cfg.sae_pretrained_name_or_path == address
    with pytest.raises(FileNotFoundError):
        SparseDictionary.from_hf("someone/dictionaries", "layer4")
    with pytest.raises(ValueError):
        auto_infer_pretrained_sae_type("neither-a-path-nor-an-address")


# ---- a stand-in for the sae_lens package ----------------------------------------------------------------------------------
@pytest.fixture
def fake_saelens(monkeypatch):
    @dataclass
    class SAEMetadata:
        model_name: str = "unknown"
        hook_name: str = ""

    @dataclass
    class _Cfg:
        d_in: int = 0
        d_sae: int = 0
        dtype: str = "torch.float32"
        device: str = "cpu"
        apply_b_dec_to_input: bool = False
        normalize_activations: str = "none"
        reshape_activations: str = "none"
        metadata: SAEMetadata = field(default_factory=SAEMetadata)

    @dataclass
    class StandardSAEConfig(_Cfg):
        pass

    @dataclass
    class JumpReLUSAEConfig(_Cfg):
        pass

    @dataclass
    class TopKSAEConfig(_Cfg):
        k: int = 0
        rescale_acts_by_decoder_norm: bool = False

    class SAE(torch.nn.Module):
        registry: dict = {}

        def __init__(self, cfg):
            super().__init__()
            self.cfg = cfg
            self.W_enc = torch.nn.Parameter(torch.zeros(cfg.d_in, cfg.d_sae))
            self.W_dec = torch.nn.Parameter(torch.zeros(cfg.d_sae, cfg.d_in))
            self.b_enc = torch.nn.Parameter(torch.zeros(cfg.d_sae))
            self.b_dec = torch.nn.Parameter(torch.zeros(cfg.d_in))

        @classmethod
        def from_pretrained(cls, release, sae_id):
            return cls.registry[(release, sae_id)]

    class StandardSAE(SAE):
        pass

    class TopKSAE(SAE):
        pass

    class JumpReLUSAE(SAE):
        def __init__(self, cfg):
            super().__init__(cfg)
            self.threshold = torch.nn.Parameter(torch.ones(cfg.d_sae))

    @dataclass
    class _Release:
        saes_map: dict

    pkg = types.ModuleType("sae_lens")
    pkg.__spec__ = types.SimpleNamespace(name="sae_lens", loader=None, origin="stand-in", submodule_search_locations=[])
    for cls in (SAE, StandardSAE, TopKSAE, JumpReLUSAE, StandardSAEConfig, TopKSAEConfig, JumpReLUSAEConfig):
        setattr(pkg, cls.__name__, cls)
    saes = types.ModuleType("sae_lens.saes")
    saes_sae = types.ModuleType("sae_lens.saes.sae")
    saes_sae.SAEMetadata = SAEMetadata
    loading = types.ModuleType("sae_lens.loading")
    directory = types.ModuleType("sae_lens.loading.pretrained_saes_directory")
    directory.get_pretrained_saes_directory = lambda: {"a-release": _Release({"blocks.3": "path/in/release"})}
    for name, mod in (("sae_lens", pkg), ("sae_lens.saes", saes), ("sae_lens.saes.sae", saes_sae), ("sae_lens.loading", loading),
                      ("sae_lens.loading.pretrained_saes_directory", directory)):  # fmt: skip
        monkeypatch.setitem(sys.modules, name, mod)
    import importlib.util

    real_find_spec = importlib.util.find_spec
    monkeypatch.setattr(importlib.util, "find_spec", lambda name, *a, **k: pkg.__spec__ if name == "sae_lens" else real_find_spec(name, *a, **k))
    return pkg


@pytest.mark.parametrize("act_fn,gate", [("relu", True), ("topk", True), ("topk", False), ("jumprelu", True)])
def test_saelens_conversion_both_ways(fake_saelens, act_fn, gate):
    m = _sae(act_fn, sparsity_include_decoder_norm=gate)
    out = m.to_saelens(model_name="tiny-lm")
    want_cls = {"relu": fake_saelens.StandardSAE, "topk": fake_saelens.TopKSAE, "jumprelu": fake_saelens.JumpReLUSAE}[act_fn]
    assert type(out) is want_cls and out.cfg.d_in == 16 and out.cfg.d_sae == 64
    assert out.cfg.metadata.hook_name == "blocks.3.hook_resid_post" and out.cfg.metadata.model_name == "tiny-lm"
    assert torch.equal(out.W_enc, m.W_E) and torch.equal(out.W_dec, m.W_D) and torch.equal(out.b_enc, m.b_E) and torch.equal(out.b_dec, m.b_D)
    if act_fn == "topk":
        assert out.cfg.k == 5 and out.cfg.rescale_acts_by_decoder_norm == gate
    if act_fn == "jumprelu":
        assert torch.allclose(out.threshold, m.activation_function.log_jumprelu_threshold.exp())
    back = SparseAutoEncoder.from_saelens(out, device="cpu")
    assert back.cfg.act_fn == act_fn and back.cfg.hook_point_in == "blocks.3.hook_resid_post"
    if act_fn == "topk":
        assert back.cfg.top_k == 5 and back.cfg.sparsity_include_decoder_norm == gate
    for (name, a), (_, b) in zip(m.named_parameters(), back.named_parameters()):
        assert torch.allclose(a, b, atol=1e-6), name
    if gate or act_fn != "topk":  # (a plain ReLU / JumpReLU SAELens model has no decoder-norm gate to carry over)
        x = torch.randn(9, 16)
        if act_fn == "topk":
            assert torch.allclose(m.forward(x), back.forward(x), atol=1e-6)


def test_saelens_release_address_is_resolved_through_its_directory(fake_saelens):
    m = _sae("jumprelu")
    fake_saelens.SAE.registry[("a-release", "blocks.3")] = m.to_saelens()
    assert auto_infer_pretrained_sae_type("a-release:blocks.3") == PretrainedSAEType.SAELENS
    assert auto_infer_pretrained_sae_type("a-release:blocks.4") == PretrainedSAEType.HUGGINGFACE  # unknown to SAELens: a hub address
    got = SparseDictionary.from_pretrained("a-release:blocks.3", device="cpu")
    assert type(got) is SparseAutoEncoder and got.cfg.act_fn == "jumprelu"
    assert torch.allclose(got.W_D, m.W_D) and torch.allclose(got.activation_function.log_jumprelu_threshold, m.activation_function.log_jumprelu_threshold, atol=1e-6)
    with pytest.raises(ValueError):
        SAEConfig.from_pretrained("a-release:blocks.3")  # a SAELens release has no configuration file of ours
    with pytest.raises(AssertionError):
        _sae("topk", hook_point_out="blocks.3.hook_mlp_out").to_saelens()  # transcoders have no SAELens counterpart
