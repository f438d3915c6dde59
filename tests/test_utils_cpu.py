"""Small host-side pieces that the larger tests only touch in passing: dictionaries of tensors, the hierarchical timer, the
clock sampler (against a stand-in for the management library: reading only), the bucketed gradient reduction of the
autograd path (two gloo ranks) and the TopK -> JumpReLU conversion of a cross-layer transcoder."""

import sys
import time
import types

import pytest
import torch

from language_model_saes_b200.testing import distributed_test
from language_model_saes_b200.utils import tensor_dict as TD
from language_model_saes_b200.utils.timer import Timer


def test_dictionaries_of_tensors_sort_select_and_join_by_their_key():
    g = torch.Generator().manual_seed(0)
    d = {"elt": torch.randn(7, 3, generator=g), "ctx": torch.randint(0, 100, (7, 3), generator=g), "vec": torch.randn(7, 3, 5, generator=g)}
    s = TD.sort_dict_of_tensor(d, sort_dim=0, sort_key="elt", descending=True)
    order = d["elt"].argsort(0, descending=True)
    for col in range(3):
        assert torch.equal(s["elt"][:, col], d["elt"][order[:, col], col])
        assert torch.equal(s["ctx"][:, col], d["ctx"][order[:, col], col])
        assert torch.equal(s["vec"][:, col], d["vec"][order[:, col], col])  # whole trailing slices move with their key
    top = TD.topk_dict_of_tensor(d, 4)
    assert all(torch.equal(top[k], s[k][:4]) for k in d)
    assert TD.topk_dict_of_tensor(d, 99)["elt"].shape[0] == 7
    both = TD.concat_dict_of_tensor(d, s)
    assert both["vec"].shape == (14, 3, 5) and TD.batch_size(both) == 14
    with pytest.raises(AssertionError):
        TD.batch_size({"a": torch.zeros(3), "b": torch.zeros(4)})
    moved = TD.move_dict_of_tensor_to_device({"t": torch.zeros(2), "meta": ["x"]}, "cpu")
    assert moved["meta"] == ["x"] and moved["t"].device.type == "cpu"


def test_timer_nests_regions_counts_calls_and_stays_silent_when_off():
    t = Timer()
    assert t is Timer()  # one timer per process
    t.reset()
    t.disable()
    with t.time("off"):
        pass
    assert t.get_all_timers() == {}
    t.enable()
    try:
        @t.time("inner")
        def work():
            time.sleep(0.01)

        for _ in range(3):
            with t.time("outer"):
                work()
        assert t.get_count("outer") == 3 and t.get_count("inner") == 3
        assert t.get_time("outer") >= t.get_time("inner") >= 0.025
        assert t.get_average_time("inner") == pytest.approx(t.get_time("inner") / 3)
        assert any(path.endswith("outer/inner") or "inner" in path for path in t.get_all_timers())
        text = t.summary()
        assert "outer" in text and "inner" in text
        assert t.get_active_timers() == []
    finally:
        t.disable()
        t.reset()


def test_clock_sampler_reports_median_clock_and_throttle_reasons_from_the_management_library(monkeypatch):
    """The sampler only READS: clocks, power and the reason bits. Here the library is a stand-in that plays a run at full
    clock with the power cap active for a while."""
    from language_model_saes_b200.utils.clocks import ClockSampler

    calls = {"n": 0}
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlInit = lambda: None
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("gpu", i)
    fake.nvmlDeviceGetHandleByUUID = lambda u: ("gpu", u)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965
    fake.nvmlDeviceGetPowerUsage = lambda h: 950_000  # milliwatts

    def clock(h, kind):
        calls["n"] += 1
        return 1965 if calls["n"] % 4 else 1410

    fake.nvmlDeviceGetClockInfo = clock
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0x4 if calls["n"] > 3 else 0  # sw_power_cap
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda i: types.SimpleNamespace(uuid=None))
    s = ClockSampler(0, period_s=0.002)
    s.start()
    time.sleep(0.05)
    out = s.stop()
    assert out["sm_max_mhz"] == 1965 and out["sm_mhz"] == 1965 and out["samples"] >= 8
    assert out["reasons"] == ["sw_power_cap"] and out["power_w_max"] == pytest.approx(950.0)
    assert not any(name.startswith("nvmlDeviceSet") or "Reset" in name for name in dir(fake))  # nothing of the kind was needed


@distributed_test(nproc_per_node=2, backend="gloo")
def test_bucketed_gradient_reduction_averages_every_gradient_once():
    import torch.distributed as dist

    from language_model_saes_b200.parallel.data_parallel import reduce_gradients

    r = dist.get_rank()
    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.zeros(n)) for n in (5, 300, 7)] + [torch.nn.Parameter(torch.zeros(4, dtype=torch.float64))]
    params.append(torch.nn.Parameter(torch.zeros(3)))  # stays without a gradient
    for i, p in enumerate(params[:-1]):
        p.grad = torch.full_like(p, float(i + 1) * (r + 1))
    reduce_gradients(params, dist.group.WORLD, bucket_bytes=1024)  # several buckets, one dtype change
    for i, p in enumerate(params[:-1]):
        assert torch.allclose(p.grad, torch.full_like(p, float(i + 1) * 1.5)), i
    assert params[-1].grad is None
    reduce_gradients(params, dist.group.WORLD, average=False)
    assert torch.allclose(params[0].grad, torch.full_like(params[0], 3.0))
    reduce_gradients(params, None)  # no group: untouched
    assert torch.allclose(params[0].grad, torch.full_like(params[0], 3.0))


def test_topk_cross_layer_transcoder_becomes_a_jumprelu_one_with_the_same_codes():
    from language_model_saes_b200.models.clt import CLTConfig, CrossLayerTranscoder
    from language_model_saes_b200.utils.topk_to_jumprelu_conversion import topk_to_jumprelu_conversion

    torch.manual_seed(0)
    L, d, F, k, B = 2, 16, 64, 4, 128
    cfg = CLTConfig(hook_points_in=["i0", "i1"], hook_points_out=["o0", "o1"], d_model=d, expansion_factor=F / d, act_fn="batchlayertopk", top_k=k,
                    device="cpu", dtype=torch.float32, norm_activation="inference")  # fmt: skip
    m = CrossLayerTranscoder(cfg)
    m.init_parameters()
    with torch.no_grad():
        m.W_E.mul_(6.0)
    g = torch.Generator().manual_seed(1)
    batches = [{f"{io}{l}": torch.randn(B, d, generator=g) for io in "io" for l in range(L)} | {"tokens": torch.ones(B, dtype=torch.long)} for _ in range(2)]
    x, enc_kw, _ = m.prepare_input(m.normalize_activations(batches[0]))
    before = m.encode(x, **enc_kw)
    assert int((before != 0).sum()) == k * B
    out = topk_to_jumprelu_conversion(m, iter(batches))
    assert out is m and m.cfg.act_fn == "jumprelu" and not m.cfg.sparsity_include_decoder_norm
    after = m.encode(x, **enc_kw)
    # the threshold is the smallest kept score of that batch: the same entries fire (up to the one that sits on it)
    assert abs(int((after != 0).sum()) - k * B) <= 1
    agree = ((after != 0) == (before != 0)).float().mean()
    assert float(agree) > 0.9999
    both = (after != 0) & (before != 0)
    assert torch.allclose(after[both], before[both], rtol=1e-5, atol=1e-6)


def test_misc_helpers():
    from language_model_saes_b200.utils import misc

    for name, dt in (("float32", torch.float32), ("torch.bfloat16", torch.bfloat16), ("fp16", torch.float16), ("torch.float", torch.float32)):
        if name in misc.str_dtype_map:
            assert misc.convert_str_to_torch_dtype(name) is dt
    assert misc.convert_str_to_torch_dtype(misc.convert_torch_dtype_to_str(torch.bfloat16)) is torch.bfloat16
    with pytest.raises(ValueError, match="Unsupported data type"):
        misc.convert_str_to_torch_dtype("float7")
    with pytest.raises(ValueError, match="Unsupported data type"):
        misc.convert_torch_dtype_to_str(torch.complex64)
    t = torch.arange(12).view(3, 4)
    assert misc.tensor_id(t) == misc.tensor_id(t.view(3, 4)) and misc.tensor_id(t) != misc.tensor_id(t.t()) != misc.tensor_id(t[1:])
    assert misc.pad_and_truncate_tokens(torch.tensor([[1, 2, 3]]), 5, pad_token_id=9).tolist() == [[1, 2, 3, 9, 9]]
    assert misc.pad_and_truncate_tokens(torch.tensor([[1, 2, 3]]), 2).tolist() == [[1, 2]]
    assert misc.get_slice_length(slice(2, None, 3), 10) == 3 and misc.get_slice_length(slice(-2, None), 10) == 2
    assert misc.is_master()

    class Tok:
        def __call__(self, text, return_tensors=None):
            return types.SimpleNamespace(input_ids=torch.tensor([[len(w) for w in text.split()]]))

    assert misc.ensure_tokenized("ab cde f", Tok()).tolist() == [2, 3, 1]
    assert misc.ensure_tokenized(torch.tensor([[4, 5]]), None).tolist() == [4, 5]
    assert misc.ensure_tokenized([7, 8, 9], None).dtype == torch.long
    with pytest.raises(TypeError):
        misc.ensure_tokenized(3.5, None)


def test_activation_norm_is_the_mean_row_norm_of_the_first_batches():
    from language_model_saes_b200.utils.misc import calculate_activation_norm

    g = torch.Generator().manual_seed(0)
    batches = [{"a": torch.randn(10, 8, generator=g) * (i + 1), "b": torch.randn(10, 8, generator=g)} for i in range(5)]
    got = calculate_activation_norm(iter(batches), ["a", "b"], batch_num=3)
    want = torch.cat([b["a"] for b in batches[:3]]).norm(dim=-1).mean()
    assert got["a"] == pytest.approx(float(want), rel=1e-5) and set(got) == {"a", "b"}
    with pytest.warns(UserWarning, match="ended before"):
        short = calculate_activation_norm(iter(batches[:2]), ["b"], batch_num=8)
    assert short["b"] == pytest.approx(float(torch.cat([b["b"] for b in batches[:2]]).norm(dim=-1).mean()), rel=1e-5)


def test_resource_loaders_shard_datasets_and_pick_backends(tiny_lm_workspace):
    from language_model_saes_b200 import resource_loaders as R
    from language_model_saes_b200.config import DatasetConfig

    cfg = DatasetConfig(dataset_name_or_path=str(tiny_lm_workspace / "data"), is_dataset_on_disk=True)
    ds, meta = R.load_dataset(cfg)
    assert meta is None and len(ds) == 64
    part, meta = R.load_dataset(cfg, n_shards=4, start_shard=1)
    assert meta == {"shard_idx": 1, "n_shards": 4} and len(part) == 16 and part[0]["text"] == ds[16]["text"]  # contiguous shards
    assert len(R.load_dataset_shard(cfg, 3, 4)) == 16
    assert R.infer_model_backend("Qwen/Qwen2.5-VL-7B-Instruct") == "qwen_vl" and R.infer_model_backend("EleutherAI/pythia-160m") == "hooked"
    from conftest import tiny_lm_config

    lm = R.load_model(tiny_lm_config(tiny_lm_workspace))
    assert type(lm).__name__ == "HookedLanguageModel"
    bad = tiny_lm_config(tiny_lm_workspace).model_copy(update={"backend": "nope"})
    with pytest.raises(ValueError, match="unknown backend"):
        R.load_model(bad)


def test_conversion_runner_saves_a_jumprelu_cross_layer_transcoder(tmp_path):
    from safetensors.torch import save_file

    from language_model_saes_b200 import ActivationFactoryActivationsSource, ActivationFactoryConfig, ActivationFactoryTarget
    from language_model_saes_b200.models.clt import CLTConfig, CrossLayerTranscoder
    from language_model_saes_b200.models.sparse_dictionary import SparseDictionary
    from language_model_saes_b200.runners import PretrainedSAE
    from language_model_saes_b200.runners.topk_to_jumprelu_conversion import ConvertTopKToJumpReLUSettings, convert_topk_to_jumprelu

    torch.manual_seed(0)
    L, d, F, k = 2, 16, 64, 4
    hooks_in, hooks_out = [f"blocks.{l}.ln2.hook_normalized" for l in range(L)], [f"blocks.{l}.hook_mlp_out" for l in range(L)]
    cfg = CLTConfig(hook_points_in=hooks_in, hook_points_out=hooks_out, d_model=d, expansion_factor=F / d, act_fn="batchlayertopk", top_k=k,
                    device="cpu", dtype=torch.float32, norm_activation="inference")  # fmt: skip
    m = CrossLayerTranscoder(cfg)
    m.init_parameters()
    with torch.no_grad():
        m.W_E.mul_(6.0)
    src = tmp_path / "topk"
    src.mkdir()
    m.save_pretrained(src)
    m.cfg.save_hyperparameters(src)
    g = torch.Generator().manual_seed(2)
    tokens = torch.randint(3, 50, (8, 12), generator=g)
    for hp in hooks_in + hooks_out:
        (tmp_path / "cache" / hp).mkdir(parents=True)
        for c in range(2):
            save_file({"activation": torch.randn(8, 12, d, generator=g), "tokens": tokens, "mask": torch.ones(8, 12, dtype=torch.bool),
                       "attention_mask": torch.ones(8, 12, dtype=torch.bool)}, str(tmp_path / "cache" / hp / f"chunk-{c}.safetensors"))  # fmt: skip
    factory = ActivationFactoryConfig(
        sources=[ActivationFactoryActivationsSource(name="cache", path=str(tmp_path / "cache"), device="cpu", num_workers=0, prefetch=None)],
        target=ActivationFactoryTarget.ACTIVATIONS_1D, hook_points=hooks_in + hooks_out, batch_size=64)  # fmt: skip
    out = tmp_path / "jumprelu"
    out.mkdir()
    convert_topk_to_jumprelu(ConvertTopKToJumpReLUSettings(sae=PretrainedSAE(pretrained_name_or_path=str(src), device="cpu", dtype=torch.float32),
                                                           sae_name="clt-j", sae_series="t", activation_factory=factory, device_type="cpu",
                                                           exp_result_path=str(out)))  # fmt: skip
    back = SparseDictionary.from_pretrained(str(out), device="cpu", dtype=torch.float32, fold_activation_scale=False)
    assert back.cfg.act_fn == "jumprelu" and not back.cfg.sparsity_include_decoder_norm
    x = torch.randn(64, L, d, generator=g)
    l0 = float((back.encode(x) != 0).sum()) / 64
    assert 0.5 * k < l0 < 2.0 * k  # about k codes per token on fresh data from the same distribution
    assert torch.equal(back.W_E, m.W_E)
