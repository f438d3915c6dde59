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
