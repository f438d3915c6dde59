"""JumpReLU and its straight-through threshold gradient against the written definition (activation_functions.py:15-140 of
the reference project): forward ``x * 1[x > theta]``, ``dx = dy * 1[x > theta]``, and a rectangle-window estimate for
``theta`` that reaches the stored ``log theta`` through the chain rule."""

import pytest
import torch

from language_model_saes_b200.activation_functions import JumpReLU, STEFunction


def _manual(x, theta, dy, w, reduce_dims):
    mask = x > theta
    hit = ((x - theta).abs() < 0.5 * w) & (x > 0)
    dtheta = (torch.where(hit, -theta / w, torch.zeros(())) * dy).sum(reduce_dims)
    return x * mask, dy * mask, dtheta


def test_forward_and_both_gradients_of_a_feature_threshold():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 5, 16, generator=g, dtype=torch.float64).requires_grad_()
    log_theta = (torch.rand(16, generator=g, dtype=torch.float64) - 0.7).requires_grad_()
    dy = torch.randn(6, 5, 16, generator=g, dtype=torch.float64)
    w = 0.8  # wide enough that many entries fall in the window
    y = STEFunction.apply(x, log_theta.exp(), w, (-1,))
    y.backward(dy)
    want_y, want_dx, want_dtheta = _manual(x.detach(), log_theta.detach().exp(), dy, w, (0, 1))
    assert torch.equal(y, want_y)
    assert torch.equal(x.grad, want_dx)
    assert want_dtheta.abs().sum() > 0
    assert torch.allclose(log_theta.grad, want_dtheta * log_theta.detach().exp())  # d theta / d log theta = theta


def test_negative_inputs_never_move_a_threshold():
    # a threshold below half a window has part of its window at negative inputs; those do not count
    x = torch.tensor([[-0.05, 0.05, 0.2]], dtype=torch.float64)
    theta = torch.full((3,), 0.1, dtype=torch.float64, requires_grad=True)
    STEFunction.apply(x, theta, 0.5, (-1,)).backward(torch.ones(1, 3, dtype=torch.float64))
    assert theta.grad.tolist() == [0.0, pytest.approx(-0.2), pytest.approx(-0.2)]


def test_layer_by_feature_thresholds_keep_both_axes():
    g = torch.Generator().manual_seed(1)
    act = JumpReLU(0.6, shape=(3, 8), dims_to_keep_in_bwd=(-2, -1), dtype=torch.float64)
    with torch.no_grad():
        act.log_jumprelu_threshold.copy_(torch.rand(3, 8, generator=g, dtype=torch.float64) - 0.8)
    x = torch.randn(10, 3, 8, generator=g, dtype=torch.float64).requires_grad_()
    dy = torch.randn(10, 3, 8, generator=g, dtype=torch.float64)
    act(x).backward(dy)
    theta = act.get_jumprelu_threshold().detach()
    _, want_dx, want_dtheta = _manual(x.detach(), theta, dy, 0.6, (0,))
    assert torch.equal(x.grad, want_dx)
    assert act.log_jumprelu_threshold.grad.shape == (3, 8)
    assert torch.allclose(act.log_jumprelu_threshold.grad, want_dtheta * theta)
    with pytest.raises(AssertionError):
        JumpReLU(0.6, shape=(3, 8), dtype=torch.float64)  # one kept axis for a two-axis threshold


def test_the_module_computes_in_its_own_dtype_and_returns_the_callers():
    act = JumpReLU(0.1, shape=(4,), dtype=torch.float32)
    with torch.no_grad():
        act.log_jumprelu_threshold.fill_(-1.0)
    x = torch.tensor([[0.2, 0.5, -1.0, 0.36]], dtype=torch.bfloat16)
    y = act(x)
    assert y.dtype == torch.bfloat16
    assert y.tolist() == [[0.0, 0.5, 0.0, 0.0]]  # exp(-1) = 0.3679 > 0.36
    assert act.dim_maps()["log_jumprelu_threshold"].local_shape((4,), None) == (4,)
    assert act.override_dtypes() == {"log_jumprelu_threshold": torch.float32}
