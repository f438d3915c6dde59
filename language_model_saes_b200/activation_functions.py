"""JumpReLU with a straight-through estimator for its threshold.

Semantics of activation_functions.py:15-140 in the reference project:
forward ``y = x * 1[x > theta]`` with ``theta = exp(log_theta)``; backward ``dx = dy * 1[x > theta]`` and
``dtheta = sum dy * (-theta / w) * 1[|x - theta| < w/2 and x > 0]`` (rectangle window of width ``w``), summed
over every dimension that ``theta`` does not have. ``log_jumprelu_threshold`` is sharded along its last
dimension under feature (``model``) parallelism; this module holds the local shard.
"""

from __future__ import annotations

import torch

from .parallel.mesh import DimMap


class STEFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input: torch.Tensor, threshold: torch.Tensor, window: float, dims_to_keep_in_bwd: tuple[int, ...]):
        mask = input > threshold
        ctx.save_for_backward(input, threshold, mask)
        ctx.window = float(window)
        ctx.keep = tuple(dims_to_keep_in_bwd)
        return input * mask

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        input, threshold, mask = ctx.saved_tensors
        w = ctx.window
        in_window = ((input - threshold).abs() < 0.5 * w) & (input > 0)
        grad_thr = torch.where(in_window, -threshold / w, torch.zeros((), dtype=input.dtype, device=input.device)) * grad_output
        nd = grad_thr.ndim
        keep = {d % nd for d in ctx.keep}
        reduce_dims = tuple(i for i in range(nd) if i not in keep)
        if reduce_dims:
            grad_thr = grad_thr.sum(dim=reduce_dims)
        return grad_output * mask, grad_thr, None, None


class FusedSTEFunction(torch.autograd.Function):
    """The same function as ``STEFunction`` for thresholds that cover the trailing dimensions of a contiguous CUDA
    input, as two streaming sm_100a kernels (``ops/csrc/jumprelu.cu``): the mask is never materialised, the backward
    reads ``x`` and ``dy`` once, writes ``dx`` once and sends the rare window hits to fp32 atomics. Takes
    ``log_theta`` (the parameter itself), so ``exp`` and its chain rule are inside the kernels too."""

    @staticmethod
    def forward(ctx, input: torch.Tensor, log_threshold: torch.Tensor, window: float):
        from .ops import native

        ctx.save_for_backward(input, log_threshold)
        ctx.window = float(window)
        return native.load().jumprelu(input, log_threshold.contiguous(), None, None, float(window))

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        from .ops import native

        input, log_threshold = ctx.saved_tensors
        dlog = torch.zeros(log_threshold.numel(), dtype=torch.float32, device=input.device)
        dx = native.load().jumprelu(input, log_threshold.contiguous(), grad_output.contiguous(), dlog, ctx.window)
        return dx, dlog.view_as(log_threshold).to(log_threshold.dtype), None


def _fusable(input: torch.Tensor, log_threshold: torch.Tensor, keep: tuple[int, ...]) -> bool:
    n = log_threshold.ndim
    return (
        input.is_cuda and input.is_contiguous() and input.dtype in (torch.float32, torch.bfloat16)
        and log_threshold.numel() % 4 == 0 and log_threshold.numel() > 0
        and tuple(input.shape[-n:]) == tuple(log_threshold.shape)
        and tuple(sorted(d % input.ndim for d in keep)) == tuple(range(input.ndim - n, input.ndim))
    )  # fmt: skip


class JumpReLU(torch.nn.Module):
    def __init__(
        self,
        jumprelu_threshold_window: float,
        *,
        shape: tuple[int, ...],
        dims_to_keep_in_bwd: tuple[int, ...] = (-1,),
        device: torch.device | str | None = None,
        dtype: torch.dtype,
        device_mesh=None,
    ):
        super().__init__()
        self.jumprelu_threshold_window = jumprelu_threshold_window
        self.shape = tuple(shape)
        self.dims_to_keep_in_bwd = tuple(dims_to_keep_in_bwd)
        self.device_mesh = device_mesh
        self.dtype = dtype
        assert len(self.dims_to_keep_in_bwd) == len(self.shape), (
            f"dims_to_keep_in_bwd must have the same length as shape, got {self.dims_to_keep_in_bwd} and {self.shape}"
        )
        local_shape = self.dim_maps()["log_jumprelu_threshold"].local_shape(self.shape, device_mesh)
        self.log_jumprelu_threshold = torch.nn.Parameter(torch.empty(local_shape, device=device, dtype=dtype))

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x = input.to(self.dtype)
        if _fusable(x, self.log_jumprelu_threshold, self.dims_to_keep_in_bwd):
            out = FusedSTEFunction.apply(x, self.log_jumprelu_threshold, self.jumprelu_threshold_window)
        else:
            out = STEFunction.apply(x, self.log_jumprelu_threshold.exp(), self.jumprelu_threshold_window, self.dims_to_keep_in_bwd)
        return out.to(input.dtype)

    def get_jumprelu_threshold(self) -> torch.Tensor:
        return self.log_jumprelu_threshold.exp()

    def dim_maps(self) -> dict[str, DimMap]:
        return {"log_jumprelu_threshold": DimMap({"model": len(self.shape) - 1})}

    def override_dtypes(self) -> dict[str, torch.dtype]:
        return {"log_jumprelu_threshold": self.dtype}
