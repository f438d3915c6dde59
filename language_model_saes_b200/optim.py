"""Learning-rate schedules, SparseAdam, gradient norms and clipping.

Schedules and their closed forms, the masked Adam variant and the (unusual) gradient-norm definition follow
optim.py of the reference project (:23-139 schedules, :142-254 SparseAdam, :257-292 norm and clipping).
Differences: parameters are local shards, so the norm sums squares over feature shards explicitly and, under
data parallelism, gradients are expected to be already reduced (``parallel.data_parallel.reduce_gradients``)
before norms are taken; the norm and the clip factor stay on the device (no host sync) unless the caller
converts them.
"""

from __future__ import annotations

import math
from typing import Any, Iterable

import torch
import torch.distributed as dist
import torch.optim.lr_scheduler as lr_scheduler
from torch.optim import Optimizer

from .parallel.mesh import mesh_dim_size, mesh_group


def schedule_lambda(name: str | None, **kw: Any):
    """Multiplicative learning-rate factor as a function of the step index for the named schedule."""
    name = (name or "constant").lower()
    warm = kw.get("warm_up_steps", 0)
    total = kw.get("training_steps")
    if name == "constant":
        return lambda s: 1.0
    assert total is not None, "training_steps must be provided"
    if name == "constantwithwarmup":
        cool = kw.get("cool_down_steps", 0)
        end = kw.get("lr_end_ratio", 0.0)

        def f(s: int) -> float:
            terms = [1.0]
            if warm > 0:
                terms.append((s + 1) / warm)
            if cool > 0:
                terms.append(end + (1 - end) / cool * max(total - s, 1))
            return min(terms)

        return f
    if name == "constantwithwarmupsmooth":
        gamma = 0.5
        cool_start = total - int(1.5 * warm)

        def f(s: int) -> float:
            if s < gamma * warm:
                return 2 * (s + 1) / (warm * (1 + gamma))
            if s < warm:
                return 1 - ((s / warm - 1) ** 2) / (1 - gamma**2)
            if s < cool_start:
                return 1.0
            return 0.5 * (1 + math.cos(math.pi * (s - cool_start) / (total - cool_start)))

        return f
    if name == "linearwarmupdecay":
        return lambda s: (s + 1) / warm if s < warm else (total - s) / (total - warm)
    if name == "cosineannealing":
        # closed form of torch's CosineAnnealingLR(T_max=training_steps, eta_min=lr_end) when nothing else touches the
        # rate: eta_min + (base - eta_min) * (1 + cos(pi * s / T_max)) / 2, as a factor of the base rate
        eta_min, base = kw.get("lr_end", 0.0), kw.get("base_lr")
        assert eta_min == 0.0 or base, "a non-zero lr_end needs base_lr to express the schedule as a factor"
        floor = eta_min / base if base else 0.0
        return lambda s: floor + (1 - floor) * 0.5 * (1 + math.cos(math.pi * s / total))
    if name == "cosineannealingwarmup":
        end = kw.get("lr_end", 0.0)

        def f(s: int) -> float:
            if s < warm:
                return (s + 1) / warm
            return end + 0.5 * (1 - end) * (1 + math.cos(math.pi * (s - warm) / (total - warm)))

        return f
    if name == "exponentialwarmup":
        end = kw.get("lr_end", 1 / 32)
        return lambda s: (s + 1) / warm if s < warm else math.pow(end, (s - warm) / (total - warm))
    raise ValueError(f"Unsupported scheduler: {name}")


def get_scheduler(scheduler_name: str | None, optimizer: Optimizer, **kwargs: Any):
    name = (scheduler_name or "constant").lower()
    if name == "cosineannealing":
        return lr_scheduler.CosineAnnealingLR(optimizer, T_max=kwargs["training_steps"], eta_min=kwargs.get("lr_end", 0))
    if name == "cosineannealingwarmrestarts":
        t0 = kwargs["training_steps"] // kwargs.get("num_cycles", 1)
        return lr_scheduler.CosineAnnealingWarmRestarts(optimizer, T_0=t0, eta_min=kwargs.get("lr_end", 0))
    return lr_scheduler.LambdaLR(optimizer, lr_lambda=schedule_lambda(name, **kwargs))


class SparseAdam(Optimizer):
    """Adam that touches a parameter element only where its gradient is non-zero: both moments decay every
    step, but gain a contribution, and the parameter moves, only at non-zero-gradient positions; a parameter
    whose whole gradient is zero is skipped (its step counter does not advance)."""

    def __init__(self, params, lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0):  # fmt: skip
        if lr < 0 or eps < 0 or weight_decay < 0 or not (0 <= betas[0] < 1) or not (0 <= betas[1] < 1):
            raise ValueError("invalid SparseAdam hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None or not bool(p.grad.any()):
                    continue
                g = p.grad
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["step"] += 1
                if group["weight_decay"] != 0:
                    g = g.add(p, alpha=group["weight_decay"])
                mask = g != 0
                m = st["exp_avg"].mul_(b1)
                v = st["exp_avg_sq"].mul_(b2)
                m.add_(torch.where(mask, (1 - b1) * g, torch.zeros_like(g)))
                v.add_(torch.where(mask, (1 - b2) * g * g, torch.zeros_like(g)))
                step_size = group["lr"] * math.sqrt(1 - b2 ** st["step"]) / (1 - b1 ** st["step"])
                upd = step_size * m / (v.sqrt() + group["eps"])
                p.sub_(torch.where(mask, upd, torch.zeros_like(upd)))
        return loss


def compute_grad_norm(params: Iterable[torch.nn.Parameter], device_mesh=None, sharded: Iterable[bool] | None = None) -> torch.Tensor:
    """``||g||_2 / sqrt(nnz(g))`` over all given parameters, as a 0-d device tensor.

    ``sharded[i]`` says whether parameter i is split over the ``model`` mesh dimension (its squares and
    non-zero count are summed over shards) or replicated there (counted once). Defaults to all-sharded, which
    matches the reference's behaviour for its weight matrices.
    """
    params = [p for p in params if p.grad is not None]
    assert params, "No gradients found"
    flags = list(sharded) if sharded is not None else [True] * len(params)
    dev = params[0].grad.device
    acc = torch.zeros(4, device=dev, dtype=torch.float32)  # sq_sharded, nnz_sharded, sq_repl, nnz_repl
    for p, sh in zip(params, flags):
        g = p.grad.float()
        o = 0 if sh else 2
        acc[o] += g.pow(2).sum()
        acc[o + 1] += (g != 0).sum()
    if mesh_dim_size(device_mesh, "model") > 1:
        part = acc[:2].clone()
        dist.all_reduce(part, group=mesh_group(device_mesh, "model"))
        acc[:2] = part
    return (acc[0] + acc[2]).sqrt() / (acc[1] + acc[3]).sqrt()


def clip_grad_norm(params: Iterable[torch.nn.Parameter], max_norm: float, device_mesh=None,
                   sharded: Iterable[bool] | None = None) -> torch.Tensor:  # fmt: skip
    """Scale gradients by ``max_norm / (norm + 1e-6)`` when the norm exceeds ``max_norm``; returns the norm.
    The comparison happens on the device: the factor is ``where(norm > max, max / (norm + 1e-6), 1)``."""
    params = [p for p in params if p.grad is not None]
    norm = compute_grad_norm(params, device_mesh, sharded)
    if math.isfinite(max_norm):
        factor = torch.where(norm > max_norm, max_norm / (norm + 1e-6), torch.ones_like(norm))
        for p in params:
            p.grad.mul_(factor.to(p.grad.dtype))
    return norm
