"""Training loop.

Configuration fields, schedules (k, l1 coefficient, learning rate), checkpoint layout and logged keys follow
trainer.py of the reference project (TrainerConfig :51-125, checkpoints :155-307, initialisation :309-401,
dead-feature statistics :403-454, step :456-510, logging :512-562, fit :576-671).

Two execution paths share this loop:

* the fused path (``ops.fused_step.FusedTopKSAEStep``) for TopK sparse autoencoders on CUDA: one fixed
  sequence of hand-written kernels per step, no autograd graph, no dense [batch, d_sae] tensor;
* the generic path for every other model / loss: autograd over the model's ``compute_loss``, gradients
  averaged explicitly over the ``data`` mesh dimension, torch or SparseAdam optimizer.

Neither path synchronises with the host inside a step: the progress-bar loss, token counts and metrics are read
back only every ``log_frequency`` steps.
"""

from __future__ import annotations

import json
import math
import os
from pathlib import Path
from typing import Any, Callable, Iterable, Iterator, Literal, Tuple

import torch
import torch.distributed as dist
from pydantic import ConfigDict, Field
from torch import Tensor
from torch.optim import Adam, Optimizer

from .config import BaseConfig, OptionalTorchDType
from .metrics import (
    ExplainedVarianceMetric,
    FrequencyMetric,
    GradientNormMetric,
    L0Metric,
    L2NormErrorMetric,
    LossMetric,
    MeanFeatureActMetric,
    Metric,
    ModelSpecificMetric,
)
from .models.sparse_dictionary import SparseDictionary
from .optim import SparseAdam, clip_grad_norm, get_scheduler
from .parallel.data_parallel import reduce_gradients
from .parallel.health import PeerLost
from .parallel.mesh import is_primary_rank, mesh_dim_size, mesh_group
from .utils.logging import get_distributed_logger, log_metrics
from .utils.tensor_specs import apply_token_mask
from .utils.timer import timer

logger = get_distributed_logger("trainer")


class TrainerConfig(BaseConfig):
    model_config = ConfigDict(arbitrary_types_allowed=True)

    l1_coefficient: float | None = 0.00008
    l1_coefficient_warmup_steps: int | float = 0.1
    lp_coefficient: float | None = None
    auxk_coefficient: float | None = None
    amp_dtype: OptionalTorchDType = Field(default=torch.bfloat16, exclude=True, validate_default=False)
    sparsity_loss_type: Literal["power", "tanh", "tanh-quad", None] = None
    tanh_stretch_coefficient: float = 4.0
    frequency_scale: float = 0.01
    p: int = 1
    initial_k: int | float | None = None
    k_warmup_steps: int | float = 0.1
    k_cold_booting_steps: int | float = 0
    k_schedule_type: Literal["linear", "exponential"] = "linear"
    k_exponential_factor: float = 3.0
    k_aux: int = 512
    dead_threshold: float = 10_000_000
    skip_metrics_calculation: bool = False
    gradient_accumulation_steps: int = 1

    lr: float | dict[str, float] = 0.0004
    betas: Tuple[float, float] = (0.9, 0.999)
    optimizer_class: Literal["adam", "sparseadam"] = "adam"
    optimizer_foreach: bool = True
    lr_scheduler_name: Literal[
        "constant", "constantwithwarmup", "linearwarmupdecay", "cosineannealing", "cosineannealingwarmup", "exponentialwarmup"
    ] = "constantwithwarmup"
    lr_end_ratio: float = 1 / 32
    lr_warm_up_steps: int | float = 5000
    lr_cool_down_steps: int | float = 0.2
    jumprelu_lr_factor: float = 1.0
    clip_grad_norm: float = 0.0
    feature_sampling_window: int = 1000
    total_training_tokens: int = 300_000_000

    log_frequency: int = 1000
    eval_frequency: int = 1000
    n_checkpoints: int = 10
    check_point_save_mode: Literal["log", "linear"] = "log"

    from_pretrained_path: str | None = None
    exp_result_path: str = "results"

    prefetch_to_device: bool = True
    """Copy the next host batch to the GPU on a side stream while the current step runs."""
    shard_host_copies: bool = True
    """With ``prefetch_to_device`` under feature (``model``) parallelism: every rank of a replica copies 1/n of each
    host batch and the rows are all-gathered over NVLink. Requires what the activation pipeline guarantees: the ranks
    of one replica see the same batches."""
    heartbeat_timeout_s: float | None = None
    """Multi-process runs: publish a heartbeat every step through the process group's store and, before each step, raise
    ``parallel.health.PeerLost`` when a peer has left or has been silent for this long (None: off)."""
    checkpoint_on_failure: bool = False
    """Save a full trainer checkpoint under ``exp_result_path`` when ``fit`` ends with an exception (a lost peer included;
    only this rank's view is saved then, without collectives, so it is meant for unsharded or data-parallel models)."""
    use_fused_kernels: bool = True
    """Run eligible models (TopK SAE, MSE loss, Adam, CUDA) on the fused kernel path."""
    use_peer_memory_collectives: bool = True
    """Under feature sharding on the fused path, exchange candidates / partial reconstructions with the fused
    peer-memory kernels (NVLink loads and stores issued by the compute kernels) instead of NCCL collectives."""

    def model_post_init(self, __context):
        super().model_post_init(__context)
        Path(self.exp_result_path, "checkpoints").mkdir(parents=True, exist_ok=True)
        assert self.lr_end_ratio <= 1, "lr_end_ratio must be in 0 to 1 (inclusive)."
        if self.from_pretrained_path is not None:
            assert os.path.exists(self.from_pretrained_path), f"from_pretrained_path {self.from_pretrained_path} does not exist"


class WandbConfig(BaseConfig):
    wandb_project: str = "gpt2-sae-training"
    exp_name: str | None = None
    wandb_entity: str | None = None
    wandb_run_id: str | None = None
    wandb_resume: Literal["allow", "must", "never", "auto"] = "never"


class _DevicePrefetcher:
    """Iterator over device batches that keeps ONE batch in flight: while step ``i`` computes, the host->device copy
    of batch ``i + 1`` runs on its own stream (the copy engine), so the copy costs no step time. Host tensors should be
    pinned, otherwise the copy is synchronous on the host. Batches that are already on the device pass through.

    ``replica_group``: ranks that hold the SAME host batch (the feature-parallel ranks of one data-parallel replica).
    Each of them then copies only its 1/n of the rows over PCIe and the rows are all-gathered over NVLink on the copy
    stream: n times less host-memory and PCIe traffic per step, which is what bounds an 8-GPU node when every rank pulls
    the whole batch."""

    def __init__(self, host_iter: Iterator[dict[str, Any]], device: torch.device, replica_group=None):
        self.host_iter = host_iter
        self.device = device
        self.copy_stream = torch.cuda.Stream(device=device)
        self.group = replica_group if replica_group is not None and dist.get_world_size(replica_group) > 1 else None
        self._ready: tuple[dict[str, Any], torch.cuda.Event | None] | None = None
        self._exhausted = False
        self._issue()

    def _move(self, v: Tensor) -> Tensor:
        if self.group is not None:
            n, r = dist.get_world_size(self.group), dist.get_rank(self.group)
            if v.ndim >= 1 and v.shape[0] % n == 0 and v.shape[0] >= n and v.numel() * v.element_size() >= (1 << 20):
                rows = v.shape[0] // n
                part = v[r * rows : (r + 1) * rows].to(self.device, non_blocking=True)
                out = torch.empty(v.shape, dtype=v.dtype, device=self.device)
                dist.all_gather_into_tensor(out.view(-1), part.reshape(-1), group=self.group)
                return out
        return v.to(self.device, non_blocking=True)

    def _issue(self) -> None:
        try:
            batch = next(self.host_iter)
        except StopIteration:
            self._ready, self._exhausted = None, True
            return
        batch = Trainer._mask_summary(batch)
        if not any(isinstance(v, Tensor) and v.device.type == "cpu" for v in batch.values()):
            self._ready = (batch, None)
            return
        with torch.cuda.stream(self.copy_stream):
            moved = {k: (self._move(v) if isinstance(v, Tensor) and v.device.type == "cpu" else v) for k, v in batch.items()}
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        self._ready = (moved, ev)

    def __iter__(self):
        return self

    def __next__(self) -> dict[str, Any]:
        if self._ready is None:
            raise StopIteration
        batch, ev = self._ready
        self._issue()  # next copy starts before this batch's kernels are launched
        if ev is not None:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(ev)
            for v in batch.values():
                if isinstance(v, Tensor) and v.is_cuda:
                    v.record_stream(cur)
        return batch


class _LossReader:
    """Reads the loss of every logged step back to the host without stalling the launch of the next step: the value is
    copied into one of two pinned scalars on the producing stream and picked up one step later, when its copy has long
    finished, so the host stays one step ahead of the device instead of waiting for each step to end. On CPU tensors it
    is an ordinary read."""

    def __init__(self):
        self._slots: list[tuple[Tensor, Any] | None] = [None, None]
        self._pinned: list[Tensor | None] = [None, None]
        self._n = 0

    def _take(self, slot: int) -> float | None:
        entry = self._slots[slot]
        if entry is None:
            return None
        host, ev = entry
        ev.synchronize()
        self._slots[slot] = None
        if host[1] != 0:
            from .ops import sae_kernels as K

            code = int(host[1])
            err = (K.CollectiveTimeout if code == 5 else K.KernelStatusError)(
                f"kernel status {code} ({K._STATUS_NAMES.get(code, 'unknown')}), detail={int(host[2])}, block={int(host[3])}, aux={int(host[4])}"
            )
            err.code = code
            raise err
        return float(host[0])

    def push(self, loss: Tensor, status: Tensor | None = None) -> float | None:
        """Queue ``loss`` and return the most recent value whose copy has completed (None on the first call). ``status``
        (the kernels' int32 status word) travels with it: a recorded bounded-wait expiry raises when it is picked up."""
        if not loss.is_cuda:
            return float(loss)
        slot = self._n & 1
        self._n += 1
        if self._pinned[slot] is None:
            self._pinned[slot] = torch.empty(5, dtype=torch.float32, pin_memory=True)
        host = self._pinned[slot]
        host[:1].copy_(loss.detach().float().reshape(1), non_blocking=True)
        if status is not None:
            host[1:5].copy_(status[:4], non_blocking=True)  # int32 -> fp32: the codes are small integers
        else:
            host[1:5].zero_()
        ev = torch.cuda.Event()
        ev.record()
        self._slots[slot] = (host, ev)
        return self._take(slot ^ 1)

    def flush(self) -> float | None:
        """The last queued value (waits for it)."""
        vals = [self._take((self._n + i) & 1) for i in range(2)]
        vals = [v for v in vals if v is not None]
        return vals[-1] if vals else None


class Trainer:
    def __init__(self, cfg: TrainerConfig):
        self.cfg = cfg
        self.last_loss: float | None = None  # most recent loss value read back by fit()
        self.checkpoint_thresholds: list[int] = []
        self.total_training_steps: int = 0
        self.lr_warm_up_steps: int = 0
        self.lr_cool_down_steps: int = 0
        self.k_warmup_steps: int = 0
        self.k_cold_booting_steps: int = 0
        self.l1_coefficient_warmup_steps: int = 0
        self.cur_step: int = 0
        self.cur_tokens: int = 0
        self.optimizer: Optimizer | None = None
        self.scheduler = None
        self.wandb_logger = None
        self.metrics: list[Metric] = []
        self.tokens_since_last_activation: Tensor | None = None
        self.is_dead: Tensor | None = None
        self.fused = None  # FusedTopKSAEStep when the fused path is active
        self._fused_aux = None  # ops.fused_step.AuxK when the fused path trains with the Aux-K loss
        self._lr_lambda: Callable[[int], float] | None = None
        self._pending_optimizer_state: dict | None = None
        self._interval: dict[str, Any] = {}
        self._tokens_on_device: Tensor | None = None

    # ---- checkpoints -------------------------------------------------------------------------
    def save_checkpoint(self, sae: SparseDictionary, checkpoint_path: Path | str) -> None:
        """Model + optimizer + scheduler + trainer state under ``<path>/checkpoints/step_<N>/``. Beyond the
        reference's files it also writes ``extra_state.pt`` (dead-feature counters and RNG state), which
        older readers ignore."""
        self._before_parameters_leave(sae)
        ckpt_dir = Path(checkpoint_path) / "checkpoints" / f"step_{self.cur_step}"
        primary = is_primary_rank(sae.device_mesh)
        if primary:
            os.makedirs(ckpt_dir, exist_ok=True)
        if sae.device_mesh is not None and dist.is_initialized():
            dist.barrier()
        if primary:
            sae.cfg.save_hyperparameters(ckpt_dir)
        sae.save_checkpoint(ckpt_dir / "sae_weights.safetensors")
        opt_state = self._gather_optimizer_state(sae)
        if primary:
            torch.save(
                {
                    "cur_step": self.cur_step,
                    "cur_tokens": self.cur_tokens,
                    "total_training_steps": self.total_training_steps,
                    "lr_warm_up_steps": self.lr_warm_up_steps,
                    "lr_cool_down_steps": self.lr_cool_down_steps,
                    "k_warmup_steps": self.k_warmup_steps,
                    "k_cold_booting_steps": self.k_cold_booting_steps,
                    "l1_coefficient_warmup_steps": self.l1_coefficient_warmup_steps,
                    "checkpoint_thresholds": self.checkpoint_thresholds,
                    "cfg": self.cfg,
                },
                ckpt_dir / "trainer.pt",
            )
            if self.wandb_logger is not None:
                with open(ckpt_dir / "wandb_run_id.json", "w") as f:
                    json.dump({"wandb_run_id": self.wandb_logger.id}, f)
            if opt_state is not None:
                torch.save(opt_state, ckpt_dir / "optimizer.pt")
            if self.scheduler is not None:
                torch.save(self.scheduler.state_dict(), ckpt_dir / "scheduler.pt")
            extra = {"torch_rng": torch.get_rng_state()}
            if self.tokens_since_last_activation is not None:
                extra["tokens_since_last_activation"] = self.tokens_since_last_activation.cpu()
            torch.save(extra, ckpt_dir / "extra_state.pt")
        logger.info(f"Checkpoint saved to {ckpt_dir}")

    def _gather_optimizer_state(self, sae: SparseDictionary) -> dict | None:
        """Optimizer state with full (un-sharded) logical tensors, keyed by parameter name. Collective."""
        maps = sae.dim_maps()
        names = {id(p): n for n, p in sae.named_parameters()}

        def full(name: str, t: Tensor) -> Tensor:
            if sae.device_mesh is not None and name in maps and t.ndim > 0:
                t = maps[name].gather(t, sae.device_mesh)
            return t.detach().cpu().contiguous()

        if self.fused is not None:
            st = self.fused.optimizer_state()
            out = {"format": "by_name", "step": st["step"], "state": {}}
            for name, d in st.items():
                if name != "step":
                    out["state"][name] = {k: full(name, v) for k, v in d.items()}
            return out
        if self.optimizer is None:
            return None
        out = {"format": "by_name", "state": {}, "param_groups": [
            {k: v for k, v in g.items() if k != "params"} for g in self.optimizer.param_groups]}  # fmt: skip
        for p, st in self.optimizer.state.items():
            name = names[id(p)]
            out["state"][name] = {k: (full(name, v) if isinstance(v, Tensor) else v) for k, v in st.items()}
        return out

    def _load_optimizer_state(self, sae: SparseDictionary, sd: dict) -> None:
        maps = sae.dim_maps()

        def local(name: str, t: Tensor, like: Tensor) -> Tensor:
            if sae.device_mesh is not None and name in maps and t.ndim > 0 and tuple(t.shape) != tuple(like.shape):
                t = maps[name].shard(t, sae.device_mesh)
            return t.to(like.device)

        if self.fused is not None:
            params = dict(sae.named_parameters())
            st = {"step": sd.get("step", 0)}
            for name, d in sd["state"].items():
                if name in params:
                    st[name] = {k: local(name, v, params[name]) for k, v in d.items() if isinstance(v, Tensor) and v.ndim > 0}
                    if "step" in d and not st["step"]:
                        st["step"] = int(d["step"])
            self.fused.load_optimizer_state(st)
            return
        assert self.optimizer is not None
        for name, p in sae.named_parameters():
            if name in sd["state"]:
                self.optimizer.state[p] = {
                    k: (local(name, v, p).to(p.dtype if v.is_floating_point() and v.ndim > 0 else v.dtype) if isinstance(v, Tensor) else v)
                    for k, v in sd["state"][name].items()
                }

    @classmethod
    def from_checkpoint(cls, sae: SparseDictionary, checkpoint_path: str) -> "Trainer":
        ckpt_dir = Path(checkpoint_path)
        trainer_path = ckpt_dir / "trainer.pt"
        if not os.path.exists(trainer_path):
            raise ValueError(f"Trainer checkpoint not found at {trainer_path}")
        state = torch.load(trainer_path, map_location="cpu", weights_only=False)
        cfg = state.get("cfg")
        if cfg is None:
            raise ValueError("Checkpoint does not contain trainer config")
        trainer = cls(cfg)
        trainer.cfg.from_pretrained_path = checkpoint_path
        for key in ("cur_step", "cur_tokens", "total_training_steps", "lr_warm_up_steps", "lr_cool_down_steps",
                    "k_warmup_steps", "k_cold_booting_steps", "l1_coefficient_warmup_steps", "checkpoint_thresholds"):  # fmt: skip
            setattr(trainer, key, state[key])
        trainer._initialize_optimizer(sae)
        opt_path = ckpt_dir / "optimizer.pt"
        if opt_path.exists():
            sd = torch.load(opt_path, map_location="cpu", weights_only=False)
            if sd.get("format") == "by_name":
                trainer._load_optimizer_state(sae, sd)
            elif trainer.fused is not None:
                # a torch-format state_dict (the reference's layout): its entries are keyed by parameter position in the
                # param groups, which are in named_parameters order here
                names = [n for n, _ in sae.named_parameters()]
                order = [i for g in sd.get("param_groups", []) for i in g["params"]]
                by_name = {"format": "by_name", "state": {}}
                for pos, i in enumerate(order):
                    if i in sd["state"] and pos < len(names):
                        by_name["state"][names[pos]] = sd["state"][i]
                if by_name["state"]:
                    trainer._load_optimizer_state(sae, by_name)
                else:
                    logger.warning("optimizer.pt holds no per-parameter state that maps onto this model: the fused path starts from zero moments")
            elif trainer.optimizer is not None:
                trainer.optimizer.load_state_dict(sd)
        sched_path = ckpt_dir / "scheduler.pt"
        if sched_path.exists() and trainer.scheduler is not None:
            trainer.scheduler.load_state_dict(torch.load(sched_path, map_location="cpu", weights_only=False))
            # a freshly built scheduler has put its step-0 rate into the optimizer: restore the rate of the saved step
            if trainer.optimizer is not None:
                for group, lr in zip(trainer.optimizer.param_groups, trainer.scheduler.get_last_lr()):
                    group["lr"] = lr
        extra_path = ckpt_dir / "extra_state.pt"
        if extra_path.exists():
            extra = torch.load(extra_path, map_location="cpu", weights_only=False)
            trainer._restored_dead_counter = extra.get("tokens_since_last_activation")
        logger.info(f"Checkpoint loaded from {checkpoint_path} (step {trainer.cur_step})")
        return trainer

    # ---- initialisation ----------------------------------------------------------------------
    @timer.time("initialize_trainer")
    def _initialize_trainer(self, sae: SparseDictionary, first_batch: dict[str, Tensor], wandb_logger=None):
        bs = first_batch["tokens"].numel() * mesh_dim_size(sae.device_mesh, "data")
        self._first_batch_rows = first_batch["tokens"].numel()
        self.total_training_steps = self.cfg.total_training_tokens // bs

        def steps(v: float | int) -> int:
            if isinstance(v, float):
                assert 0 <= v <= 1.0
                return int(v * self.total_training_steps)
            return v

        self.lr_warm_up_steps = steps(self.cfg.lr_warm_up_steps)
        self.lr_cool_down_steps = steps(self.cfg.lr_cool_down_steps)
        self.k_warmup_steps = steps(self.cfg.k_warmup_steps)
        self.k_cold_booting_steps = steps(self.cfg.k_cold_booting_steps)
        self.l1_coefficient_warmup_steps = steps(self.cfg.l1_coefficient_warmup_steps)
        n = self.cfg.n_checkpoints
        if n > 0 and self.total_training_steps > 0:
            if self.cfg.check_point_save_mode == "linear":
                stride = max(self.total_training_steps // n, 1)
                self.checkpoint_thresholds = list(range(0, self.total_training_steps, stride))[1:]
            else:
                # log-spaced in steps (the thresholds are compared with the step counter)
                self.checkpoint_thresholds = sorted(
                    {math.ceil(2 ** (i / n * math.log2(self.total_training_steps))) for i in range(1, n)}
                )
        self.wandb_logger = wandb_logger

    @timer.time("initialize_optimizer")
    def _initialize_optimizer(self, sae: SparseDictionary):
        assert isinstance(self.cfg.lr, float)
        sched_kwargs = dict(
            warm_up_steps=self.lr_warm_up_steps, cool_down_steps=self.lr_cool_down_steps,
            training_steps=self.total_training_steps, lr_end_ratio=self.cfg.lr_end_ratio,
        )  # fmt: skip
        from .ops.fused_step import FusedTopKSAEStep
        from .optim import schedule_lambda

        ok, why = (False, "disabled") if not self.cfg.use_fused_kernels else FusedTopKSAEStep.supports(sae, self.cfg)
        if ok:
            comm = None
            rows = getattr(self, "_first_batch_rows", None)
            if self.cfg.use_peer_memory_collectives and mesh_dim_size(sae.device_mesh, "model") > 1 and rows:
                try:
                    from .parallel.symm import SymmComm

                    k_max = int(max(sae.cfg.top_k, self.cfg.initial_k or 0))
                    comm = SymmComm(mesh_group(sae.device_mesh, "model"), torch.device(sae.cfg.device), rows, k_max, sae.cfg.d_model)
                except Exception as e:  # noqa: BLE001
                    logger.warning(f"peer-memory collectives unavailable ({e}); using NCCL collectives")
            dp_comm = None
            dp = mesh_dim_size(sae.device_mesh, "data")
            F_l = sae.W_D.shape[0]
            if self.cfg.use_peer_memory_collectives and dp > 1 and rows and F_l % dp == 0:
                try:
                    from .parallel.symm import DataParallelComm

                    # every replica keeps the gathered rows of x, d x_hat and the three code tensors of a step; a
                    # batch-level top-k gives rows of varying width, bounded by the list capacity of its compaction
                    k_cap = -(-int(max(sae.cfg.top_k, self.cfg.initial_k or 0)) * (8 if sae.cfg.act_fn == "batchtopk" else 1) // 8) * 8
                    n_rows, d = rows * dp, sae.cfg.d_model
                    zones = {"x": n_rows * d * 2, "dxhat": n_rows * d * 2, "idx": n_rows * k_cap * 4,
                             "act": n_rows * k_cap * 4, "dact": n_rows * k_cap * 4}  # fmt: skip
                    dp_comm = DataParallelComm(mesh_group(sae.device_mesh, "data"), torch.device(sae.cfg.device), F_l, d, zones)
                except Exception as e:  # noqa: BLE001
                    logger.warning(f"peer-memory data parallelism unavailable ({e}); replicas repeat the full update")
            self.fused = FusedTopKSAEStep(sae, betas=self.cfg.betas, comm=comm, dp_comm=dp_comm)
            logger.info("Training on the fused sm_100a kernel path" + (" with peer-memory collectives" if comm or dp_comm else ""))
        else:
            from .ops.fused_crosscoder import FusedCrosscoderStep

            from .ops.fused_clt import FusedCLTStep
            from .ops.fused_lorsa import FusedLorsaStep

            ok_cc, why_cc = (False, "disabled") if not self.cfg.use_fused_kernels else FusedCrosscoderStep.supports(sae, self.cfg)
            ok_clt, why_clt = (False, "disabled") if not self.cfg.use_fused_kernels else FusedCLTStep.supports(sae, self.cfg)
            ok_lorsa, why_lorsa = (False, "disabled") if not self.cfg.use_fused_kernels else FusedLorsaStep.supports(sae, self.cfg)
            if ok_cc:
                self.fused = FusedCrosscoderStep(sae, betas=self.cfg.betas, jumprelu_lr_factor=self.cfg.jumprelu_lr_factor)
                logger.info(f"Training the JumpReLU {type(sae).__name__} on the fused sm_100a kernel path")
            elif ok_clt:
                self.fused = FusedCLTStep(sae, betas=self.cfg.betas)
                logger.info("Training the cross-layer transcoder on the fused sm_100a kernel path")
            elif ok_lorsa:
                self.fused = FusedLorsaStep(sae, betas=self.cfg.betas)
                logger.info("Training the low-rank sparse attention dictionary on the fused kernel path")
            else:
                reason = {"Crosscoder": why_cc, "CrossLayerTranscoder": why_clt, "LowRankSparseAttention": why_lorsa}.get(type(sae).__name__, why)
                if type(sae).__name__ == "SparseAutoEncoder" and sae.cfg.act_fn == "jumprelu":
                    reason = why_cc
                logger.info(f"Training on the generic autograd path ({reason})")
        groups = []
        for g in sae.get_parameters():
            if not g["params"]:
                continue
            groups.append({**g, "lr": self.cfg.jumprelu_lr_factor * self.cfg.lr} if g["name"] == "jumprelu" else g)
        if self.cfg.optimizer_class == "adam":
            kw: dict[str, Any] = {"foreach": self.cfg.optimizer_foreach}
            if all(p.is_cuda for g in groups for p in g["params"]):
                kw = {"fused": True}
            optimizer: Optimizer = Adam(groups, lr=self.cfg.lr, betas=self.cfg.betas, **kw)
        else:
            optimizer = SparseAdam(groups, lr=self.cfg.lr, betas=self.cfg.betas)
        self.optimizer = optimizer
        self.scheduler = get_scheduler(self.cfg.lr_scheduler_name, optimizer, **sched_kwargs)
        # the fused path never steps the torch scheduler: it evaluates the same schedule in closed form
        self._lr_lambda = schedule_lambda(self.cfg.lr_scheduler_name, base_lr=float(self.cfg.lr), **sched_kwargs)

    def _initialize_dead_statistics(self, sae: SparseDictionary) -> None:
        n_local = sae.local_shape("b_E", (sae.cfg.d_sae,))[0] if "b_E" in sae.dim_maps() else sae.cfg.d_sae
        dev = next(sae.parameters()).device
        self.tokens_since_last_activation = torch.zeros(n_local, device=dev, dtype=torch.long)
        restored = getattr(self, "_restored_dead_counter", None)
        if restored is not None and restored.numel() == n_local:
            self.tokens_since_last_activation.copy_(restored)
        self.is_dead = self.tokens_since_last_activation >= self.cfg.dead_threshold

    @torch.no_grad()
    def update_dead_statistics(self, feature_acts: Tensor, mask: Tensor | None, specs: tuple[str, ...]) -> Tensor:
        """Reset the counter of every feature that fired in this batch, advance the others by the number of
        valid tokens (summed over data-parallel ranks), and return ``counter >= dead_threshold``."""
        assert self.tokens_since_last_activation is not None and self.is_dead is not None
        valid = mask.sum() if mask is not None else torch.tensor(feature_acts[..., 0].numel(), device=feature_acts.device)
        fired, _ = apply_token_mask(feature_acts, specs, mask, "sum")
        fired = fired.gt(0)
        group = getattr(self, "_dp_group", None)
        if group is not None and dist.get_world_size(group) > 1:
            fired_i = fired.to(torch.int32)
            dist.all_reduce(fired_i, group=group)
            fired = fired_i > 0
            valid = valid.clone()
            dist.all_reduce(valid, group=group)
        self.tokens_since_last_activation = torch.where(
            fired, torch.zeros_like(self.tokens_since_last_activation), self.tokens_since_last_activation + valid
        )
        self.is_dead = self.tokens_since_last_activation >= self.cfg.dead_threshold
        return self.is_dead

    # ---- schedules ---------------------------------------------------------------------------
    def _current_k(self, sae: SparseDictionary) -> int | None:
        if "topk" not in sae.cfg.act_fn or self.k_warmup_steps <= 0 or self.cfg.initial_k is None:
            return None  # no k schedule (the reference insists on initial_k here; leaving it unset means "constant k")
        assert self.cfg.initial_k >= sae.cfg.top_k, "initial_k must be greater than or equal to top_k"
        if self.cur_step < self.k_cold_booting_steps:
            return int(self.cfg.initial_k)
        progress = min(1.0, (self.cur_step - self.k_cold_booting_steps) / self.k_warmup_steps)
        if self.cfg.k_schedule_type == "exponential":
            f = self.cfg.k_exponential_factor
            progress = (1.0 - math.exp(-f * progress)) / (1.0 - math.exp(-f))
        k = self.cfg.initial_k + (sae.cfg.top_k - self.cfg.initial_k) * progress
        return max(sae.cfg.top_k, math.ceil(k))

    def _l1_coefficient(self) -> float:
        if self.cfg.l1_coefficient is None:
            return 1.0
        if self.l1_coefficient_warmup_steps <= 0:
            return self.cfg.l1_coefficient
        return min(1.0, self.cur_step / self.l1_coefficient_warmup_steps) * self.cfg.l1_coefficient

    @timer.time("training_step")
    def _training_step(self, sae: SparseDictionary, batch: dict[str, Tensor]) -> dict[str, Any]:
        k = self._current_k(sae)
        if k is not None:
            sae.set_current_k(k)
        auxk = self.cfg.auxk_coefficient or 0.0
        return sae.compute_loss(
            batch,
            sparsity_loss_type=self.cfg.sparsity_loss_type,
            tanh_stretch_coefficient=self.cfg.tanh_stretch_coefficient,
            p=self.cfg.p,
            return_aux_data=True,
            l1_coefficient=self._l1_coefficient(),
            lp_coefficient=self.cfg.lp_coefficient or 0.0,
            auxk_coefficient=auxk,
            frequency_scale=self.cfg.frequency_scale,
            k_aux=self.cfg.k_aux,
            update_dead_statistics=self.update_dead_statistics if auxk > 0.0 else None,
        )

    # ---- logging -----------------------------------------------------------------------------
    def _emit(self, sae: SparseDictionary, metrics: dict[str, Any]) -> None:
        if is_primary_rank(sae.device_mesh):
            log_metrics(logger.logger, metrics, step=self.cur_step + 1, title="Training Metrics")
        if timer.enabled:
            logger.info(f"\nTimer Summary:\n{timer.summary()}\n")
        if self.wandb_logger is not None:
            self.wandb_logger.log(metrics, step=self.cur_step + 1)

    def _details(self, ctx: dict[str, Any], lr: float) -> dict[str, Any]:
        return {
            "details/current_learning_rate": lr,
            "details/n_training_tokens": self.cur_tokens,
            "details/l1_coefficient": ctx.get("l1_coefficient"),
            "details/lp_coefficient": ctx.get("lp_coefficient"),
            "details/auxk_coefficient": ctx.get("auxk_coefficient"),
        }

    @torch.no_grad()
    @timer.time("log")
    def _log(self, sae: SparseDictionary, ctx: dict[str, Any]):
        assert self.optimizer is not None, "Optimizer must be initialized"
        if not self.metrics:
            self.metrics = [
                FrequencyMetric(sae), LossMetric(sae), MeanFeatureActMetric(sae), ExplainedVarianceMetric(sae),
                L0Metric(sae), L2NormErrorMetric(sae), ModelSpecificMetric(sae), GradientNormMetric(sae),
            ]  # fmt: skip
        for metric in self.metrics:
            ctx = {**ctx, **metric.update(ctx)}
        if (self.cur_step + 1) % self.cfg.log_frequency == 0:
            out: dict[str, Any] = {}
            for metric in self.metrics:
                out.update(metric.compute())
            out.update(self._details(ctx, self.optimizer.param_groups[0]["lr"]))
            out.update(sae.log_statistics())
            self._emit(sae, out)

    @torch.no_grad()
    def _family_metrics(self, sae: SparseDictionary, batch: dict[str, Tensor]) -> dict[str, Any]:
        """The generic path's metric set (explained variance, l0, error norms, feature frequencies, the model's own
        figures) for ONE batch, from the model's own forward pass without a graph: what the fused steps of the crosscoder,
        cross-layer transcoder and Lorsa families log on a logging step (their kernels keep no dense reconstruction to
        measure). The batch is the logging step's, seen after that step's update. Collective under a mesh: every rank
        reaches it on the same steps."""
        nb = sae.normalize_activations(batch)
        dev_type = torch.device(sae.cfg.device).type
        amp = self.cfg.amp_dtype is not None and (dev_type == "cuda" or self.cfg.amp_dtype == torch.bfloat16)
        with torch.autocast(device_type=dev_type, dtype=self.cfg.amp_dtype, enabled=amp):
            ctx = self._training_step(sae, nb)
            metrics = [FrequencyMetric(sae), LossMetric(sae), MeanFeatureActMetric(sae), ExplainedVarianceMetric(sae),
                       L0Metric(sae), L2NormErrorMetric(sae), ModelSpecificMetric(sae)]  # fmt: skip
            for metric in metrics:
                ctx = {**ctx, **metric.update(ctx)}
            out: dict[str, Any] = {}
            for metric in metrics:
                out.update(metric.compute())
        return out

    @torch.no_grad()
    def _log_fused(self, sae: SparseDictionary, x: Tensor, label: Tensor, mask: Tensor | None, loss: Tensor, lr: float):
        """Metrics of the fused path. Per step only three small device accumulations happen (loss, per-feature
        fire counts from the step's counting sort, token count); the dense quantities (explained variance,
        error norms) are evaluated on the logging step's batch."""
        f = self.fused
        acc = self._interval
        if not acc:
            acc["loss"] = torch.zeros((), device=x.device)
            acc["fire"] = torch.zeros(f.F, device=x.device, dtype=torch.float32)
            acc["tokens"] = 0
            acc["steps"] = 0
        acc["loss"] += loss
        if f.last_grad_norm is not None and self.cfg.clip_grad_norm > 0:  # interval maximum, as GradientNormMetric keeps it
            acc["grad_norm"] = torch.maximum(acc.get("grad_norm", f.last_grad_norm), f.last_grad_norm)
        n_rows = f.groups.entries.numel() and (x.shape[0] * f.dp)
        acc["fire"] += (f.main_counts if f.main_counts is not None else f.groups.counts[: f.F]).float()
        acc["tokens"] += n_rows
        acc["steps"] += 1
        if (self.cur_step + 1) % self.cfg.log_frequency != 0:
            return
        idx, act, xhat = f.forward_dense(x, sae.current_k)
        lab = label.float()
        err = (xhat - lab).pow(2).sum(-1)
        var = (lab - lab.mean(0)).pow(2).sum(-1)
        stats = torch.stack([
            err.mean(), var.mean(), (1 - err / var).mean(), err.sqrt().mean(), lab.norm(dim=-1).mean(),
        ])  # fmt: skip
        sparse = torch.stack([act.sum(), (idx >= 0).sum().float()])
        if f.tp > 1:
            dist.all_reduce(sparse, group=f.tp_group)
        freq = acc["fire"] / max(acc["tokens"], 1)
        counts = torch.stack([(freq > 1e-1).sum(), (freq > 1e-2).sum(), (freq < 1e-5).sum(), (freq < 1e-6).sum(),
                              (freq < 1e-7).sum(), freq.sum()]).float()  # fmt: skip
        if f.tp > 1:
            dist.all_reduce(counts, group=f.tp_group)
        mean_loss = acc["loss"] / acc["steps"]
        if f.dp > 1:
            pack = torch.cat([stats, mean_loss.reshape(1)])
            dist.all_reduce(pack, group=f.dp_group)
            pack /= f.dp
            stats, mean_loss = pack[:5], pack[5]
        s, c, sp = stats.tolist(), counts.tolist(), sparse.tolist()
        out = {
            "losses/overall_loss": float(mean_loss), "losses/mse_loss": float(mean_loss),
            "metrics/explained_variance": 1 - s[0] / s[1], "metrics/explained_variance_legacy": s[2],
            "metrics/l0": c[5], "metrics/l2_norm_error": s[3], "metrics/l2_norm_error_ratio": s[3] / s[4],
            "metrics/mean_feature_act": sp[0] / max(sp[1], 1.0),
            "sparsity/above_1e-1": c[0], "sparsity/above_1e-2": c[1], "sparsity/below_1e-5": c[2],
            "sparsity/below_1e-6": c[3], "sparsity/below_1e-7": c[4],
        }  # fmt: skip
        if "grad_norm" in acc:
            before = float(acc["grad_norm"])
            out["metrics/gradient_norm_before_clipping"] = before
            out["metrics/gradient_norm_per_param"] = min(before, self.cfg.clip_grad_norm)
        if f.batch_level:  # tokens whose batch-level codes exceeded the fixed list width since the last report
            out["details/batchtopk_list_overflow_tokens"] = int(f.list_overflow)
            f.list_overflow.zero_()
        if self._fused_aux is not None:
            out["details/auxk_dead_capacity"] = self._fused_aux.capacity
            out["details/auxk_truncated_steps"] = int(self._fused_aux.truncated_steps)
        out.update(self._details({}, lr))
        f.sync_params()  # (no-op unless the optimizer state is sharded over replicas)
        out.update(sae.log_statistics())
        self._interval = {}
        self._emit(sae, out)

    @timer.time("save_checkpoint")
    def _maybe_save_sae_checkpoint(self, sae: SparseDictionary):
        if self.checkpoint_thresholds and self.cur_step >= self.checkpoint_thresholds[0]:
            self._before_parameters_leave(sae)
            sae.save_checkpoint(os.path.join(self.cfg.exp_result_path, "checkpoints", f"{self.cur_step}.safetensors"))
            self.checkpoint_thresholds.pop(0)

    # ---- main loop ---------------------------------------------------------------------------
    def fit(
        self,
        sae: SparseDictionary,
        activation_stream: Iterable[dict[str, Tensor]],
        eval_fn: Callable[[SparseDictionary], None] | None = None,
        wandb_logger=None,
    ) -> bool | None:
        """Train until ``total_training_tokens`` are consumed. Returns True when the stream ended first."""
        from tqdm import tqdm

        timer.reset()
        stream = iter(activation_stream)
        dev = torch.device(sae.cfg.device)
        if dev.type == "cuda" and self.cfg.prefetch_to_device:
            # feature-parallel ranks of a replica read identical batches: each copies a slice, NVLink does the rest
            shared = mesh_group(sae.device_mesh, "model") if self.cfg.shard_host_copies else None
            stream = _DevicePrefetcher(stream, next(sae.parameters()).device, replica_group=shared)
        try:
            batch = next(stream)
        except StopIteration:
            logger.info("the activation stream is empty")
            return True
        if self.cfg.from_pretrained_path is None:
            self._initialize_trainer(sae, batch, wandb_logger)
            self._initialize_optimizer(sae)
        else:
            self.wandb_logger = wandb_logger
        self._dp_group = mesh_group(sae.device_mesh, "data")
        if self.cfg.auxk_coefficient is not None and self.cfg.auxk_coefficient > 0.0:
            self._initialize_dead_statistics(sae)
        assert self.optimizer is not None and self.scheduler is not None
        bar = tqdm(total=self.total_training_steps, smoothing=0.001, disable=not is_primary_rank(sae.device_mesh))
        bar.update(self.cur_step)
        dp = mesh_dim_size(sae.device_mesh, "data")
        accum = max(1, self.cfg.gradient_accumulation_steps)
        loss_reader = _LossReader()
        heartbeat = self._make_heartbeat()
        finished = False
        try:
            while True:
                with timer.time("training_iteration"):
                    if heartbeat is not None:
                        heartbeat.beat(self.cur_step)
                        heartbeat.check()  # before this step's collectives: a lost peer ends the run here, not in a hang
                    bar.update(1)
                    sae.train()
                    batch = self._to_model_device(sae, batch)
                    if self.fused is not None:
                        loss = self._fused_iteration(sae, batch)
                    else:
                        loss = self._generic_iteration(sae, batch, accum)
                    if (self.cur_step + 1) % self.cfg.log_frequency == 0:
                        shown = loss_reader.push(loss, self._kernel_status(sae))
                        if shown is not None:
                            bar.set_description(f"loss: {shown:.2f}")
                    if eval_fn is not None and (self.cur_step + 1) % self.cfg.eval_frequency == 0:
                        with timer.time("evaluation"):
                            self._before_parameters_leave(sae)
                            eval_fn(sae)
                    self.cur_step += 1
                    self.cur_tokens += self._count_tokens(batch) * dp
                    self._maybe_save_sae_checkpoint(sae)
                    if self.cur_step >= self.total_training_steps:
                        finished = True
                        break
                    with timer.time("refresh_batch"):
                        del batch
                        batch = next(stream)
        except StopIteration:
            finished = True
            logger.info("the current stream has ended")
            if heartbeat is not None:
                heartbeat.leave("end of the activation stream")
            return True
        except Exception as e:
            logger.error(f"Training failed: {e}")
            if heartbeat is not None and not isinstance(e, PeerLost):
                heartbeat.leave(f"{type(e).__name__}: {e}")
            if self.cfg.checkpoint_on_failure:
                self._save_failure_checkpoint(sae)
            raise
        finally:
            last = loss_reader.flush()
            if last is not None:
                self.last_loss = last
            bar.close()
            if self.fused is not None:
                self.fused.join()  # the last update may still be running on its own stream
                if finished:  # collective: only when every rank left the loop in step
                    self.fused.sync_params()
        return None

    def _before_parameters_leave(self, sae: SparseDictionary) -> None:
        """Before parameters are written out or handed to other code on the fused path: fold the update stream back,
        raise if a kernel recorded an error (a timed-out collective leaves the step's data unusable; the update kernels
        skip themselves after one, so the parameters are those of the last good step, but nothing more must be saved as
        if training had gone on), and gather the master rows that other replicas own."""
        if self.fused is None:
            return
        self.fused.join()
        dev = next(sae.parameters()).device
        if dev.type == "cuda":
            from .ops import sae_kernels as K

            K.check_status(dev)
        self.fused.sync_params()

    @staticmethod
    def _mask_summary(batch: dict[str, Any]) -> dict[str, Any]:
        """For a batch whose token mask is still in host memory: note the number of valid tokens and whether all are valid
        under private keys, so that no later step needs to ask the device."""
        mask = batch.get("mask")
        if isinstance(mask, Tensor) and mask.device.type == "cpu" and "_n_valid" not in batch:
            n = int(mask.sum())
            batch = {**batch, "_n_valid": n, "_mask_all": n == mask.numel()}
        return batch

    def _all_tokens_valid(self, batch: dict[str, Any]) -> bool:
        """Whether the batch's mask (if any) is all true. A mask in host memory was summarised when the batch came in; a
        mask on the device costs one read, which is remembered for as long as the very same tensor object comes back
        unmodified (a stream that reuses one device mask for every batch is asked once, not once per step). The tensor is
        kept referenced meanwhile, so that its memory cannot be handed to another mask that would look the same."""
        mask = batch.get("mask")
        if mask is None:
            return True
        if "_mask_all" in batch:
            return bool(batch["_mask_all"])
        if mask.device.type == "cpu":
            return bool(mask.all())
        seen = getattr(self, "_device_mask_seen", None)
        if seen is not None and seen[0] is mask and seen[1] == mask._version and seen[2] is not None:
            return seen[2]
        ok = bool(mask.all())
        self._device_mask_seen = (mask, mask._version, ok)
        return ok

    def _count_tokens(self, batch: dict[str, Any]) -> int:
        """Valid tokens of a batch for the progress counters. A mask that lives on the device is counted there and folded
        in at the next logging step (one read per logging interval instead of one per step)."""
        if "_n_valid" in batch:
            return int(batch["_n_valid"])
        mask = batch.get("mask")
        if mask is None:
            return batch["tokens"].numel()
        if not mask.is_cuda:
            return int(mask.sum())
        total = mask.sum()
        self._tokens_on_device = total if self._tokens_on_device is None else self._tokens_on_device + total
        if (self.cur_step % max(1, self.cfg.log_frequency)) == 0:
            n, self._tokens_on_device = int(self._tokens_on_device), None
            return n
        return 0

    def _kernel_status(self, sae: SparseDictionary) -> Tensor | None:
        """The status word of this model's device when hand-written kernels are in play (read back with the loss)."""
        dev = next(sae.parameters()).device
        if self.fused is None or dev.type != "cuda":
            return None
        from .ops import sae_kernels as K

        return K.status_buffer(dev)

    def _make_heartbeat(self):
        if self.cfg.heartbeat_timeout_s is None or not dist.is_initialized() or dist.get_world_size() == 1:
            return None
        from .parallel.health import Heartbeat, default_store

        return Heartbeat(default_store(), dist.get_rank(), dist.get_world_size(), timeout_s=self.cfg.heartbeat_timeout_s)

    def restore_failure_checkpoint(self, sae: SparseDictionary, path: str | Path) -> None:
        """Load what ``_save_failure_checkpoint`` wrote for this rank (``<path>/rank_<r>/``): local parameter tensors, the
        step / token counters and, on the fused path, this rank's Adam moments. Call after ``fit`` has built the
        optimizer for the same mesh, or on a trainer whose optimizer is initialised."""
        rank = dist.get_rank() if dist.is_initialized() else 0
        src = Path(path) / f"rank_{rank}"
        local = torch.load(src / "local_state.pt", map_location="cpu", weights_only=False)
        with torch.no_grad():
            for k, v in sae.state_dict().items():
                if k in local:
                    v.copy_(local[k].to(v.device))
        state = torch.load(src / "trainer.pt", map_location="cpu", weights_only=False)
        self.cur_step, self.cur_tokens = state["cur_step"], state["cur_tokens"]
        fo = state.get("fused_optimizer")
        if self.fused is not None and fo is not None:
            assert tuple(fo["own_rows"]) == tuple(self.fused.own_rows), "the failure checkpoint was written for another layout"
            self.fused.t = int(fo["step"])
            for n, pair in fo["state"].items():
                for dst, srct in zip(self.fused.state[n], pair):
                    dst.copy_(srct.to(dst.device))
            self.fused.refresh()
        elif self.optimizer is not None and "optimizer" in state:
            self.optimizer.load_state_dict(state["optimizer"])

    def _save_failure_checkpoint(self, sae: SparseDictionary) -> None:
        """Best effort, this rank only and without collectives (the other ranks may be gone): the model's local tensors,
        the optimizer and the trainer state under ``<exp_result_path>/failure/rank_<r>/``."""
        try:
            if self.fused is not None:
                self.fused.join()
            rank = dist.get_rank() if dist.is_initialized() else 0
            out = Path(self.cfg.exp_result_path) / "failure" / f"rank_{rank}"
            os.makedirs(out, exist_ok=True)
            torch.save({k: v.detach().cpu() for k, v in sae.state_dict().items()}, out / "local_state.pt")
            sae.cfg.save_hyperparameters(out)
            state = {"cur_step": self.cur_step, "cur_tokens": self.cur_tokens, "total_training_steps": self.total_training_steps,
                     "cfg": self.cfg}  # fmt: skip
            if self.fused is not None:
                # this rank's moments as they are (its shard, and under a sharded optimizer state its feature rows only)
                state["fused_optimizer"] = {
                    "step": self.fused.t, "own_rows": tuple(self.fused.own_rows),
                    "state": {n: tuple(t.detach().cpu() for t in st) for n, st in self.fused.state.items() if st is not None},
                }
            elif self.optimizer is not None:
                state["optimizer"] = self.optimizer.state_dict()
            if self.scheduler is not None:
                state["scheduler"] = self.scheduler.state_dict()
            torch.save(state, out / "trainer.pt")
            logger.info(f"failure checkpoint saved to {out} (step {self.cur_step})")
        except Exception as e:  # noqa: BLE001  (the original exception matters more)
            logger.error(f"could not save a failure checkpoint: {e}")

    @staticmethod
    def _to_model_device(sae: SparseDictionary, batch: dict[str, Any]) -> dict[str, Any]:
        """Host batches (ideally pinned) are copied to the model's device asynchronously on the current stream."""
        dev = torch.device(sae.cfg.device)
        if dev.type != "cuda":
            return batch
        batch = Trainer._mask_summary(batch)
        return {
            k: (v.to(dev, non_blocking=True) if isinstance(v, Tensor) and v.device.type == "cpu" else v)
            for k, v in batch.items()
        }

    def _generic_iteration(self, sae: SparseDictionary, batch: dict[str, Tensor], accum: int) -> Tensor:
        assert self.optimizer is not None and self.scheduler is not None
        batch = sae.normalize_activations(batch)
        dev_type = torch.device(sae.cfg.device).type
        amp = self.cfg.amp_dtype is not None and (dev_type == "cuda" or self.cfg.amp_dtype == torch.bfloat16)
        with torch.autocast(device_type=dev_type, dtype=self.cfg.amp_dtype, enabled=amp):
            ctx = self._training_step(sae, batch)
        with timer.time("backward"):
            (ctx["loss"] / accum).backward()
        if (self.cur_step + 1) % accum != 0:
            return ctx["loss"].detach()
        with timer.time("reduce_gradients"):
            reduce_gradients(sae.parameters(), mesh_group(sae.device_mesh, "data"))
            if mesh_dim_size(sae.device_mesh, "head") > 1:
                # Parameters that are not split over the head dimension (a crosscoder's shared JumpReLU thresholds) are
                # replicated on the head ranks, each of which holds the gradient of its own heads only: sum them, or the
                # replicas drift apart (the model scales its loss by 1 / head ranks, so the sum is the gradient of the
                # mean over all heads).
                maps = sae.dim_maps()
                shared = [p for n, p in sae.named_parameters() if p.grad is not None and "head" not in maps.get(n, {})]
                if shared:
                    flat = torch.cat([p.grad.reshape(-1).float() for p in shared])
                    dist.all_reduce(flat, group=mesh_group(sae.device_mesh, "head"))
                    off = 0
                    for p in shared:
                        p.grad.copy_(flat[off : off + p.numel()].view_as(p.grad))
                        off += p.numel()
        with timer.time("clip_grad_norm"):
            ctx["grad_norm_before_clipping"] = clip_grad_norm(
                [p for n, p in sae.named_parameters() if p.grad is not None and "log_jumprelu_threshold" not in n],
                max_norm=self.cfg.clip_grad_norm if self.cfg.clip_grad_norm > 0 else math.inf,
                device_mesh=sae.device_mesh,
            )
        if not self.cfg.skip_metrics_calculation:
            with torch.autocast(device_type=dev_type, dtype=self.cfg.amp_dtype, enabled=amp):
                self._log(sae, ctx)
        with timer.time("optimizer_step"):
            self.optimizer.step()
            self.optimizer.zero_grad(set_to_none=True)
        with timer.time("scheduler_step"):
            self.scheduler.step()
        return ctx["loss"].detach()

    def _fused_crosscoder_iteration(self, sae: SparseDictionary, batch: dict[str, Tensor]) -> Tensor:
        """One step of ``ops.fused_crosscoder.FusedCrosscoderStep``: this rank's hook points, normalised, stacked to
        ``[tokens, local heads, d_model]`` in bf16."""
        f = self.fused
        if not self._all_tokens_valid(batch):
            raise NotImplementedError("the fused crosscoder path trains on unmasked tokens; set use_fused_kernels=False for masked batches")
        cols = []
        for hp in sae.local_hook_points() if hasattr(sae, "local_hook_points") else [sae.cfg.hook_point_in]:
            raw = batch[hp]
            assert raw.ndim == 2, "the fused path trains on [tokens, d_model] activations"
            if sae.cfg.norm_activation == "dataset-wise":
                factor = math.sqrt(sae.cfg.d_model) / float(sae.dataset_average_activation_norm[hp])
                raw = raw if factor == 1.0 else raw * factor
            elif sae.cfg.norm_activation != "inference":
                raw = raw * sae.compute_norm_factor(raw, hp)
            if raw.shape[-1] < sae.cfg.d_model:
                raw = torch.nn.functional.pad(raw, (0, sae.cfg.d_model - raw.shape[-1]))
            cols.append(raw.to(torch.bfloat16))
        x = torch.stack(cols, dim=1)
        label = None
        if f.single and sae.cfg.hook_point_out != sae.cfg.hook_point_in:  # a transcoder: the target is another hook point
            label = self._normalised_bf16(sae, batch[sae.cfg.hook_point_out], sae.cfg.hook_point_out).unsqueeze(1)
        lr = float(self.cfg.lr) * (self._lr_lambda(self.cur_step) if self._lr_lambda is not None else 1.0)
        l1 = self._l1_coefficient() if self.cfg.sparsity_loss_type in ("tanh", "tanh-quad") else 0.0
        loss = f.step(x, lr, l1_coefficient=l1, tanh_stretch=self.cfg.tanh_stretch_coefficient,
                      lp_coefficient=float(self.cfg.lp_coefficient or 0.0), sparsity_loss_type=self.cfg.sparsity_loss_type or "tanh",
                      frequency_scale=self.cfg.frequency_scale, label=label)
        if not self.cfg.skip_metrics_calculation and (self.cur_step + 1) % self.cfg.log_frequency == 0:
            last = {k: float(v) for k, v in f.last.items()}
            out = self._family_metrics(sae, batch)
            out.update({"losses/overall_loss": float(loss), "losses/mse_loss": last["l_rec"], "losses/sparsity_loss": last["l_s"],
                        "losses/lp_loss": last["l_p"], "metrics/l0_candidates": last["l0"],
                        "details/list_overflow_tokens": int(f.list_overflow)})  # fmt: skip
            out.update(self._details({"l1_coefficient": l1}, lr))
            out.update(sae.log_statistics())
            self._emit(sae, out)
        return loss

    def _normalised_bf16(self, sae: SparseDictionary, raw: Tensor, hook_point: str) -> Tensor:
        """One hook point's activations scaled to the model's norm convention, in bf16, without a device scalar."""
        if sae.cfg.norm_activation == "dataset-wise":
            factor = math.sqrt(sae.cfg.d_model) / float(sae.dataset_average_activation_norm[hook_point])
            raw = raw if factor == 1.0 else raw * factor
        elif sae.cfg.norm_activation != "inference":
            raw = raw * sae.compute_norm_factor(raw, hook_point)
        return raw.to(torch.bfloat16)

    def _fused_clt_iteration(self, sae: SparseDictionary, batch: dict[str, Tensor]) -> Tensor:
        """One step of ``ops.fused_clt.FusedCLTStep``: inputs ``[tokens, layers, d]``, targets ``[layers, tokens, d]``."""
        f = self.fused
        # a token mask in the batch plays no part: this model's loss is the mean over all tokens and layers on the generic
        # path too (models/clt.py compute_loss; clt.py:1059-1067 of the reference project)
        d = sae.cfg.d_model
        # layer-major [layers, tokens, d]: what the per-layer GEMMs and the update kernels read
        xt = torch.stack([self._normalised_bf16(sae, batch[hp], hp).reshape(-1, d) for hp in sae.cfg.hook_points_in], dim=0)
        x = xt.transpose(0, 1)
        y = torch.stack([self._normalised_bf16(sae, batch[hp], hp).reshape(-1, d) for hp in sae.cfg.hook_points_out], dim=0)
        k = self._current_k(sae)
        if k is not None:
            sae.set_current_k(k)
        lr = float(self.cfg.lr) * (self._lr_lambda(self.cur_step) if self._lr_lambda is not None else 1.0)
        loss = f.step(x, y, sae.current_k, lr, xt=xt)
        if not self.cfg.skip_metrics_calculation and (self.cur_step + 1) % self.cfg.log_frequency == 0:
            out = self._family_metrics(sae, batch)
            out.update({"losses/overall_loss": float(loss), "losses/mse_loss": float(loss)})
            out.update(self._details({}, lr))
            out.update(sae.log_statistics())
            self._emit(sae, out)
        return loss

    def _fused_lorsa_iteration(self, sae: SparseDictionary, batch: dict[str, Tensor]) -> Tensor:
        """One step of ``ops.fused_lorsa.FusedLorsaStep``: inputs and targets ``[batch, seq, d_model]``."""
        f = self.fused
        mask = batch.get("mask")
        row_weight = None
        if mask is not None:
            all_valid = batch.get("_mask_all")
            if all_valid is None and mask.device.type != "cpu":
                # A mask on the device is not read back for its own sake: weights cost a few small kernels, a read stalls the
                # host. Only when the very same tensor comes back (a stream that reuses one mask) is it worth asking once.
                seen = getattr(self, "_device_mask_seen", None)
                if seen is not None and seen[0] is mask and seen[1] == mask._version:
                    all_valid = self._all_tokens_valid(batch)
                else:
                    self._device_mask_seen = (mask, mask._version, None)
            if not all_valid:
                # masked tokens weigh 0, the others tokens / valid tokens, computed on the device (no wait for the count)
                w = mask.reshape(-1).float()
                n = w.sum()
                if f.dp > 1:  # the mean is over the valid tokens of all replicas
                    dist.all_reduce(n, group=f.dp_group)
                row_weight = w * (w.numel() * f.dp / n.clamp_min(1.0))
        hin, hout = sae.cfg.hook_point_in, sae.cfg.hook_point_out
        x = self._normalised_bf16(sae, batch[hin], hin)
        y = self._normalised_bf16(sae, batch[hout], hout)
        assert x.ndim == 3, "low-rank sparse attention trains on [batch, seq, d_model] activations"
        k = self._current_k(sae)
        if k is not None:
            sae.set_current_k(k)
        lr = float(self.cfg.lr) * (self._lr_lambda(self.cur_step) if self._lr_lambda is not None else 1.0)
        loss = f.step(x, y, sae.current_k, lr, row_weight=row_weight)
        if not self.cfg.skip_metrics_calculation and (self.cur_step + 1) % self.cfg.log_frequency == 0:
            out = self._family_metrics(sae, batch)
            out.update({"losses/overall_loss": float(loss), "losses/mse_loss": float(loss)})
            out.update(self._details({}, lr))
            out.update(sae.log_statistics())
            self._emit(sae, out)
        return loss

    def _fused_iteration(self, sae: SparseDictionary, batch: dict[str, Tensor]) -> Tensor:
        f = self.fused
        if type(f).__name__ == "FusedCrosscoderStep":
            return self._fused_crosscoder_iteration(sae, batch)
        if type(f).__name__ == "FusedLorsaStep":
            return self._fused_lorsa_iteration(sae, batch)
        if type(f).__name__ == "FusedCLTStep":
            return self._fused_clt_iteration(sae, batch)
        hin, hout = sae.cfg.hook_point_in, sae.cfg.hook_point_out
        x_raw = batch[hin]
        assert x_raw.ndim == 2, "the fused path trains on [tokens, d_model] activations"

        def normalised(raw: Tensor, hook_point: str) -> Tensor:
            # A constant factor stays a Python number: building a device scalar from it every step (what
            # compute_norm_factor returns) is a synchronous copy, after which the host can no longer run ahead of the
            # device; a factor of exactly 1 costs no kernel at all.
            mode = sae.cfg.norm_activation
            if mode == "inference":
                scaled = raw
            elif mode == "dataset-wise":
                assert sae.dataset_average_activation_norm is not None, "dataset_average_activation_norm must be provided from Initializer"
                factor = math.sqrt(sae.cfg.d_model) / float(sae.dataset_average_activation_norm[hook_point])
                scaled = raw if factor == 1.0 else raw * factor
            else:
                scaled = raw * sae.compute_norm_factor(raw, hook_point)
            return scaled.to(torch.bfloat16).contiguous()

        x = normalised(x_raw, hin)
        label = x if hout == hin else normalised(batch[hout], hout)
        mask = batch.get("mask")
        row_weight, n_global = None, None
        if mask is not None and not batch.get("_mask_all", False):
            # Masked rows get weight 0, valid rows B_global / n_valid, computed on the device: the kernels keep their host
            # constant 2 / B_global as the gradient scale and no step waits for the device to count its valid tokens.
            w = mask.reshape(-1).float()
            n = w.sum()
            if f.dp > 1:
                n = n.clone()
                dist.all_reduce(n, group=f.dp_group)
            n_global = w.numel() * f.dp
            row_weight = w * (n_global / n.clamp_min(1.0))
        k = self._current_k(sae)
        if k is not None:
            sae.set_current_k(k)
        lr_factor = self._lr_lambda(self.cur_step) if self._lr_lambda is not None else 1.0
        lr = float(self.cfg.lr) * lr_factor
        aux = None
        if self.cfg.auxk_coefficient:
            if self._fused_aux is None:
                from .ops.fused_step import AuxK

                assert self.tokens_since_last_activation is not None, "dead statistics are initialised in fit()"
                self._fused_aux = AuxK(f.F, self.cfg.k_aux, self.cfg.auxk_coefficient, self.cfg.dead_threshold, x.device,
                                       counter=self.tokens_since_last_activation)  # fmt: skip
            aux = self._fused_aux
        loss = f.step(x, label, sae.current_k, lr, row_weight=row_weight, n_tokens_global=n_global, aux=aux,
                      clip_grad_norm=max(0.0, self.cfg.clip_grad_norm))
        if aux is not None:  # keep the trainer's view (checkpoints, logging) in step with the engine's counters
            self.tokens_since_last_activation, self.is_dead = aux.tokens_since_last_activation, aux.is_dead
        if not self.cfg.skip_metrics_calculation:
            self._log_fused(sae, x, label, mask, loss, lr)
        return loss

