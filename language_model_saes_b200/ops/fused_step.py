"""One training step of a TopK (or BatchTopK) sparse autoencoder as a fixed sequence of sm_100a kernels, without autograd.

What it computes is the reference's step for a TopK ``SparseAutoEncoder`` trained with the MSE loss and Adam
(trainer.py:576-671, models/sae.py:288-377, models/sparse_dictionary.py:841-886 of the reference project):
encode, per-token top-k of the decoder-norm-gated pre-activations, decode, mean-over-tokens of the summed
squared error, backward, Adam. How it computes it:

1. encoder GEMM (tcgen05) with the top-k epilogue        -> candidates per row and column range
2. candidate merge (+ one exchange between feature shards) -> sparse codes (idx, act) [B, k]
3. sparse decode fused with loss, d x_hat and d act        -> no dense [B, F] tensor exists at any point
4. counting sort of the codes by feature
5. per feature row: rebuild the sparse gradient rows of W_D and W_E^T in registers and apply Adam, refresh
   the bf16 shadows and the decoder row norms                -> no dense gradient tensor exists either

Optionally steps 5 (bound by HBM bandwidth: it streams every parameter and both Adam moments) and 1 of the NEXT step
(bound by the tensor cores) overlap: the dictionary is cut into a few feature chunks, the update runs chunk by chunk on its own
stream and the next step's encoder GEMM sweeps chunk ``c`` on a high-priority stream as soon as chunk ``c`` is updated
(the running top-k is carried from one chunk's launch to the next). Ordering is by stream events only; arithmetic
and results are those of the unchunked sequence.

Parallel layouts: ``model`` (features sharded; candidates are exchanged and the partial reconstructions
summed) and ``data`` (batch sharded; instead of all-reducing dense gradients of size 2*d*F, ranks exchange
their rows of x, d x_hat and the sparse codes, which is all the gradient depends on, and every replica
rebuilds the identical full-batch gradient).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..parallel.mesh import mesh_dim_size, mesh_group, mesh_local_rank
from . import sae_kernels as K


def _mm_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b`` for bf16 matrices with an fp32 result (a plain library GEMM: fp32 accumulation, no bf16 rounding of the
    output, so that sums over feature shards or replicas do not depend on how the work was split)."""
    if a.is_cuda:
        try:
            return torch.mm(a, b, out_dtype=torch.float32)
        except (TypeError, RuntimeError):  # a build without the out_dtype overload: bf16 output, widened afterwards
            return (a @ b).float()
    return a.float() @ b.float()


def merge_codes_over_shards(idx_l: torch.Tensor, act_l: torch.Tensor, gate_l: torch.Tensor | None, k: int, tp: int, tp_rank: int,
                            group) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
    """Every shard holds its own top-``k`` codes ``(idx_l, act_l)`` of each row; keep those that are among the ``k``
    largest gated values of the row over all shards (all-gather of the lists, merge, own slots only, packed from slot 0)."""
    B = idx_l.shape[0]
    g_l = act_l * gate_l[idx_l.clamp_min(0).long()] if gate_l is not None else act_l
    all_g = torch.empty(tp * B, k, dtype=torch.float32, device=idx_l.device)
    all_i = torch.empty(tp * B, k, dtype=torch.int32, device=idx_l.device)
    dist.all_gather_into_tensor(all_g, g_l.float().contiguous(), group=group)
    dist.all_gather_into_tensor(all_i, idx_l.contiguous(), group=group)
    all_g = all_g.view(tp, B, k).permute(1, 0, 2).reshape(B, tp * k).contiguous()
    all_i = all_i.view(tp, B, k).permute(1, 0, 2).reshape(B, tp * k).contiguous()
    merge = K.topk_merge if k <= 64 else K.ref_topk_merge  # the merge kernel's lists hold at most 64 codes per row
    return merge(all_g, all_i, k, gate_l, own=(tp_rank * k, (tp_rank + 1) * k))


class AuxK:
    """State and settings of the Aux-K loss on the fused path: per-feature count of valid tokens since the feature
    last fired; a feature is dead once the count reaches ``dead_threshold`` (trainer.py:403-454 of the reference).

    Nothing here makes the host wait for the step it is issuing. The dead features of a step are gathered into a compact dictionary
    of ``capacity`` rows for the auxiliary encoder pass; the capacity follows the number of dead features with a lag: the
    count of every step is copied to pinned memory and read two steps later, and the
    capacity is then set to that count plus a quarter plus 1024 rows (at least ``k_aux``, in steps of 256 rows): every
    product of the auxiliary pass costs in proportion to the capacity, so the headroom is kept small. Should the dead
    features of a step outnumber the capacity (they grew by more than that within the lag), that step's auxiliary
    top-k sees the first ``capacity`` of them by index; ``truncated_steps`` counts such steps."""

    def __init__(self, n_features: int, k_aux: int, coefficient: float, dead_threshold: float, device, counter: torch.Tensor | None = None):
        self.k_aux, self.coefficient, self.dead_threshold = int(k_aux), float(coefficient), dead_threshold
        self.n_features = n_features
        self.tokens_since_last_activation = counter if counter is not None else torch.zeros(n_features, dtype=torch.long, device=device)
        self.is_dead = self.tokens_since_last_activation >= dead_threshold
        self.capacity = self._bucket(int(self.is_dead.sum()))
        self.truncated_steps = torch.zeros((), dtype=torch.long, device=device)
        self._pending: list[tuple[torch.Tensor, object]] = []

    def _bucket(self, n_dead: int) -> int:
        rows = max(self.k_aux, n_dead + n_dead // 4 + 1024)
        return min(-(-self.n_features // 8) * 8, -(-rows // 256) * 256)

    def update(self, fired: torch.Tensor, n_valid_tokens) -> torch.Tensor:
        """``fired``: per feature, non-zero where it fired in this step (over every replica); ``n_valid_tokens``: number or
        0-d tensor of valid tokens of the (global) step."""
        c = self.tokens_since_last_activation
        self.tokens_since_last_activation = torch.where(fired > 0, torch.zeros_like(c), c + n_valid_tokens)
        self.is_dead = self.tokens_since_last_activation >= self.dead_threshold
        return self.is_dead

    LAG = 2  # steps between a count leaving the device and its use: the same on every rank, so capacities agree

    def observe(self, n_dead: torch.Tensor) -> None:
        """Feed the lagged capacity estimate with this step's number of dead features (0-d device tensor). The count is
        copied to pinned memory now and read ``LAG`` steps later (its copy has long completed by then, the wait on its
        event returns at once). The lag is a fixed number of steps rather than "whenever the copy is seen to be done",
        because replicas and shards that exchange buffers sized by the capacity must all switch in the same step."""
        self.truncated_steps += n_dead > self.capacity
        if not n_dead.is_cuda:
            self.capacity = self._bucket(int(n_dead))
            return
        host = torch.empty((), dtype=torch.long, pin_memory=True)
        host.copy_(n_dead, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._pending.append((host, ev))
        if len(self._pending) > self.LAG:
            old, old_ev = self._pending.pop(0)
            old_ev.synchronize()
            self.capacity = self._bucket(int(old))


class FusedTopKSAEStep:
    def __init__(self, sae, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, comm=None,
                 overlap_chunks: int | None = None, dp_comm=None):
        """``comm``: a ``parallel.symm.SymmComm`` over the model group switches the two cross-shard exchanges
        from NCCL collectives to the fused peer-memory kernels. ``dp_comm``: a ``parallel.symm.DataParallelComm`` over
        the data group: the replicas exchange their rows in one peer-store kernel and the optimizer state is sharded by
        feature row (each replica updates ``F / dp`` rows and stores the new bf16 rows, norms and biases into every
        replica; the fp32 master rows of the other replicas' shares go stale until ``sync_params``).
        ``overlap_chunks``: number of feature chunks of the update / next-encode overlap (default: environment variable
        ``LMSAE_OVERLAP_CHUNKS``, else 1 = off)."""
        cfg = sae.cfg
        self.sae = sae
        self.mesh = sae.device_mesh
        self.tp = mesh_dim_size(self.mesh, "model")
        self.dp = mesh_dim_size(self.mesh, "data")
        self.tp_rank = mesh_local_rank(self.mesh, "model")
        self.tp_group = mesh_group(self.mesh, "model")
        self.dp_group = mesh_group(self.mesh, "data")
        self.comm = comm  # optional peer-memory communicator (parallel.symm.SymmComm) for the model group
        self.dp_comm = dp_comm if self.dp > 1 else None
        self.betas, self.eps = betas, eps
        self.use_gate = cfg.sparsity_include_decoder_norm
        self.batch_level = cfg.act_fn == "batchtopk"
        self._batch_thr: torch.Tensor | None = None  # last batch-level threshold (device), a hint for the next selection
        self.WE = sae.W_E.data.t()
        self.WD = sae.W_D.data
        assert self.WE.is_contiguous() and self.WD.is_contiguous(), "weights must be feature-major and contiguous"
        assert self.WE.dtype == torch.float32, "the fused step keeps fp32 master weights"
        self.bE = sae.b_E.data
        self.bD = sae.b_D.data if cfg.use_decoder_bias else None
        F, d = self.WD.shape
        self.F, self.d = F, d
        dev = self.WD.device
        z = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)  # noqa: E731
        if self.dp_comm is not None:
            # shadows, norms and the encoder bias live in the data group's symmetric buffer: the replica that updates a
            # feature row stores the new values into every replica's copy
            assert self.dp_comm.F == F and self.dp_comm.d == d and F % self.dp == 0
            views = self.dp_comm.param_views()
            self.WE_bf16, self.WD_bf16, self.dec_norm = views["WE_bf16"], views["WD_bf16"], views["dec_norm"]
            views["bE"].copy_(self.bE)
            sae.b_E.data = views["bE"]
            self.bE = sae.b_E.data
            self.own_rows = self.dp_comm.own_rows()
        else:
            self.WE_bf16 = torch.empty(F, d, dtype=torch.bfloat16, device=dev)
            self.WD_bf16 = torch.empty(F, d, dtype=torch.bfloat16, device=dev)
            self.dec_norm = torch.empty(F, dtype=torch.float32, device=dev)
            self.own_rows = (0, F)
        Fo = self.own_rows[1] - self.own_rows[0]  # rows whose optimizer state this rank holds
        self.state = {
            "W_E": (z(Fo, d), z(Fo, d)), "W_D": (z(Fo, d), z(Fo, d)), "b_E": (z(Fo), z(Fo)),
            "b_D": (z(d), z(d)) if self.bD is not None else None,
        }  # fmt: skip
        self._masters_stale = False
        self.groups: K.FeatureGroups | None = None
        self.loss_sum = z(1)
        self.aux_sum = z(1)
        self.batch_list_factor = int(os.environ.get("LMSAE_BATCH_LIST_FACTOR", "8"))
        self.list_overflow = torch.zeros(1, dtype=torch.int64, device=dev)  # tokens whose batch-level codes did not fit
        self.last_aux_loss: torch.Tensor | None = None
        self.main_counts: torch.Tensor | None = None
        self.grad_sq = z(1)
        self.last_grad_norm: torch.Tensor | None = None  # global gradient norm before clipping (set when clipping is on)
        self.phase_marks: list[tuple[str, torch.cuda.Event]] | None = None  # see start_phase_timing()
        self.t = 0
        # ---- update / next-encode overlap ----
        tiles = (F + 255) // 256
        if overlap_chunks is None:
            # Off by default. Measured on a B200 (d_model 4096, 131072 features, batch 4096): the update kernel needs
            # four CTAs per SM to reach its 5.4 TB/s, which leaves no registers for a GEMM CTA next to it; capped at two
            # CTAs per SM the two kernels do overlap but the update slows down by more than the GEMM time it hides
            # (10.8 ms per step against 9.2 ms in sequence).
            n_chunks = min(int(os.environ.get("LMSAE_OVERLAP_CHUNKS", "1")), tiles // 16)
        else:
            n_chunks = min(overlap_chunks, tiles)
        n_chunks = max(1, n_chunks) if self.WD.is_cuda else 1
        rows = -(-tiles // n_chunks) * 256
        self.chunks = [(lo, min(F, lo + rows)) for lo in range(0, F, rows)]
        self.adam_done: list[torch.cuda.Event | None] = [None] * len(self.chunks)
        self._inflight: tuple | None = None  # tensors the update stream may still be reading
        self.overlap_ctas_per_sm = int(os.environ.get("LMSAE_OVERLAP_CTAS", "2"))
        if len(self.chunks) > 1:
            self.gemm_stream = torch.cuda.Stream(device=dev, priority=-1)
            self.adam_stream = torch.cuda.Stream(device=dev)
        self.refresh()

    # ---- bookkeeping -------------------------------------------------------------------------
    @staticmethod
    def supports(sae, trainer_cfg=None) -> tuple[bool, str]:
        """Whether this model / training configuration can run on the fused path, and if not, why."""
        from ..models.sae import SparseAutoEncoder

        cfg = sae.cfg
        if type(sae) is not SparseAutoEncoder:
            return False, "model is not a plain SparseAutoEncoder"
        checks = [
            (cfg.act_fn in ("topk", "batchtopk"), "activation is neither topk nor batchtopk"),
            (not cfg.use_glu_encoder, "GLU encoder"),
            (sae.W_D.is_cuda, "not on a CUDA device"),
            (cfg.dtype == torch.float32, "parameters are not fp32"),
            (cfg.d_model % 8 == 0 and sae.W_D.shape[0] % 8 == 0, "d_model / local d_sae not multiples of 8"),
            (cfg.d_model <= 8192, "d_model > 8192"),
            (not any(hp.fwd_hooks or hp.bwd_hooks for hp in sae.hook_points()), "hooks are attached"),
            (mesh_dim_size(sae.device_mesh, "head") == 1 and mesh_dim_size(sae.device_mesh, "sweep") == 1, "head/sweep mesh"),
        ]
        if trainer_cfg is not None:
            checks += [
                (trainer_cfg.sparsity_loss_type is None, "sparsity loss"),
                (not trainer_cfg.lp_coefficient, "lp loss"),
                (trainer_cfg.optimizer_class == "adam", "optimizer is not adam"),
                (trainer_cfg.amp_dtype == torch.bfloat16, "amp dtype is not bf16"),
                (trainer_cfg.gradient_accumulation_steps == 1, "gradient accumulation"),
            ]
        for ok, why in checks:
            if not ok:
                return False, why
        return True, ""

    # ---- per-phase device timing (diagnostics) -------------------------------------------------
    def start_phase_timing(self) -> None:
        """From now on ``step`` drops a timing event into the stream after each of its phases. Events are markers, not
        synchronisation points; ``phase_times`` reads them back."""
        self.phase_marks = []

    def _mark(self, name: str) -> None:
        if self.phase_marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.phase_marks.append((name, ev))

    def phase_times(self) -> dict[str, float]:
        """Mean milliseconds per step of every phase since ``start_phase_timing`` (synchronises), and stops the marking.
        A phase's time runs from the previous mark to its own, so it contains the wait for peers that the phase's
        kernels do on entry."""
        marks, self.phase_marks = self.phase_marks or [], None
        torch.cuda.synchronize()
        total: dict[str, float] = {}
        steps = max(1, sum(1 for n, _ in marks if n == "begin"))
        for (_, a), (name, b) in zip(marks, marks[1:]):
            name = "between_steps" if name == "begin" else name
            total[name] = total.get(name, 0.0) + a.elapsed_time(b)
        return {n: t / steps for n, t in total.items()}

    def join(self) -> None:
        """Make the current stream wait for every update launched so far (call before reading or writing the weights,
        the optimizer state or the bf16 shadows outside ``step``)."""
        if any(e is not None for e in self.adam_done):
            cur = torch.cuda.current_stream(self.WD.device)
            for e in self.adam_done:
                if e is not None:
                    cur.wait_event(e)
            self.adam_done = [None] * len(self.chunks)
        self._inflight = None

    def refresh(self) -> None:
        """Re-derive bf16 shadows and decoder norms from the fp32 masters (after loading / editing weights)."""
        self.join()
        K.row_norm_shadow(self.WD, self.dec_norm, self.WD_bf16)
        K.row_norm_shadow(self.WE, None, self.WE_bf16)

    def _full_rows(self, t: torch.Tensor) -> torch.Tensor:
        """A row-sharded state tensor (this replica's feature rows) as the full local-shard tensor (collective)."""
        if self.dp_comm is None:
            return t
        out = torch.empty(self.dp * t.shape[0], *t.shape[1:], dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=self.dp_group)
        return out

    def sync_params(self) -> None:
        """With the optimizer state sharded over replicas, each replica's fp32 master rows of the OTHER replicas' shares
        are stale between steps (only the bf16 shadows, norms and biases are published every step). This gathers the
        current master rows into every replica's ``W_E`` / ``W_D`` (collective; call before saving or inspecting the
        parameters)."""
        self.join()
        if self.dp_comm is None or not self._masters_stale:
            return
        lo, hi = self.own_rows
        self.WD.copy_(self._full_rows(self.WD[lo:hi]))
        self.WE.copy_(self._full_rows(self.WE[lo:hi]))
        self._masters_stale = False

    def optimizer_state(self) -> dict:
        """Adam state in logical parameter shapes (W_E as [d, F]); collective when the state is sharded over replicas."""
        self.join()
        out = {"step": self.t}
        for name, st in self.state.items():
            if st is None:
                continue
            m, v = st
            if name != "b_D":
                m, v = self._full_rows(m), self._full_rows(v)
            out[name] = {"exp_avg": m.t() if name == "W_E" else m, "exp_avg_sq": v.t() if name == "W_E" else v}
        return out

    def load_optimizer_state(self, sd: dict) -> None:
        self.join()
        self.t = int(sd["step"])
        lo, hi = self.own_rows
        for name, st in self.state.items():
            if st is None or name not in sd:
                continue
            m, v = st
            src_m, src_v = sd[name]["exp_avg"], sd[name]["exp_avg_sq"]
            if name == "W_E":
                src_m, src_v = src_m.t(), src_v.t()
            if name != "b_D" and src_m.shape[0] != m.shape[0]:
                src_m, src_v = src_m[lo:hi], src_v[lo:hi]
            m.copy_(src_m)
            v.copy_(src_v)

    # ---- the step ----------------------------------------------------------------------------
    def _candidates_chunked(self, x: torch.Tensor, k: int, gate) -> tuple[torch.Tensor, torch.Tensor]:
        """Encoder GEMM + top-k candidates, one launch per feature chunk on the high-priority stream; chunk ``c`` starts
        when the previous step's update of chunk ``c`` is done."""
        cur = torch.cuda.current_stream(x.device)
        ready = torch.cuda.Event()
        ready.record(cur)
        x.record_stream(self.gemm_stream)
        S = min(K.choose_splits(x.shape[0], hi - lo) for lo, hi in self.chunks)
        with torch.cuda.stream(self.gemm_stream):
            self.gemm_stream.wait_event(ready)
            state = None
            for c, (lo, hi) in enumerate(self.chunks):
                if self.adam_done[c] is not None:
                    self.gemm_stream.wait_event(self.adam_done[c])
                cv, ci, _ = K.encoder_topk_candidates(
                    x, self.WE_bf16[lo:hi], self.bE[lo:hi], gate[lo:hi] if gate is not None else None, k,
                    num_splits=S, n_index_offset=lo, resume=state, compact_smem=True,
                )
                state = (cv, ci)
            done = torch.cuda.Event()
            done.record(self.gemm_stream)
        cur.wait_event(done)
        cv.record_stream(cur)
        ci.record_stream(cur)
        # everything below on `cur` is ordered after every update of the previous step
        self.adam_done = [None] * len(self.chunks)
        self._inflight = None
        return cv, ci

    def encode(self, x: torch.Tensor, k: int, _in_step: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
        """Sparse codes (idx, act) [B, k] of bf16 inputs ``x`` [B, d] over this rank's features; under
        feature sharding only globally selected entries survive, packed from slot 0 of every row on."""
        gate = self.dec_norm if self.use_gate else None
        if self.batch_level:
            return self._encode_batch_level(x, k, gate)
        chunked = _in_step and len(self.chunks) > 1 and k <= 64 and x.is_cuda
        if not chunked:
            self.join()
        fused_topk = k <= 64 and x.is_cuda
        use_comm = self.tp > 1 and self.comm is not None and x.shape[0] == self.comm.B and k <= self.comm.k_max
        if fused_topk:
            if chunked:
                cv, ci = self._candidates_chunked(x, k, gate)
            else:
                cv, ci, _ = K.encoder_topk_candidates(x, self.WE_bf16, self.bE, gate, k)
            self._mark("encoder_gemm_topk")
            if self.tp == 1:
                return K.topk_merge(cv, ci, k, gate)
            if use_comm:
                # local merge whose epilogue is the all-gather of the shard's list, then the merge over shards, which
                # waits for the peers' flags inside its kernel
                self.comm.merge_push(cv, ci, k)
                self._mark("local_merge_push")
                out = self.comm.merge_shards(k, gate)
                self._mark("merge_shards")
                return out
            idx_l, g_l = K.topk_merge(cv, ci, k, gate, emit_gated=True)
            self._mark("local_merge")
        else:
            H = K.encoder_hidden(x, self.WE_bf16, self.bE)
            idx_l, act_l = K.row_topk(H, k, gate, None)
            if self.tp == 1:
                return idx_l, act_l
            g_l = act_l * gate[idx_l.clamp_min(0).long()] if gate is not None else act_l
            if use_comm:
                self.comm.push_candidates(g_l, idx_l)
                return self.comm.merge_shards(k, gate)
        B = x.shape[0]
        all_g = torch.empty(self.tp * B, k, dtype=torch.float32, device=x.device)
        all_i = torch.empty(self.tp * B, k, dtype=torch.int32, device=x.device)
        dist.all_gather_into_tensor(all_g, g_l.contiguous(), group=self.tp_group)
        dist.all_gather_into_tensor(all_i, idx_l.contiguous(), group=self.tp_group)
        all_g = all_g.view(self.tp, B, k).permute(1, 0, 2).reshape(B, self.tp * k).contiguous()
        all_i = all_i.view(self.tp, B, k).permute(1, 0, 2).reshape(B, self.tp * k).contiguous()
        return K.topk_merge(all_g, all_i, k, gate, own=(self.tp_rank * k, (self.tp_rank + 1) * k))

    def _encode_batch_level(self, x: torch.Tensor, k: int, gate) -> tuple[torch.Tensor, torch.Tensor]:
        """BatchTopK: keep the ``k * batch`` largest gated pre-activations of the whole batch (over all feature shards)
        instead of ``k`` per token (models/sparse_dictionary.py:775-788 of the reference project). The GEMM stores the
        gated pre-activations in bf16, a radix select over their bit patterns finds the threshold (shards add their
        histograms), and one compaction pass turns the survivors into padded code lists. The rows' code counts differ;
        the lists have a fixed width of ``batch_list_factor * k`` (default 8) so that nothing is read back to the host.
        A token with more codes than that keeps its first ones by column and is counted in ``self.list_overflow``,
        which the trainer reports with the metrics."""
        from . import select_kernels as S

        self.join()
        G = K.encoder_hidden(x, self.WE_bf16, self.bE, gate=gate)
        self._mark("encoder_gemm_hidden")
        B = x.shape[0]
        tp_group = self.tp_group if self.tp > 1 else None
        # (the previous batch's threshold, lowered by a quarter, as the histogram pass's floor: see positive_thresholds)
        floor = self._batch_thr * 0.75 if self._batch_thr is not None and G.is_cuda else None
        thr, n_ties = S.positive_thresholds(G.view(1, 1, -1), k * B, tp_group, return_remaining=True, floor=floor)
        self._batch_thr = thr
        self._mark("batch_threshold_select")
        # exactly k * B codes: of the entries equal to the (bf16) threshold only as many as the selection still needs
        cap = -(-self.batch_list_factor * k // 8) * 8
        out = S.threshold_rows_to_sparse(G, thr, gate, n_ties=n_ties, tie_group=tp_group, cap=cap, overflow=self.list_overflow)
        self._mark("rows_to_code_lists")
        return out

    def step(
        self,
        x: torch.Tensor,
        label: torch.Tensor,
        k: int,
        lr: float,
        row_weight: torch.Tensor | None = None,
        n_tokens_global: int | None = None,
        grad_mul: torch.Tensor | None = None,
        want_grad_norm: bool = False,
        aux: "AuxK | None" = None,
        clip_grad_norm: float = 0.0,
    ) -> torch.Tensor:
        """Forward, backward and Adam update for one batch; returns the mean loss (0-d device tensor, local
        batch). ``x`` / ``label``: normalised bf16 [B, d]; ``row_weight``: optional 0/1 token mask. ``aux`` adds the
        Aux-K dead-feature loss (its mean is left in ``self.last_aux_loss`` and included in the returned loss).
        ``clip_grad_norm`` > 0 scales the gradient down when its norm (2-norm over the root of the number of non-zero
        entries, the trainer's definition; left in ``self.last_grad_norm``) exceeds that value: the gradient is never materialised, so the sparse gradient
        kernel runs twice, first without writing anything to accumulate the squared norm, then with the factor."""
        if aux is not None:
            return self._step_auxk(x, label, k, lr, row_weight, n_tokens_global, aux, clip_grad_norm)
        B = x.shape[0]
        n_global = n_tokens_global if n_tokens_global is not None else B * self.dp
        grad_scale = 2.0 / n_global
        use_comm = self.tp > 1 and self.comm is not None and B == self.comm.B and (self.batch_level or k <= self.comm.k_max)
        sharded = self.dp_comm is not None
        overlap = len(self.chunks) > 1 and k <= 64 and grad_mul is None and not want_grad_norm and not clip_grad_norm and not sharded
        self._mark("begin")
        if self.dp_comm is not None:
            self.dp_comm.wait_params()  # the other replicas' rows of the previous update must have landed in the shadows
        idx, act = self.encode(x, k, _in_step=overlap)
        self._mark("merge")
        self.loss_sum.zero_()
        if use_comm:
            # loss_sum collects the rows this rank owns; scale to a local-batch estimate for the return value
            dxhat, _ = self.comm.decode_reduce_loss(idx, act, self.WD_bf16, label, self.bD, row_weight, grad_scale, self.loss_sum)
            self._mark("decode_reduce_loss")
            dact = self.comm.dact(idx, self.WD_bf16)  # waits for the owners' gradient rows inside the kernel
            self._mark("dact")
        elif self.tp == 1:
            dxhat, dact, _ = K.sparse_decode_loss(idx, act, self.WD_bf16, self.bD, label, row_weight, grad_scale, self.loss_sum)
        else:
            partial = K.sparse_decode(idx, act, self.WD_bf16, None, torch.float32)
            dist.all_reduce(partial, group=self.tp_group)
            dxhat = K.mse_loss_grad(partial, label, self.bD, row_weight, grad_scale, self.loss_sum)
            dact = K.sparse_dact(idx, self.WD_bf16, dxhat)
        if self.dp_comm is not None:
            g = self.dp_comm.exchange({"x": x, "dxhat": dxhat, "idx": idx, "act": act, "dact": dact})
            x, dxhat, idx, act, dact = g["x"], g["dxhat"], g["idx"], g["act"], g["dact"]
            self._mark("dp_exchange_rows")
        elif self.dp > 1:
            x, dxhat, idx, act, dact = self._gather_rows(x, dxhat, idx, act, dact)
        if self.groups is None or self.groups.entries.numel() < idx.numel():
            self.groups = K.FeatureGroups(self.F, idx.numel(), x.device)
        if not use_comm:
            self._mark("decode_loss_dact")
        self.groups.build(idx)
        self._mark("sort_by_feature")
        self.t += 1
        b1, b2 = self.betas
        (mE, vE), (mD, vD), (mb, vb) = self.state["W_E"], self.state["W_D"], self.state["b_E"]
        gsq = None
        if want_grad_norm:
            self.grad_sq.zero_()
            gsq = self.grad_sq
        def sparse(mul, sq, update, f_range=None, ctas_per_sm=0):
            K.sparse_grad_adam(
                self.groups, act, dact, x, dxhat, self.WD, mD, vD, self.WD_bf16, self.WE, mE, vE, self.WE_bf16,
                self.bE, mb, vb, self.dec_norm, mul, sq, lr, b1, b2, self.eps, self.t, update,
                f_range=f_range if not sharded else self.own_rows, ctas_per_sm=ctas_per_sm,
                state_f0=self.own_rows[0], publish=self.dp_comm.pub_args() if sharded and update else None,
            )  # fmt: skip
            if sharded and update:
                self._masters_stale = True

        g_bD = K.colsum_bf16(dxhat) if self.bD is not None else None
        if clip_grad_norm:
            assert grad_mul is None, "pass either a gradient factor or a clipping norm"
            grad_mul, gsq = self._clip_factor(sparse, g_bD, clip_grad_norm), None
        adam = lambda f_range=None, ctas_per_sm=0: sparse(grad_mul, gsq, True, f_range, ctas_per_sm)  # noqa: E731

        def bias_update():
            if self.bD is not None:
                m, v = self.state["b_D"]
                K.adam_flat(self.bD, g_bD, m, v, lr, b1, b2, self.eps, self.t, grad_mul=grad_mul, grad_sq_sum=gsq)

        if overlap:
            cur = torch.cuda.current_stream(x.device)
            ready = torch.cuda.Event()
            ready.record(cur)
            keep = (x, label, act, dact, dxhat, idx)
            for t in keep:
                t.record_stream(self.adam_stream)
            self._inflight = keep
            with torch.cuda.stream(self.adam_stream):
                self.adam_stream.wait_event(ready)
                bias_update()
                for c, f_range in enumerate(self.chunks):
                    # two update CTAs per SM: the encoder GEMM of the next step (one CTA per SM, < 200 KB of shared
                    # memory in this mode) always finds the registers it needs next to them
                    adam(f_range, self.overlap_ctas_per_sm)
                    ev = torch.cuda.Event()
                    ev.record(self.adam_stream)
                    self.adam_done[c] = ev
        else:
            adam()
            self._mark("sparse_grad_adam")
            bias_update()
            self._mark("bias_update")
        n_local = B if row_weight is None else row_weight.sum()
        if use_comm:
            n_local = n_local / self.tp  # each rank evaluated the loss on the B / tp rows it owns
        return (self.loss_sum / n_local).squeeze(0)

    def _clip_factor(self, sparse, g_bD: torch.Tensor | None, max_norm: float, extra_fired: torch.Tensor | None = None) -> torch.Tensor:
        """The trainer's clipping factor as a 1-element device tensor. The norm is the reference project's
        (optim.py:255-292 there): ``|g|_2 / sqrt(number of non-zero gradient entries)``, and the gradient is scaled by
        ``max_norm / (norm + 1e-6)`` only when the norm exceeds ``max_norm``. ``sparse(mul, sq, update)`` launches the
        sparse gradient kernel; here it only accumulates squared gradient entries of this rank's feature rows. A
        feature that fired has ``2 d + 1`` gradient entries (its decoder row, encoder row and encoder bias), counted as
        non-zero; sharded parameters add up over the model group, the replicated decoder bias is counted once."""
        self.grad_sq.zero_()
        sparse(None, self.grad_sq, False)
        lo, hi = self.own_rows  # the rows this replica rebuilt gradients for (all of them unless the state is sharded)
        fired = (self.groups.counts[lo:hi] > 0).sum().float().reshape(1)
        if extra_fired is not None:  # features that received gradient rows from elsewhere only (dead features of Aux-K)
            fired = fired + extra_fired
        acc = torch.cat([self.grad_sq, fired * (2 * self.d + 1)])
        if self.tp > 1:
            dist.all_reduce(acc, group=self.tp_group)
        if self.dp_comm is not None:
            dist.all_reduce(acc, group=self.dp_group)
        if g_bD is not None:
            acc = acc + torch.stack([g_bD.square().sum(), (g_bD != 0).sum().float()])
        norm = (acc[0] / acc[1].clamp_min(1.0)).sqrt()
        self.last_grad_norm = norm
        return torch.where(norm > max_norm, max_norm / (norm + 1e-6), torch.ones_like(norm)).reshape(1)

    def _step_auxk(self, x, label, k, lr, row_weight, n_tokens_global, aux: "AuxK", clip_grad_norm: float = 0.0) -> torch.Tensor:
        """The step with the Aux-K loss: ``l = |e|^2 + alpha |e - e_aux|^2`` where ``e_aux`` decodes the ``k_aux`` largest
        gated pre-activations among DEAD features (models/sparse_dictionary.py:941-991 and trainer.py:428-454 of the
        reference project). The dead features are gathered into a compact dictionary of fixed capacity first (see
        ``AuxK``), so the second encoder pass costs ``capacity / F`` of the main one instead of a full pass, and no size
        travels through the host: with fewer dead features than ``k_aux`` the lists simply hold fewer codes, and with
        none the auxiliary term is switched off by a device-side factor. Works on one GPU, with feature shards (the
        auxiliary top-k is merged over shards, both reconstructions are summed over them) and with data-parallel
        replicas (dead statistics over the global batch, rows of both gradients exchanged before the update)."""
        self.join()
        self._mark("begin")
        if self.dp_comm is not None:
            self.dp_comm.wait_params()  # the other replicas' rows of the previous update must have landed in the shadows
        B = x.shape[0]
        n_global = n_tokens_global if n_tokens_global is not None else B * self.dp
        grad_scale = 2.0 / n_global
        gate = self.dec_norm if self.use_gate else None
        idx, act = self.encode(x, k)
        self._mark("merge")
        kw = idx.shape[1]  # width of the main code lists (k, or the fixed list width of a batch-level top-k)
        if self.groups is None or self.groups.entries.numel() < B * self.dp * kw:
            self.groups = K.FeatureGroups(self.F, B * self.dp * kw, x.device)
        # dead statistics first (they include this batch), from the per-feature fire counts of the main codes
        self.groups.build(idx)
        self.main_counts = self.groups.counts[: self.F].clone()  # fire counts of the real codes (for metrics)
        fired = self.main_counts
        n_valid = torch.tensor(B, device=x.device) if row_weight is None else (row_weight > 0).sum()
        if self.dp > 1:  # a feature is alive when it fired on any replica; the counters advance by the global token count
            fired, n_valid = fired.clone(), n_valid.clone()
            dist.all_reduce(fired, group=self.dp_group)
            dist.all_reduce(n_valid, group=self.dp_group)
        is_dead = aux.update(fired, n_valid)
        n_dead = is_dead.sum()
        cap = min(aux.capacity, -(-self.F // 8) * 8)
        aux.observe(n_dead)
        n_dead_all = n_dead.clone()
        if self.tp > 1:  # the auxiliary top-k runs over the dead features of ALL shards
            dist.all_reduce(n_dead_all, group=self.tp_group)
        alpha_on = (n_dead_all > 0).float().reshape(1)  # no dead feature anywhere: the auxiliary term is absent, not |e|^2
        # compact dictionary of this shard's dead features: dead rows first (ascending), alive rows behind them with gate 0
        sharded = self.dp_comm is not None
        if sharded:
            # One block of slots per replica's share of the feature rows, so that the dense gradient rows of the compact
            # dictionary can be reduce-scattered over the replicas (each needs only the rows it updates).
            cap_r = max(1, min(cap // self.dp, self.F // self.dp))
            cap = cap_r * self.dp
            per = self.F // self.dp
            order = torch.argsort((~is_dead).view(self.dp, per).to(torch.int8), dim=1, stable=True)[:, :cap_r]
            order = (order + torch.arange(self.dp, device=x.device).unsqueeze(1) * per).reshape(-1)
            valid = is_dead[order]
        else:
            order = torch.argsort((~is_dead).to(torch.int8), stable=True)[:cap]
            if order.numel() < cap:  # fewer rows than the (rounded) capacity: repeat row 0 with gate 0
                order = torch.cat([order, order.new_zeros(cap - order.numel())])
                valid = torch.cat([is_dead[order[: self.F]], is_dead.new_zeros(cap - self.F)])
            else:
                valid = is_dead[order]
        w_dead = self.WE_bf16[order]
        wd_dead = self.WD_bf16[order]
        b_dead = self.bE[order]
        g_dead = (gate[order] if gate is not None else torch.ones(cap, device=x.device)) * valid
        self._mark("dead_statistics_compact_dictionary")
        self.loss_sum.zero_()
        self.aux_sum.zero_()
        xhat = K.sparse_decode(idx, act, self.WD_bf16, None, torch.float32)
        self._mark("main_decode")
        # The auxiliary codes hold up to k_aux (hundreds of) entries per token, several times the main codes, but all of
        # them index the compact dictionary: products with its [cap, d] matrices are small dense GEMMs, far cheaper than
        # gathering a decoder row per code, so the auxiliary decode and its three gradients are dense over the compact
        # dictionary and only their result rows are handed to the update kernel.
        # (the selection itself: fused into the GEMM epilogue up to 64 codes, else over stored bf16 pre-activations)
        idx_c, act_aux = K.encoder_topk(x, w_dead, b_dead, g_dead, aux.k_aux)
        self._mark("aux_encoder_topk")
        if self.tp > 1:
            idx_c, act_aux = self._merge_shard_codes(idx_c, act_aux, g_dead, aux.k_aux)
            self._mark("aux_merge_shards")
        # dense dead activations; empty slots land in a dump column behind them (eight columns of padding: the rows of
        # the [B, cap] view below stay 16-byte aligned, which the library GEMMs need to run their fast kernels)
        A = torch.zeros(B, cap + 8, dtype=torch.bfloat16, device=x.device)
        A.scatter_(1, torch.where(idx_c >= 0, idx_c, torch.full_like(idx_c, cap)).long(), act_aux.to(torch.bfloat16))
        A = A[:, :cap]
        aux_rec = _mm_f32(A, wd_dead)
        if self.tp > 1:  # both reconstructions are sums over the shards' features
            both = torch.stack([xhat, aux_rec])
            dist.all_reduce(both, group=self.tp_group)
            xhat, aux_rec = both[0], both[1]
        self._mark("aux_decode_and_reduce")
        g_main, g_aux = K.auxk_loss_grad(xhat, aux_rec, label, self.bD, row_weight, grad_scale, aux.coefficient, self.loss_sum,
                                         self.aux_sum, alpha_factor=alpha_on)  # fmt: skip
        dact = K.sparse_dact(idx, self.WD_bf16, g_main)
        self._mark("loss_grad_dact")
        # gradient of the dead activations where they were selected (bf16 on the GPU: it is an operand of the next product)
        dA = (g_aux @ wd_dead.t() if x.is_cuda else _mm_f32(g_aux, wd_dead.t())) * (A != 0)
        extra_gD = _mm_f32(A.t(), g_aux)  # d W_D rows of the compact dictionary
        extra_gE = _mm_f32(dA.to(torch.bfloat16).t(), x)  # d W_E^T rows
        extra_gb = dA.sum(0, dtype=torch.float32)
        slots = torch.arange(cap, dtype=torch.int32, device=x.device)
        if sharded:
            # dense rows: summed over replicas, each replica receiving the block of the rows it updates (the sparse main
            # part is rebuilt from the exchanged rows below)
            mine = self.dp_comm.rank
            parts = []
            for t in (extra_gD, extra_gE):
                out = torch.empty(cap_r, t.shape[1], dtype=t.dtype, device=t.device)
                dist.reduce_scatter_tensor(out, t.contiguous(), group=self.dp_group)
                parts.append(out)
            dist.all_reduce(extra_gb, group=self.dp_group)
            extra_gD, extra_gE, extra_gb = parts[0], parts[1], extra_gb[mine * cap_r : (mine + 1) * cap_r].contiguous()
            slots = slots - mine * cap_r
            valid_mine = valid & (slots >= 0) & (slots < cap_r)
        else:
            if self.dp > 1:
                for t in (extra_gD, extra_gE, extra_gb):
                    dist.all_reduce(t, group=self.dp_group)
            valid_mine = valid
        row_of = torch.full((self.F,), -1, dtype=torch.int32, device=x.device)
        row_of.scatter_(0, order.long(), torch.where(valid_mine, slots, torch.full_like(slots, -1)))
        self._mark("aux_gradients")
        if sharded:
            g = self.dp_comm.exchange({"x": x, "dxhat": g_main, "idx": idx, "act": act, "dact": dact})
            x, g_main, idx, act, dact = g["x"], g["dxhat"], g["idx"], g["act"], g["dact"]
            self._mark("dp_exchange_rows")
        elif self.dp > 1:
            x, g_main, idx, act, dact = self._gather_rows(x, g_main, idx, act, dact)
            self._mark("dp_exchange_rows")
        self.groups.build(idx)
        self._mark("sort_by_feature")
        self.t += 1
        b1, b2 = self.betas
        (mE, vE), (mD, vD), (mb, vb) = self.state["W_E"], self.state["W_D"], self.state["b_E"]

        def sparse(mul, sq, update):
            K.sparse_grad_adam(
                self.groups, act, dact, x, g_main, self.WD, mD, vD, self.WD_bf16, self.WE, mE, vE, self.WE_bf16,
                self.bE, mb, vb, self.dec_norm, mul, sq, lr, b1, b2, self.eps, self.t, update,
                f_range=self.own_rows if sharded else None, state_f0=self.own_rows[0],
                publish=self.dp_comm.pub_args() if sharded and update else None,
                extra=(row_of, extra_gD, extra_gE, extra_gb),
            )  # fmt: skip
            if sharded and update:
                self._masters_stale = True

        g_bD = K.colsum_bf16(g_main) if self.bD is not None else None
        grad_mul = None
        if clip_grad_norm:
            lo, hi = self.own_rows
            got_aux = ((row_of[lo:hi] >= 0) & (self.groups.counts[lo:hi] == 0)).sum().float().reshape(1)
            grad_mul = self._clip_factor(sparse, g_bD, clip_grad_norm, extra_fired=got_aux)
        sparse(grad_mul, None, True)
        self._mark("sparse_grad_adam")
        if self.bD is not None:
            m, v = self.state["b_D"]
            K.adam_flat(self.bD, g_bD, m, v, lr, b1, b2, self.eps, self.t, grad_mul=grad_mul)
        self._mark("bias_update")
        n_local = B if row_weight is None else row_weight.sum()
        self.last_aux_loss = (self.aux_sum / n_local).squeeze(0)
        return ((self.loss_sum + self.aux_sum) / n_local).squeeze(0)

    def _merge_shard_codes(self, idx_l: torch.Tensor, act_l: torch.Tensor, gate_l: torch.Tensor | None, k: int):
        return merge_codes_over_shards(idx_l, act_l, gate_l, k, self.tp, self.tp_rank, self.tp_group)

    def _gather_rows(self, *tensors: torch.Tensor) -> list[torch.Tensor]:
        out = []
        for t in tensors:
            buf = torch.empty(self.dp * t.shape[0], *t.shape[1:], dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(buf, t.contiguous(), group=self.dp_group)
            out.append(buf)
        return out

    @torch.no_grad()
    def forward_dense(self, x: torch.Tensor, k: int):
        """Codes and reconstruction for metric computation: (idx, act, x_hat fp32)."""
        self.join()
        idx, act = self.encode(x, k)
        xhat = K.sparse_decode(idx, act, self.WD_bf16, None, torch.float32)
        if self.tp > 1:
            dist.all_reduce(xhat, group=self.tp_group)
        if self.bD is not None:
            xhat = xhat + self.bD
        return idx, act, xhat
