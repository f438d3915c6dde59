"""One training step of a JumpReLU crosscoder as a fixed sequence of sm_100a kernels, without autograd.

What it computes is the reference's step for a ``Crosscoder`` (models/crosscoder.py:350-378 encode, :384-469 decode,
models/sparse_dictionary.py:841-936 loss, activation_functions.py:15-64 JumpReLU with its straight-through threshold
gradient): every head encodes its own activation, the pre-activations are summed over ALL heads, each head gates the sum
with its decoder norms, applies ``JumpReLU`` and decodes with its own decoder; the loss is the mean over tokens and heads
of the squared error plus, optionally, the ``tanh`` sparsity penalty; Adam on every parameter. How it computes it:

1. head sum: one tcgen05 GEMM accumulates the local heads in its K loop (K = local heads x d_model) and stores bf16 into a
   symmetric buffer; one kernel sums that matrix over the head ranks in place (``parallel.symm.AllReduceComm``: the owner
   of a share reads the sum with ``multimem.ld_reduce`` -- added inside the NVSwitch -- and writes it to every rank with
   ``multimem.st``; peer loads / stores without a multicast mapping)                        -> S [B, F] bf16, all ranks
2. selection: one compaction pass keeps, per token, the features whose sum passes the threshold of ANY head
   (``S > min_h theta / ||W_D,h row||``): every rank derives the same lists in the same order; a head's codes are the
   list entries that pass ITS threshold (zero otherwise)                      -> idx [B, cap], per head act [B, cap]
3. per local head: sparse decode fused with the loss, d x_hat and d act (``sparse_decode_loss``)
4. the gradient of the shared sum is the sum over all heads of the heads' code gradients where the head is active: the
   lists are aligned on all ranks, so this is a small all-reduce of a [B, cap] array
5. per local head: the sparse gradient + Adam kernel rebuilds d W_D (codes x d x_hat) and d W_E^T (d S x inputs) rows from
   the lists and updates both matrices, bf16 shadows and decoder norms in one pass; no dense gradient exists
6. threshold gradient: the rectangle window of the straight-through estimator is wide (the default width 2 covers most
   positive pre-activations), so this gradient needs d loss / d act at INACTIVE entries too: one dense tcgen05 GEMM per
   head, G = d x_hat . W_D^T [B, F] bf16, and one streaming kernel that adds up G inside the window against S.

Restrictions: ``jumprelu`` activation, MSE loss with optional ``tanh`` sparsity loss, Adam, fp32 parameters with bf16
compute, heads split over the ``head`` mesh dimension only (no ``model`` / ``data`` sharding). A token with more
candidate features than the list width keeps its first ones by column and is counted in ``list_overflow``.

A JumpReLU ``SparseAutoEncoder`` that reconstructs its own input (models/sae.py:320-375 of the reference project) is the
one-head case of the same computation (``JumpReLU(pre * ||W_D row||) / ||W_D row||``, the same loss terms), so the step
takes it too: its parameters are viewed as ``[1, F, d]`` / ``[1, F]`` / ``[1, d]`` without a copy.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..parallel.mesh import mesh_dim_size, mesh_group
from . import sae_kernels as K
from . import select_kernels as S
from .fused_step import _mm_f32


def TANH_QUAD_ON_FUSED_PATH() -> bool:
    """The ``tanh-quad`` penalty on the fused step is verified against autograd on the CPU (the step's torch statements) and
    uses the same kernels as the ``tanh`` penalty, but it has not run on a GPU: the trainer takes it only on request."""
    return "1" in (os.environ.get("LMSAE_FUSED_TANH_QUAD", "0"), os.environ.get("LMSAE_FUSED_CPU_VERIFIED", "0"))


def FEATURE_SHARDS_ON_FUSED_PATH() -> bool:
    """Feature (``model``) shards of this step are verified against one process with ``gloo`` ranks on the CPU and use the
    kernels and NCCL calls of the other steps' shard paths, but have not run on GPUs: the trainer takes them only on request."""
    return "1" in (os.environ.get("LMSAE_FUSED_JUMPRELU_SHARDS", "0"), os.environ.get("LMSAE_FUSED_CPU_VERIFIED", "0"))


class FusedCrosscoderStep:
    def __init__(self, cc, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, list_width: int = 256,
                 jumprelu_lr_factor: float = 1.0):  # fmt: skip
        cfg = cc.cfg
        self.cc = cc
        self.betas, self.eps = betas, eps
        self.single = cc.W_D.ndim == 2  # a plain SAE: one head, parameters without the head axis
        self.head_size = mesh_dim_size(cc.device_mesh, "head")
        self.head_group = mesh_group(cc.device_mesh, "head")
        self.dp = mesh_dim_size(cc.device_mesh, "data")
        self.dp_group = mesh_group(cc.device_mesh, "data")
        self.tp = mesh_dim_size(cc.device_mesh, "model")  # features split over ranks: everything per feature stays local
        self.tp_group = mesh_group(cc.device_mesh, "model")
        self.window = float(cfg.jumprelu_threshold_window)
        self.cap = -(-list_width // 8) * 8
        self.jumprelu_lr_factor = jumprelu_lr_factor
        if self.single:
            self.H = self.H_l = 1
            self.F, self.d = cc.W_D.shape[0], cfg.d_model
            self.WE = cc.W_E.data.t().unsqueeze(0)  # [1, F, d]: views of the parameters' storage
            self.WD = cc.W_D.data.unsqueeze(0)
            self.bE, self.bD = cc.b_E.data.unsqueeze(0), cc.b_D.data.unsqueeze(0)
        else:
            self.H, self.H_l = cfg.n_heads, cc.n_heads_local
            self.F, self.d = cc.d_sae_local, cfg.d_model
            self.WE = cc.W_E.data.transpose(1, 2)  # [H_l, F, d], contiguous views of the parameters' storage
            self.WD = cc.W_D.data
            self.bE, self.bD = cc.b_E.data, cc.b_D.data
        assert self.WE.is_contiguous() and self.WD.is_contiguous() and self.WE.dtype == torch.float32
        self.log_theta = cc.activation_function.log_jumprelu_threshold.data
        dev = self.WD.device
        H_l, F, d = self.H_l, self.F, self.d
        z = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)  # noqa: E731
        self.WE_bf16 = torch.empty(H_l, F, d, dtype=torch.bfloat16, device=dev)
        self.WD_bf16 = torch.empty(H_l, F, d, dtype=torch.bfloat16, device=dev)
        self.dec_norm = torch.empty(H_l, F, dtype=torch.float32, device=dev)
        self.state = {"W_E": (z(H_l, F, d), z(H_l, F, d)), "W_D": (z(H_l, F, d), z(H_l, F, d)), "b_E": (z(H_l, F), z(H_l, F)),
                      "b_D": (z(H_l, d), z(H_l, d)), "log_theta": (z(F), z(F))}  # fmt: skip
        self.groups: K.FeatureGroups | None = None
        self.loss_sum = z(1)
        self.list_overflow = torch.zeros(1, dtype=torch.int64, device=dev)
        self.last: dict[str, torch.Tensor] = {}
        self.comm = None
        self.own_rows = (0, F)
        self.t = 0
        self.refresh()

    @staticmethod
    def supports(cc, trainer_cfg=None) -> tuple[bool, str]:
        from ..models.crosscoder import Crosscoder
        from ..models.sae import SparseAutoEncoder

        cfg = cc.cfg
        if type(cc) is SparseAutoEncoder:
            sae_checks = [
                (not cfg.use_glu_encoder, "GLU encoder"),
                (cfg.sparsity_include_decoder_norm, "activations are not gated by the decoder norms"),
                (cfg.use_decoder_bias, "no decoder bias"),
                (mesh_dim_size(cc.device_mesh, "head") == 1 and mesh_dim_size(cc.device_mesh, "sweep") == 1, "head/sweep mesh"),
            ]  # fmt: skip
            n_features = cc.W_D.shape[0]
        elif type(cc) is Crosscoder:
            sae_checks = []
            n_features = cc.d_sae_local
        else:
            return False, "model is neither a Crosscoder nor a plain SparseAutoEncoder"
        checks = sae_checks + [
            (cfg.act_fn == "jumprelu", "activation is not jumprelu"),
            (cc.W_D.is_cuda or trainer_cfg is None, "not on a CUDA device"),
            (cfg.dtype == torch.float32, "parameters are not fp32"),
            (cfg.d_model % 64 == 0, "d_model is not a multiple of 64"),
            (n_features % 8 == 0, "d_sae is not a multiple of 8"),
            (mesh_dim_size(cc.device_mesh, "model") == 1 or FEATURE_SHARDS_ON_FUSED_PATH(), "feature sharding (set LMSAE_FUSED_JUMPRELU_SHARDS=1)"),
            (not any(hp.fwd_hooks or hp.bwd_hooks for hp in cc.hook_points()), "hooks are attached"),
        ]  # fmt: skip
        if trainer_cfg is not None:
            checks += [
                (trainer_cfg.sparsity_loss_type in (None, "tanh") or (trainer_cfg.sparsity_loss_type == "tanh-quad" and TANH_QUAD_ON_FUSED_PATH()),
                 "sparsity loss other than tanh (tanh-quad: set LMSAE_FUSED_TANH_QUAD=1)"),
                (not trainer_cfg.auxk_coefficient, "aux-k loss"),
                (trainer_cfg.optimizer_class == "adam", "optimizer is not adam"),
                (trainer_cfg.amp_dtype == torch.bfloat16, "amp dtype is not bf16"),
                (trainer_cfg.gradient_accumulation_steps == 1, "gradient accumulation"),
                (not trainer_cfg.clip_grad_norm, "gradient clipping"),
                (not trainer_cfg.lp_coefficient or mesh_dim_size(cc.device_mesh, "data") == 1, "lp loss with data parallelism"),
            ]
        for ok, why in checks:
            if not ok:
                return False, why
        return True, ""

    def refresh(self) -> None:
        """Re-derive bf16 shadows and decoder norms from the fp32 masters (after loading / editing weights)."""
        for h in range(self.H_l):
            K.row_norm_shadow(self.WD[h], self.dec_norm[h], self.WD_bf16[h])
            K.row_norm_shadow(self.WE[h], None, self.WE_bf16[h])

    def join(self) -> None:
        pass

    def sync_params(self) -> None:
        pass

    def _head_sum(self, x16: torch.Tensor) -> torch.Tensor:
        """``sum over all heads of (x_h W_E,h^T + b_E,h)`` as bf16 [B, F] on every rank."""
        from ..parallel.symm import AllReduceComm

        B = x16.shape[0]
        if not x16.is_cuda:  # plain statement (CPU): local heads in one product, the other ranks by an all-reduce
            w = self.WE_bf16.view(self.H_l * self.F, self.d).float().view(self.H_l, self.F, self.d)
            s = torch.einsum("bhd,hfd->bf", x16.float().view(B, self.H_l, self.d), w) + self.bE.sum(0)
            if self.head_size > 1:
                dist.all_reduce(s, group=self.head_group)
            return s.to(torch.bfloat16)
        if self.comm is None or self.comm.max_rows < B:
            self.comm = AllReduceComm(self.head_group if self.head_size > 1 else None, x16.device, B, self.F)
        # the GEMM accumulates the local heads in one K loop and stores bf16 straight into the symmetric buffer ...
        P = self.comm.matrix(B)
        K._ext().head_sum_gemm(x16, self.WE_bf16.view(self.H_l * self.F, self.d), self.bE.sum(0).contiguous(), self.H_l, self.F, self.F,
                               True, K.status_buffer(x16.device), P)  # fmt: skip
        # ... which one kernel then sums over the head ranks in place (NVSwitch multicast loads / stores where available)
        return self.comm.all_reduce(B) if self.head_size > 1 else P

    def step(self, x: torch.Tensor, lr: float, l1_coefficient: float = 0.0, tanh_stretch: float = 4.0,
             row_weight: torch.Tensor | None = None, lp_coefficient: float = 0.0, sparsity_loss_type: str = "tanh",
             frequency_scale: float = 0.01, label: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
        """``x``: normalised bf16 activations ``[B, H_l, d]`` of this rank's heads (they are also the labels). Returns the
        mean loss over tokens and this rank's heads (0-d device tensor); ``self.last`` holds its parts.

        ``lp_coefficient``: weight of the pre-activation penalty ``sum_f relu(theta_f - S_bf) * ||W_D,h row f||`` (mean over
        tokens and heads; models/sparse_dictionary.py:928-936 of the reference project), which pulls the summed
        pre-activations of INACTIVE features towards their thresholds. It is dense in ``S``: its encoder gradient is one
        more GEMM per head (``1[S < theta]^T . x_h``, handed to the update kernel as dense gradient rows), its other
        gradients are column sums of ``S`` against the thresholds."""
        assert row_weight is None, "token masks are not supported on this path"
        assert not lp_coefficient or self.dp == 1, "the pre-activation penalty is not built for replicas"
        assert sparsity_loss_type in ("tanh", "tanh-quad"), sparsity_loss_type
        # ``label [B, H_l, d]``: targets that differ from the inputs (a transcoder reads one hook point and reconstructs
        # another); the inputs still feed the encoder and its gradient
        assert label is None or label.shape == x.shape
        quad = bool(l1_coefficient) and sparsity_loss_type == "tanh-quad"
        B_l, H_l, d = x.shape  # this replica's tokens
        B = B_l * self.dp  # the step's tokens: every replica brings the same number
        H, F, cap = self.H, self.F, self.cap
        grad_scale = 2.0 / (B * H)
        x = x.contiguous()
        S_sum = self._head_sum(x.view(B_l, H_l * d))
        theta = self.log_theta.exp()
        t_head = theta / self.dec_norm  # [H_l, F]: a head is active where S > theta / ||W_D,h row||
        t_min = t_head.amin(0)
        if self.head_size > 1:
            dist.all_reduce(t_min, op=dist.ReduceOp.MIN, group=self.head_group)
        idx, s_val = S.column_threshold_rows_to_sparse(S_sum, t_min, cap, overflow=self.list_overflow)
        safe = idx.clamp_min(0).long()
        valid = idx >= 0
        # scatter target of the per-feature sums below: empty slots go to a dump element of their own row (sending them all
        # to one element would serialise a million atomic additions on it)
        dump = F + (torch.arange(B_l, device=x.device) % 1024).unsqueeze(1)
        scat = torch.where(valid, safe, dump.expand_as(safe)).reshape(-1)
        self.loss_sum.zero_()
        dS = torch.zeros(B_l, cap, dtype=torch.float32, device=x.device)
        dtheta_buf = torch.zeros(F + 1024, dtype=torch.float32, device=x.device)
        dtheta = dtheta_buf[:F]
        l_s_sum = torch.zeros((), dtype=torch.float32, device=x.device)
        per_head = []
        c = float(tanh_stretch)
        lp = None
        if lp_coefficient:
            c_lp = lp_coefficient / (B * H)
            Sf = S_sum.float()
            below = Sf < theta  # [B, F]: where the penalty is active
            count = below.sum(0).float()  # per feature: tokens below the threshold
            gap = torch.relu(theta - Sf).sum(0)  # per feature: summed distance to the threshold
            n_local = self.dec_norm.sum(0)  # [F]: norms summed over this rank's heads ...
            n_all = n_local.clone()
            if self.head_size > 1:  # ... and over all heads: the shared sum feels every head's term
                dist.all_reduce(n_all, group=self.head_group)
            dtheta += c_lp * n_local * count  # (summed over the head ranks below, with the rest of d theta)
            lp = {"mask": below.to(torch.bfloat16), "row_scale": -c_lp * n_all, "gb": -c_lp * n_all * count, "gap": gap,
                  "rows": torch.arange(F, dtype=torch.int32, device=x.device), "c": c_lp}  # fmt: skip
            l_p_sum = c_lp * (gap * n_local).sum() * H / H_l  # mean over tokens and THIS rank's heads
        mult = None  # per-feature factor on every derivative of the sparsity penalty (1 for the plain tanh penalty)
        if quad:
            # tanh-quad: l_s = l1 * sum_f q_f (1 + q_f / scale) with q_f the mean of tanh(c * act * norm) over ALL tokens and
            # heads (models/sparse_dictionary.py:906-915 of the reference project). Its derivative with respect to one entry is
            # the tanh penalty's times (1 + 2 q_f / scale): one pass over the lists for q, then the tanh code with that factor.
            q_sum = torch.zeros(F + 1024, dtype=torch.float32, device=x.device)
            for h in range(H_l):
                active_h = valid & (s_val > t_head[h][safe])
                u_h = torch.tanh(c * s_val * self.dec_norm[h][safe]) * active_h
                q_sum.index_add_(0, scat, u_h.reshape(-1))
            q = q_sum[:F]
            if self.head_size > 1:
                dist.all_reduce(q, group=self.head_group)
            if self.dp > 1:
                dist.all_reduce(q, group=self.dp_group)
            q = q / (B * H)
            mult = 1.0 + 2.0 * q / frequency_scale
            l_s_quad = l1_coefficient * (q * (1.0 + q / frequency_scale)).sum()
        for h in range(H_l):
            xh = x[:, h].contiguous()
            n_h = self.dec_norm[h]
            active = valid & (s_val > t_head[h][safe])
            act = torch.where(active, s_val, torch.zeros_like(s_val))
            target = xh if label is None else label[:, h].contiguous()
            if self.tp == 1:
                dxhat, dact, _ = K.sparse_decode_loss(idx, act, self.WD_bf16[h], self.bD[h], target, None, grad_scale, self.loss_sum)
            else:
                # feature shards: partial reconstructions summed over the shards, then loss and output gradient (the same on
                # every shard), then the code gradients of this shard's features
                xhat = K.sparse_decode(idx, act, self.WD_bf16[h], None, torch.float32)
                dist.all_reduce(xhat, group=self.tp_group)
                dxhat = K.mse_loss_grad(xhat, target, self.bD[h], None, grad_scale, self.loss_sum)
                dact = K.sparse_dact(idx, self.WD_bf16[h], dxhat)
            n_e = n_h[safe]
            self_scale = None
            coef = 0.0
            if l1_coefficient:
                u = torch.tanh(c * act * n_e)
                sech2 = 1.0 - u * u
                l_s_sum = l_s_sum + (u * active).sum()
                coef = l1_coefficient * c / (B * H)
                m_e = mult[safe] if mult is not None else 1.0  # the tanh-quad factor of every entry's feature
                dact = dact + coef * n_e * sech2 * active * m_e
                # the penalty also pulls on the decoder norm: d / d W_D[f] = (sum_b coef * act * sech^2) * W_D[f] / ||W_D[f]||
                per_feat = torch.zeros(F + 1024, dtype=torch.float32, device=x.device)
                per_feat.index_add_(0, scat, (coef * act * sech2 * active * m_e).reshape(-1))
                self_scale = per_feat[:F] / n_h
            if lp is not None:  # the penalty's pull on this head's decoder norms: d / d W_D[f] = c * gap_f * W_D[f] / ||W_D[f]||
                pull = lp["c"] * lp["gap"] / n_h
                self_scale = pull if self_scale is None else self_scale + pull
            dS_h = dact * active
            dS += dS_h
            # threshold gradient: dense part (reconstruction gradient at every entry inside the window) ...
            # (the tanh penalty's derivative with respect to the JumpReLU output is coef at every entry with zero activation:
            # the dense pass adds it per window hit)
            G = K.encoder_hidden(dxhat, self.WD_bf16[h], None)  # [B, F] bf16 = d x_hat . W_D^T
            if mult is None:
                S.jumprelu_window_grad(G, S_sum, n_h, theta, self.window, dtheta, add_per_hit=coef if l1_coefficient else 0.0)
            else:
                # the per-hit term carries a per-feature factor here: the kernel runs with 0 and with 1 per hit; the difference
                # of the two sums is (hits of the feature) x (-theta / window), which is then scaled by coef x factor
                d0 = torch.zeros(F, dtype=torch.float32, device=x.device)
                d1 = torch.zeros(F, dtype=torch.float32, device=x.device)
                S.jumprelu_window_grad(G, S_sum, n_h, theta, self.window, d0, add_per_hit=0.0)
                S.jumprelu_window_grad(G, S_sum, n_h, theta, self.window, d1, add_per_hit=1.0)
                dtheta += d0 + coef * mult * (d1 - d0)
            if l1_coefficient:  # ... and the active entries, whose derivative is coef * sech^2, are corrected on the lists
                x_e = s_val * n_e
                hit = active & ((x_e - theta[safe]).abs() < 0.5 * self.window)
                contrib = coef * (sech2 - 1.0) * (-theta[safe] / self.window) * hit * m_e
                dtheta_buf.index_add_(0, scat, contrib.reshape(-1))
            per_head.append((xh, act, dxhat, self_scale))
        if self.head_size > 1:  # the lists are the same on every rank: the sum over heads is element-wise
            dist.all_reduce(dS, group=self.head_group)
            dist.all_reduce(dtheta, group=self.head_group)
        n_valid = valid.sum()
        if self.tp > 1:  # figures that are sums over features: the shards' parts add up (reporting only)
            part = torch.stack([l_s_sum, n_valid.float(), l_s_quad if quad else l_s_sum.new_zeros(()), l_p_sum if lp is not None else l_s_sum.new_zeros(())])
            dist.all_reduce(part, group=self.tp_group)
            l_s_sum, n_valid = part[0], part[1]
            if quad:
                l_s_quad = part[2]
            if lp is not None:
                l_p_sum = part[3]
        if self.dp > 1:
            # Replicas: what is a sum over tokens (threshold gradient, the penalty's pull on the decoder norms, the losses) is
            # summed over the replicas; the lists, their gradients, the inputs and the output gradients of every replica are
            # gathered in rank order, and every replica rebuilds the same sparse rows from them.
            dist.all_reduce(dtheta, group=self.dp_group)
            sums = torch.cat([self.loss_sum, l_s_sum.reshape(1), n_valid.reshape(1).float()])
            dist.all_reduce(sums, group=self.dp_group)
            self.loss_sum.copy_(sums[:1])
            l_s_sum, n_valid = sums[1], sums[2]
            idx, dS = self._gather_rows(idx), self._gather_rows(dS)
            gathered = []
            for xh, act, dxhat, self_scale in per_head:
                if self_scale is not None:
                    dist.all_reduce(self_scale, group=self.dp_group)
                gathered.append((self._gather_rows(xh), self._gather_rows(act), self._gather_rows(dxhat), self_scale))
            per_head = gathered
        if self.groups is None or self.groups.entries.numel() < idx.numel():
            self.groups = K.FeatureGroups(F, idx.numel(), x.device)
        self.groups.build(idx)
        self.t += 1
        b1, b2 = self.betas
        for h, (xh, act, dxhat, self_scale) in enumerate(per_head):
            (mE, vE), (mD, vD), (mb, vb) = self.state["W_E"], self.state["W_D"], self.state["b_E"]
            extra = None
            if lp is not None:  # dense encoder gradient rows of the pre-activation penalty: -c N_f (1[S < theta]^T x_h)[f, :]
                gE = _mm_f32(lp["mask"].t(), xh) * lp["row_scale"].unsqueeze(1)
                extra = (lp["rows"], None, gE, lp["gb"])
            K.sparse_grad_adam(self.groups, act, dS, xh, dxhat, self.WD[h], mD[h], vD[h], self.WD_bf16[h], self.WE[h], mE[h], vE[h],
                               self.WE_bf16[h], self.bE[h], mb[h], vb[h], self.dec_norm[h], None, None, lr, b1, b2, self.eps, self.t,
                               True, wd_self_scale=self_scale, extra=extra)  # fmt: skip
            m, v = self.state["b_D"]
            K.adam_flat(self.bD[h], K.colsum_bf16(dxhat), m[h], v[h], lr, b1, b2, self.eps, self.t)
        m, v = self.state["log_theta"]
        K.adam_flat(self.log_theta, dtheta * theta, m, v, lr * self.jumprelu_lr_factor, b1, b2, self.eps, self.t)
        l_rec = (self.loss_sum / (B * H_l)).squeeze(0)
        l_s = l_s_quad if quad else l1_coefficient * l_s_sum / (B * H_l)
        l_p = l_p_sum if lp is not None else torch.zeros((), device=x.device)
        self.last = {"l_rec": l_rec, "l_s": l_s, "l_p": l_p, "l0": n_valid / B}
        return l_rec + l_s + l_p

    def _gather_rows(self, t: torch.Tensor) -> torch.Tensor:
        """``[rows, n]`` of every replica stacked in rank order."""
        t = t.contiguous()
        out = torch.empty(self.dp * t.shape[0], *t.shape[1:], dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=self.dp_group)
        return out

    def optimizer_state(self) -> dict:
        out = {"step": self.t}
        names = {"W_E": "W_E", "W_D": "W_D", "b_E": "b_E", "b_D": "b_D", "log_theta": "activation_function.log_jumprelu_threshold"}
        for key, (m, v) in self.state.items():
            tr = (lambda t: t.transpose(1, 2)) if key == "W_E" else (lambda t: t)
            if self.single and key != "log_theta":  # logical shapes of the SAE's parameters (no head axis)
                out[names[key]] = {"exp_avg": tr(m).squeeze(0), "exp_avg_sq": tr(v).squeeze(0)}
            else:
                out[names[key]] = {"exp_avg": tr(m), "exp_avg_sq": tr(v)}
        return out

    def load_optimizer_state(self, sd: dict) -> None:
        self.t = int(sd["step"])
        names = {"W_E": "W_E", "W_D": "W_D", "b_E": "b_E", "b_D": "b_D", "log_theta": "activation_function.log_jumprelu_threshold"}
        for key, (m, v) in self.state.items():
            if names[key] in sd:
                src_m, src_v = sd[names[key]]["exp_avg"], sd[names[key]]["exp_avg_sq"]
                if self.single and key != "log_theta":
                    src_m, src_v = src_m.unsqueeze(0), src_v.unsqueeze(0)
                if key == "W_E":
                    src_m, src_v = src_m.transpose(1, 2), src_v.transpose(1, 2)
                m.copy_(src_m)
                v.copy_(src_v)
