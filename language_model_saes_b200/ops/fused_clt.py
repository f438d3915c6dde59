"""One training step of a cross-layer transcoder with a per-layer TopK activation as a fixed sequence of sm_100a kernels,
without autograd.

What it computes is the reference's step for a ``CrossLayerTranscoder`` (models/clt.py:526-573 encode, :629-709 decode of
every source layer into every later target layer, :836-876 per-feature decoder norms, MSE averaged over layers and
tokens) with Adam. How it computes it:

1. per source layer: encoder GEMM (tcgen05) with the fused top-k epilogue, gated by the feature's decoder norm over all its
   target layers, and the merge of the candidate lists (+ one all-gather of the lists between feature shards)
                                                                  -> codes (layer * F + feature, act) [B, L * k]
2. decoder fan-out: ONE gather kernel adds every active feature's rows into all its target layers (``clt_decode``); the
   dense [B, L, F] activations and the 78 per-pair products never exist. Feature shards sum their partial outputs with the
   one-kernel in-place all-reduce over peer memory (``parallel.symm.AllReduceComm``: one reduce of [L, B, d] instead of
   one collective per target layer)
3. loss and d y in one kernel, d act in one kernel (``clt_dact``), counting sort of the codes by (layer, feature)
4. updates: per TARGET layer t one launch of the sparse gradient + Adam kernel over ``W_D[t]`` seen as a
   ``[(t + 1) F, d]`` matrix (decoder side only: gradient rows rebuilt from the by-feature lists and d y[t], Adam, bf16
   shadow, squared row norms accumulated into the per-feature norm over target layers); per SOURCE layer one launch over
   ``W_E[s]`` (encoder side only). No dense gradient tensor exists; the reference materialises one per decoder.

Restrictions: ``topk`` activation with k <= 64, no sparsity loss, Adam, fp32 parameters with bf16 compute. Features may
be sharded over ``model`` and tokens split over ``data`` (replicas gather each other's codes, output gradients and inputs
and rebuild the same sparse rows).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..parallel.mesh import mesh_dim_size, mesh_group, mesh_local_rank
from . import clt_kernels as CK
from . import sae_kernels as K


def LAYERTOPK_ON_FUSED_PATH() -> bool:
    """``layertopk`` on the fused step is verified against autograd on the CPU and composed of kernels that have GPU tests of
    their own, but the composition has not run on a GPU: the trainer takes it only on request."""
    return "1" in (os.environ.get("LMSAE_FUSED_LAYERTOPK", "0"), os.environ.get("LMSAE_FUSED_CPU_VERIFIED", "0"))


class FusedCLTStep:
    def __init__(self, clt, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8):
        cfg = clt.cfg
        self.clt = clt
        self.betas, self.eps = betas, eps
        self.tp = mesh_dim_size(clt.device_mesh, "model")
        self.tp_rank = mesh_local_rank(clt.device_mesh, "model")
        self.tp_group = mesh_group(clt.device_mesh, "model")
        self.dp = mesh_dim_size(clt.device_mesh, "data")
        self.dp_group = mesh_group(clt.device_mesh, "data")
        self.L, self.F, self.d = cfg.n_layers, clt.d_sae_local, cfg.d_model
        self.use_gate = cfg.sparsity_include_decoder_norm
        self.joint = cfg.act_fn == "layertopk"  # k codes per token over all layers together, instead of k per layer
        self.batch_level = cfg.act_fn in ("batchtopk", "batchlayertopk")  # k x batch codes per layer / over all layers
        self.batch_all_layers = cfg.act_fn == "batchlayertopk"
        self.batch_list_factor = int(os.environ.get("LMSAE_BATCH_LIST_FACTOR", "8"))
        self.list_overflow = torch.zeros(1, dtype=torch.int64, device=clt.b_E.device)
        L, F, d = self.L, self.F, self.d
        self.WE = clt.W_E.data.transpose(1, 2)  # [L, F, d] contiguous view of the parameter's storage
        assert self.WE.is_contiguous() and self.WE.dtype == torch.float32
        self.bE = clt.b_E.data
        self.WD = [w.data.view((t + 1) * F, d) for t, w in enumerate(clt.W_D)]
        dev = self.WE.device
        # the decoder biases as rows of one matrix (one update launch): the parameters become views of it
        self.bD = torch.stack([b.data for b in clt.b_D]).contiguous()
        for t, b in enumerate(clt.b_D):
            b.data = self.bD[t]
        z = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)  # noqa: E731
        self.WE_bf16 = torch.empty(L, F, d, dtype=torch.bfloat16, device=dev)
        self.WD_bf16 = [torch.empty(t + 1, F, d, dtype=torch.bfloat16, device=dev) for t in range(L)]
        self.norm_sq = z(L * F)  # per (source layer, feature): squared decoder norm over all its target layers
        self.state = {"W_E": (z(L, F, d), z(L, F, d)), "b_E": (z(L, F), z(L, F)), "b_D": (z(L, d), z(L, d)),
                      "W_D": [(z((t + 1) * F, d), z((t + 1) * F, d)) for t in range(L)]}  # fmt: skip
        self.groups: K.FeatureGroups | None = None
        self.loss_sum = z(1)
        self.comm = None
        self.own_rows = (0, F)
        self.t = 0
        self.refresh()

    @staticmethod
    def supports(clt, trainer_cfg=None) -> tuple[bool, str]:
        from ..models.clt import CrossLayerTranscoder

        cfg = clt.cfg
        if type(clt) is not CrossLayerTranscoder:
            return False, "model is not a CrossLayerTranscoder"
        checks = [
            (cfg.act_fn == "topk" or (cfg.act_fn in ("layertopk", "batchtopk", "batchlayertopk") and LAYERTOPK_ON_FUSED_PATH()),
             "activation is not the per-layer topk (layertopk / batchtopk / batchlayertopk: set LMSAE_FUSED_LAYERTOPK=1)"),
            (cfg.top_k <= {"topk": 64, "layertopk": 512}.get(cfg.act_fn, 96), "k above the list width of the step"),
            # batch-level selections: lists of 8 k codes per layer (or in all); the decode kernel stages a row's codes on chip
            (cfg.act_fn not in ("batchtopk", "batchlayertopk")
             or (cfg.n_layers if cfg.act_fn == "batchtopk" else 1) * (-(-int(os.environ.get("LMSAE_BATCH_LIST_FACTOR", "8")) * cfg.top_k // 8) * 8) <= 6144,
             "code lists of a token longer than 6144 entries"),
            (clt.b_E.is_cuda or trainer_cfg is None, "not on a CUDA device"),
            (cfg.dtype == torch.float32, "parameters are not fp32"),
            (cfg.d_model % 8 == 0 and clt.d_sae_local % 8 == 0, "d_model / local d_sae not multiples of 8"),
            (not any(hp.fwd_hooks or hp.bwd_hooks for hp in clt.hook_points()), "hooks are attached"),
        ]
        if trainer_cfg is not None:
            checks += [
                (trainer_cfg.sparsity_loss_type is None, "sparsity loss"),
                (trainer_cfg.optimizer_class == "adam", "optimizer is not adam"),
                (trainer_cfg.amp_dtype == torch.bfloat16, "amp dtype is not bf16"),
                (trainer_cfg.gradient_accumulation_steps == 1, "gradient accumulation"),
                (not trainer_cfg.clip_grad_norm, "gradient clipping"),
                (not trainer_cfg.initial_k or trainer_cfg.initial_k <= {"topk": 64, "layertopk": 512}.get(cfg.act_fn, 96),
                 "k schedule starting above the list width"),
            ]
        for ok, why in checks:
            if not ok:
                return False, why
        return True, ""

    def refresh(self) -> None:
        """Re-derive bf16 shadows and the per-feature decoder norms from the fp32 masters."""
        self.norm_sq.zero_()
        for t in range(self.L):
            n = torch.empty((t + 1) * self.F, dtype=torch.float32, device=self.WE.device)
            K.row_norm_shadow(self.WD[t], n, self.WD_bf16[t].view((t + 1) * self.F, self.d))
            self.norm_sq[: (t + 1) * self.F] += n.square()
        K.row_norm_shadow(self.WE.view(self.L * self.F, self.d), None, self.WE_bf16.view(self.L * self.F, self.d))

    def join(self) -> None:
        pass

    def sync_params(self) -> None:
        pass

    def encode(self, x: torch.Tensor, k: int, xt: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """``x [B, L, d]`` bf16 -> codes ``(idx = layer * F + feature, act) [B, L * k]`` over this rank's features.
        ``xt``: the same activations layer-major ``[L, B, d]`` when the caller already has them."""
        B, L, F = x.shape[0], self.L, self.F
        gate_all = self.norm_sq.sqrt().view(L, F) if self.use_gate else None
        if xt is None:
            xt = x.transpose(0, 1).contiguous()  # one copy instead of one per layer
        if self.joint:
            return self._encode_joint(xt, k, gate_all)
        if self.batch_level:
            return self._encode_batch_level(xt, k, gate_all)
        idxs, acts = [], []
        if self.tp == 1:
            for layer in range(L):
                gate = gate_all[layer] if gate_all is not None else None
                i, a = K.encoder_topk(xt[layer], self.WE_bf16[layer], self.bE[layer], gate, k)
                idxs.append(i)
                acts.append(a)
        else:
            # feature shards: every layer's local top-k list first, then ONE all-gather of all layers' lists, then the merges
            loc_g = torch.empty(L, B, k, dtype=torch.float32, device=x.device)
            loc_i = torch.empty(L, B, k, dtype=torch.int32, device=x.device)
            for layer in range(L):
                gate = gate_all[layer] if gate_all is not None else None
                if x.is_cuda:
                    cv, ci, _ = K.encoder_topk_candidates(xt[layer], self.WE_bf16[layer], self.bE[layer], gate, k)
                    i_l, g_l = K.topk_merge(cv, ci, k, gate, emit_gated=True)
                else:
                    i_l, a_l = K.encoder_topk(xt[layer], self.WE_bf16[layer], self.bE[layer], gate, k)
                    g_l = a_l * gate[i_l.clamp_min(0).long()] if gate is not None else a_l
                loc_g[layer], loc_i[layer] = g_l, i_l
            all_g = torch.empty(self.tp, L, B, k, dtype=torch.float32, device=x.device)
            all_i = torch.empty(self.tp, L, B, k, dtype=torch.int32, device=x.device)
            dist.all_gather_into_tensor(all_g.view(self.tp * L, B, k), loc_g, group=self.tp_group)
            dist.all_gather_into_tensor(all_i.view(self.tp * L, B, k), loc_i, group=self.tp_group)
            all_g = all_g.permute(1, 2, 0, 3).reshape(L, B, self.tp * k).contiguous()
            all_i = all_i.permute(1, 2, 0, 3).reshape(L, B, self.tp * k).contiguous()
            for layer in range(L):
                gate = gate_all[layer] if gate_all is not None else None
                i, a = K.topk_merge(all_g[layer], all_i[layer], k, gate, own=(self.tp_rank * k, (self.tp_rank + 1) * k))
                idxs.append(i)
                acts.append(a)
        # layer * F is added to all lists at once (empty slots stay -1)
        idx = torch.stack(idxs, dim=1)  # [B, L, k]
        offset = (torch.arange(L, device=x.device, dtype=idx.dtype) * F).view(1, L, 1)
        idx = torch.where(idx >= 0, idx + offset, idx).view(B, L * k)
        return idx, torch.stack(acts, dim=1).view(B, L * k)

    def _encode_joint(self, xt: torch.Tensor, k: int, gate_all: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:
        """``layertopk``: the k largest gated pre-activations of a token over ALL (layer, feature) pairs (models/clt.py
        :298-304 of the reference project). Any of them is among the k largest of its own layer, so every layer contributes
        its own top-k list (GEMM with the fused epilogue up to k = 64, pre-activations + radix row top-k above) and the k
        best of the ``L k`` candidates are kept; feature shards then exchange their lists as the SAE step does."""
        L, F, B = self.L, self.F, xt.shape[1]
        kk = min(k, F)
        idxs, acts, gated = [], [], []
        for layer in range(L):
            gate = gate_all[layer] if gate_all is not None else None
            i, a = K.encoder_topk(xt[layer], self.WE_bf16[layer], self.bE[layer], gate, kk)
            idxs.append(torch.where(i >= 0, i + layer * F, i))
            acts.append(a)
            gated.append(a * gate[i.clamp_min(0).long()] if gate is not None else a)
        idx, act, g = torch.cat(idxs, dim=1), torch.cat(acts, dim=1), torch.cat(gated, dim=1)  # [B, L kk]
        g = torch.where(idx >= 0, g, torch.full_like(g, float("-inf")))
        top_g, pos = g.topk(min(k, g.shape[1]), dim=1)
        idx, act = torch.gather(idx, 1, pos), torch.gather(act, 1, pos)
        keep = (top_g > 0) & (idx >= 0)  # only positive gated pre-activations fire
        idx, act, top_g = torch.where(keep, idx, torch.full_like(idx, -1)), torch.where(keep, act, torch.zeros_like(act)), top_g.clamp_min(0)
        if idx.shape[1] < k:  # fewer candidates than k: pad the lists
            pad = k - idx.shape[1]
            idx = torch.nn.functional.pad(idx, (0, pad), value=-1)
            act, top_g = torch.nn.functional.pad(act, (0, pad)), torch.nn.functional.pad(top_g, (0, pad))
        if self.tp == 1:
            return idx.contiguous(), act.contiguous()
        # feature shards: every shard's k best (gated values and local indices) to all, the k best of tp k kept, own slots only
        all_g = torch.empty(self.tp * B, k, dtype=torch.float32, device=idx.device)
        all_i = torch.empty(self.tp * B, k, dtype=torch.int32, device=idx.device)
        dist.all_gather_into_tensor(all_g, top_g.float().contiguous(), group=self.tp_group)
        dist.all_gather_into_tensor(all_i, idx.to(torch.int32).contiguous(), group=self.tp_group)
        all_g = all_g.view(self.tp, B, k).permute(1, 0, 2).reshape(B, self.tp * k)
        all_i = all_i.view(self.tp, B, k).permute(1, 0, 2).reshape(B, self.tp * k)
        all_g = torch.where(all_i >= 0, all_g, torch.full_like(all_g, float("-inf")))
        _, pos = all_g.topk(k, dim=1)
        mine = (pos >= self.tp_rank * k) & (pos < (self.tp_rank + 1) * k) & (torch.gather(all_g, 1, pos) > 0)
        chosen = torch.zeros(B, self.tp * k + 1, dtype=torch.bool, device=idx.device)
        chosen.scatter_(1, torch.where(mine, pos, torch.full_like(pos, self.tp * k)), True)
        own = chosen[:, self.tp_rank * k : (self.tp_rank + 1) * k]
        return torch.where(own, idx, torch.full_like(idx, -1)).contiguous(), torch.where(own, act, torch.zeros_like(act)).contiguous()

    def _encode_batch_level(self, xt: torch.Tensor, k: int, gate_all: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:
        """``batchtopk``: per layer the ``k x batch`` largest gated pre-activations of the whole batch (over all feature
        shards); ``batchlayertopk``: the ``k x batch`` largest over all layers together (models/clt.py:330-368 of the
        reference project). As in the SAE step: gated pre-activations in bf16, a radix select of the threshold (shards add
        their histograms), one compaction pass into lists of fixed width (``LMSAE_BATCH_LIST_FACTOR`` x k per layer;
        rows with more codes are counted in ``list_overflow``), nothing read back by the host."""
        from . import select_kernels as S

        L, F, B = self.L, self.F, xt.shape[1]
        tp_group = self.tp_group if self.tp > 1 else None
        G = [K.encoder_hidden(xt[layer], self.WE_bf16[layer], self.bE[layer], gate=gate_all[layer] if gate_all is not None else None)
             for layer in range(L)]  # fmt: skip
        if self.batch_all_layers:  # one threshold for everything
            thr, ties = S.positive_thresholds(torch.stack(G, dim=1).view(1, 1, -1), k * B, tp_group, return_remaining=True)
            cap = -(-self.batch_list_factor * k // 8) * 8
            flat = torch.cat(G, dim=1)  # [B, L F]: column = layer * F + feature, the codes' index space
            div = gate_all.reshape(-1) if gate_all is not None else None
            return S.threshold_rows_to_sparse(flat, thr, div, n_ties=ties, tie_group=tp_group, cap=cap, overflow=self.list_overflow)
        cap = -(-self.batch_list_factor * k // 8) * 8
        idxs, acts = [], []
        for layer in range(L):
            thr, ties = S.positive_thresholds(G[layer].view(1, 1, -1), k * B, tp_group, return_remaining=True)
            gate = gate_all[layer] if gate_all is not None else None
            i, a = S.threshold_rows_to_sparse(G[layer], thr, gate, n_ties=ties, tie_group=tp_group, cap=cap, overflow=self.list_overflow)
            idxs.append(torch.where(i >= 0, i + layer * F, i))
            acts.append(a)
        return torch.cat(idxs, dim=1).contiguous(), torch.cat(acts, dim=1).contiguous()

    def _decode(self, idx: torch.Tensor, act: torch.Tensor) -> torch.Tensor:
        """Reconstruction ``[L, B, d]`` fp32 (summed over feature shards, decoder biases added)."""
        B, L, d = idx.shape[0], self.L, self.d
        if self.tp == 1:
            return CK.clt_decode(idx, act, self.WD_bf16, self.bD, torch.float32)
        if not idx.is_cuda:
            y = CK.clt_decode(idx, act, self.WD_bf16, None, torch.float32)
            dist.all_reduce(y, group=self.tp_group)
            return y + self.bD[:, None, :]
        from ..parallel.symm import AllReduceComm

        if self.comm is None or self.comm.max_rows < L * B:
            self.comm = AllReduceComm(self.tp_group, idx.device, L * B, d)
        part = self.comm.matrix(L * B).view(L, B, d)
        K._ext().clt_decode(idx, act, list(self.WD_bf16), None, part)  # bf16 partial rows straight into the symmetric buffer
        return self.comm.all_reduce(L * B).view(L, B, d).float() + self.bD[:, None, :]

    def step(self, x: torch.Tensor, label: torch.Tensor, k: int, lr: float, xt: torch.Tensor | None = None) -> torch.Tensor:
        """``x [B, L, d]`` normalised bf16 inputs of the L source layers (any strides when ``xt``, the same activations as a
        contiguous ``[L, B, d]``, comes with it), ``label [L, B, d]`` bf16 targets. Returns the mean loss (0-d device
        tensor)."""
        B, L, F, d = x.shape[0], self.L, self.F, self.d
        if xt is None:
            xt = x.transpose(0, 1).contiguous()  # [L, B, d]: the layers' rows for the encoder GEMMs and the encoder-side update
        idx, act = self.encode(x, k, xt)
        y = self._decode(idx, act)
        self.loss_sum.zero_()
        n_rows = L * B * self.dp  # (layer, token) pairs of the whole step: every replica brings B tokens
        dy = K.mse_loss_grad(y.view(L * B, d), label.reshape(L * B, d).contiguous(), None, None, 2.0 / n_rows, self.loss_sum)
        dy = dy.view(L, B, d)
        dact = CK.clt_dact(idx, self.WD_bf16, dy)
        if self.dp > 1:
            # Replicas: codes, their gradients, the output gradients and the inputs of every replica are gathered (rows in rank
            # order) and each replica rebuilds the same sparse rows of W_D and W_E from them: the same update everywhere, no
            # dense gradient of the 78 decoder matrices to sum.
            idx, act, dact = (self._gather_rows(t) for t in (idx, act, dact))
            dy, xt = self._gather_layer_rows(dy), self._gather_layer_rows(xt)
            dist.all_reduce(self.loss_sum, group=self.dp_group)
        if self.groups is None or self.groups.entries.numel() < idx.numel():
            self.groups = K.FeatureGroups(L * F, idx.numel(), x.device)
        self.groups.build(idx)
        off, ent = self.groups.offsets, self.groups.entries
        self.t += 1
        b1, b2 = self.betas
        self.norm_sq.zero_()
        g = K.FeatureGroups.__new__(K.FeatureGroups)
        g.entries = ent
        for t in range(L):  # decoder side, one launch per target layer
            rows = (t + 1) * F
            g.F, g.offsets = rows, off[: rows + 1]
            mD, vD = self.state["W_D"][t]
            K.sparse_grad_adam(g, act, dact, dy[t], dy[t], self.WD[t], mD, vD, self.WD_bf16[t].view(rows, d), None, None, None, None, None,
                               None, None, None, None, None, lr, b1, b2, self.eps, self.t, True, norm_sq_accum=self.norm_sq[:rows])  # fmt: skip
        (mE, vE), (mb, vb) = self.state["W_E"], self.state["b_E"]
        for s in range(L):  # encoder side, one launch per source layer
            g.F, g.offsets = F, off[s * F : (s + 1) * F + 1]
            xs = xt[s]
            K.sparse_grad_adam(g, act, dact, xs, xs, None, None, None, None, self.WE[s], mE[s], vE[s], self.WE_bf16[s], self.bE[s], mb[s],
                               vb[s], None, None, None, lr, b1, b2, self.eps, self.t, True)  # fmt: skip
        m, v = self.state["b_D"]
        K.adam_flat(self.bD.view(-1), dy.float().sum(dim=1).reshape(-1), m.view(-1), v.view(-1), lr, b1, b2, self.eps, self.t)
        return (self.loss_sum / n_rows).squeeze(0)

    def _gather_rows(self, t: torch.Tensor) -> torch.Tensor:
        """``[rows, n]`` of every replica stacked in rank order."""
        t = t.contiguous()
        out = torch.empty(self.dp * t.shape[0], *t.shape[1:], dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=self.dp_group)
        return out

    def _gather_layer_rows(self, t: torch.Tensor) -> torch.Tensor:
        """``[L, rows, d]`` of every replica -> ``[L, replicas x rows, d]`` with each layer's rows in rank order."""
        L, B, d = t.shape
        out = torch.empty(self.dp, L, B, d, dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out.view(self.dp * L, B, d), t.contiguous(), group=self.dp_group)
        return out.permute(1, 0, 2, 3).reshape(L, self.dp * B, d)

    def optimizer_state(self) -> dict:
        out = {"step": self.t, "W_E": {"exp_avg": self.state["W_E"][0].transpose(1, 2), "exp_avg_sq": self.state["W_E"][1].transpose(1, 2)},
               "b_E": {"exp_avg": self.state["b_E"][0], "exp_avg_sq": self.state["b_E"][1]}}  # fmt: skip
        for t in range(self.L):
            m, v = self.state["W_D"][t]
            out[f"W_D.{t}"] = {"exp_avg": m.view(t + 1, self.F, self.d), "exp_avg_sq": v.view(t + 1, self.F, self.d)}
            out[f"b_D.{t}"] = {"exp_avg": self.state["b_D"][0][t], "exp_avg_sq": self.state["b_D"][1][t]}
        return out

    def load_optimizer_state(self, sd: dict) -> None:
        self.t = int(sd["step"])
        if "W_E" in sd:
            self.state["W_E"][0].copy_(sd["W_E"]["exp_avg"].transpose(1, 2))
            self.state["W_E"][1].copy_(sd["W_E"]["exp_avg_sq"].transpose(1, 2))
        if "b_E" in sd:
            self.state["b_E"][0].copy_(sd["b_E"]["exp_avg"])
            self.state["b_E"][1].copy_(sd["b_E"]["exp_avg_sq"])
        for t in range(self.L):
            if f"W_D.{t}" in sd:
                self.state["W_D"][t][0].copy_(sd[f"W_D.{t}"]["exp_avg"].reshape((t + 1) * self.F, self.d))
                self.state["W_D"][t][1].copy_(sd[f"W_D.{t}"]["exp_avg_sq"].reshape((t + 1) * self.F, self.d))
            if f"b_D.{t}" in sd:
                self.state["b_D"][0][t].copy_(sd[f"b_D.{t}"]["exp_avg"])
                self.state["b_D"][1][t].copy_(sd[f"b_D.{t}"]["exp_avg_sq"])
