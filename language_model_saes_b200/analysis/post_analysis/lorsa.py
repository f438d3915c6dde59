"""Attention dictionaries add, for every kept sample of every head, its "z pattern": how much each source position
contributes to the head's activation at each target position, stored sparsely as (sample, query, key) -> value
(analysis/post_analysis/lorsa.py:46-229 of the reference project).

The patterns are not kept while streaming (they are ``ctx x ctx`` per head and sample); instead the stream is replayed
and only contexts that were selected are re-encoded. Selected (shard, context) pairs are hashed into one int64 key and
looked up with ``searchsorted``, and the per-feature split of the result is one stable sort, so the cost is linear in
the number of non-zeros instead of (features x non-zeros).
"""

from __future__ import annotations

import numpy as np
import torch
from tqdm import tqdm

from ...models.lorsa import LowRankSparseAttention
from ...parallel.mesh import is_primary_rank
from .base import PostAnalysisProcessor, register_post_analysis_processor

_SHIFT = 1 << 40  # contexts per shard stay far below this


class LorsaPostAnalysisProcessor(PostAnalysisProcessor):
    rel_threshold: float = 1e-2
    """Contributions below this fraction of the head's activation at the target position are dropped."""

    def _process_tensors(self, sae, act_times, n_analyzed_tokens, max_feature_acts, sample_result, mapper, device_mesh=None,
                         activation_factory=None, activation_factory_process_kwargs=None, clt_layer=None):  # fmt: skip
        assert isinstance(sae, LowRankSparseAttention)
        assert activation_factory is not None, "the activation stream is replayed to compute z patterns"
        dev = act_times.device
        names = [n for n, v in sample_result.items() if v is not None]
        # flat list of (sampling, sample slot, head) entries with the context they came from
        keys, heads, slots, owners, acts = [], [], [], [], []
        for si, name in enumerate(names):
            sub = sample_result[name]
            n, f, _ = sub["feature_acts"].shape
            shard = sub["shard_idx"].long() if "shard_idx" in sub else torch.zeros(n, f, dtype=torch.long, device=dev)
            keys.append((shard * _SHIFT + sub["context_idx"].long()).flatten())
            heads.append(torch.arange(f, device=dev).expand(n, f).flatten())
            slots.append(torch.arange(n, device=dev)[:, None].expand(n, f).flatten())
            owners.append(torch.full((n * f,), si, device=dev))
            acts.append(sub["feature_acts"].flatten(0, 1))
        keys, heads, slots, owners, acts = (torch.cat(t) for t in (keys, heads, slots, owners, acts))
        alive = act_times.ne(0)[heads] & (acts != 0).any(dim=-1)
        order = torch.argsort(keys, stable=True)
        sorted_keys = keys[order]
        remaining = {int(k) for k in torch.unique(keys[alive]).tolist()}

        out_entry, out_q, out_k, out_v = [], [], [], []
        bar = tqdm(total=len(remaining), desc="Processing Lorsa z patterns", disable=not is_primary_rank(device_mesh))
        for batch in activation_factory.process(**(activation_factory_process_kwargs or {})):
            if not remaining:
                break
            x_all = batch[sae.cfg.hook_point_in]
            for i, m in enumerate(batch["meta"]):
                key = int(m.get("shard_idx", 0)) * _SHIFT + int(m["context_idx"])
                if key not in remaining:
                    continue
                remaining.discard(key)
                bar.update(1)
                lo = int(torch.searchsorted(sorted_keys, key))
                hi = int(torch.searchsorted(sorted_keys, key, right=True))
                entries = order[lo:hi]
                entries = entries[alive[entries]]
                if entries.numel() == 0:
                    continue
                a = acts[entries].float()  # [e, ctx]
                z = sae.encode_z_pattern_for_head(x_all[i : i + 1].to(dev), heads[entries]).float()  # [e, q, k]
                z = z * a.ne(0)[..., None]
                z = z.masked_fill(z.abs() < self.rel_threshold * a[..., None], 0.0)
                e, q, k = z.nonzero(as_tuple=True)
                out_entry.append(entries[e]), out_q.append(q), out_k.append(k), out_v.append(z[e, q, k])
        bar.close()

        cat = lambda ts, dt: torch.cat(ts) if ts else torch.empty(0, dtype=dt, device=dev)  # noqa: E731
        entry, q, k, v = cat(out_entry, torch.long), cat(out_q, torch.long), cat(out_k, torch.long), cat(out_v, torch.float32)
        # group non-zeros by (sampling, head), keeping (sample, q, k) order inside a group
        group = owners[entry] * act_times.numel() + heads[entry]
        inner = (slots[entry] * acts.shape[-1] + q) * acts.shape[-1] + k
        perm = torch.argsort(inner, stable=True)
        perm = perm[torch.argsort(group[perm], stable=True)]
        group, slot_s, q, k, v = group[perm].cpu().numpy(), slots[entry][perm].cpu().numpy(), q[perm].cpu().numpy(), k[perm].cpu().numpy(), v[perm].cpu().numpy()
        f = act_times.numel()
        bounds = np.searchsorted(group, np.arange(len(names) * f + 1))
        for si, name in enumerate(names):
            idx_list, val_list = [], []
            for h in range(f):
                a, b = bounds[si * f + h], bounds[si * f + h + 1]
                idx_list.append(np.stack([slot_s[a:b], q[a:b], k[a:b]]))
                val_list.append(v[a:b].astype(np.float32))
            sample_result[name] = {**sample_result[name], "z_pattern_indices": idx_list, "z_pattern_values": val_list}
        return sample_result, None

    def _extra_info(self, sampling_data, i):
        return {
            **super()._extra_info(sampling_data, i),
            "z_pattern_indices": sampling_data["z_pattern_indices"][i],
            "z_pattern_values": sampling_data["z_pattern_values"][i],
        }


register_post_analysis_processor("lorsa", LorsaPostAnalysisProcessor)
