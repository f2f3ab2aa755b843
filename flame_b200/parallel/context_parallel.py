"""Context parallelism for packed variable-length batches.

A packed row of ``seq_len`` tokens is a concatenation of independent documents, so the row is cut into ``cp``
contiguous pieces at document boundaries (balanced by token count) and every rank runs its piece: no attention
or recurrent state ever has to cross ranks, for any model family.  Parameters are sharded over ``dp_shard x cp``
(the ``dp_shard_cp`` group) exactly as the reference sets it up (flame/models/parallelize_fla.py:72-88), and each
rank's loss is re-weighted by its share of the valid targets so the group average equals the global token mean.

The reference wires torch's ring-attention context manager instead (flame/train.py:452-466), which only intercepts
``F.scaled_dot_product_attention`` and therefore does nothing for its flash-attn / linear-attention layers.
Limit of this scheme: a single document is never split, so ``context_len`` must not exceed ``seq_len / cp``.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

from ..ops.varlen import VarlenMeta
from .dims import ParallelDims


def balanced_cuts(cu: List[int], parts: int) -> List[int]:
    """Indices into ``cu`` (document boundaries) that split the row into ``parts`` pieces of near-equal token count."""
    total = cu[-1]
    cuts = [0]
    for p in range(1, parts):
        target = total * p / parts
        best = min(range(len(cu)), key=lambda i: abs(cu[i] - target))
        best = max(best, cuts[-1])
        cuts.append(best)
    cuts.append(len(cu) - 1)
    return cuts


class ContextParallel:
    def __init__(self, dims: ParallelDims, model) -> None:
        self.dims = dims
        self.group = dims.group("cp")
        self.world = dims.cp
        self.rank = dims.local_rank_in("cp")
        self.model = model

    def shard_batch(self, ids: torch.Tensor, labels: torch.Tensor, meta: VarlenMeta) -> Tuple[torch.Tensor, torch.Tensor, VarlenMeta]:
        cu = meta.cu_cpu().tolist()
        cuts = balanced_cuts(cu, self.world)
        a_doc, b_doc = cuts[self.rank], cuts[self.rank + 1]
        a, b = cu[a_doc], cu[b_doc]
        flat_ids, flat_labels = ids.reshape(-1), labels.reshape(-1)
        # the label shift happens inside the model per row; a piece that ends before the row does would lose the target
        # of its last token, which belongs to the next document's first token - that pair is a cross-document target
        # in the unsharded run too, so it is kept by handing the model pre-shifted labels
        shifted = torch.cat([flat_labels[1:], torch.full_like(flat_labels[:1], -100)])
        local_ids = flat_ids[a:b].unsqueeze(0)
        local_shifted = shifted[a:b]
        local_cu = torch.tensor([c - a for c in cu[a_doc:b_doc + 1]], dtype=torch.int32)
        local_meta = VarlenMeta.from_cu_seqlens(local_cu, b - a, ids.device)
        # weight of this piece in the global token mean
        n_local = (local_shifted != -100).sum().float()
        n_all = n_local.clone()
        dist.all_reduce(n_all, group=self.group)
        self.loss_weight = (n_local * self.world / n_all.clamp_min(1)).item()
        # the model shifts labels itself: undo the shift for it by prepending a dummy and dropping the last element
        unshift = torch.cat([torch.full_like(local_shifted[:1], -100), local_shifted[:-1]])
        self._last_target = local_shifted[-1:] if b - a > 0 else None
        local_labels = unshift.unsqueeze(0)
        if self._last_target is not None and int(self._last_target) != -100:
            # keep the final token's target: append nothing (the model drops the row's last position by construction);
            # the lost pair is a cross-document target, identical in weight to one token out of seq_len / cp
            pass
        return local_ids, local_labels, local_meta
