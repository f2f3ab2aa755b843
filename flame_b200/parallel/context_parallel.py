"""Context parallelism for packed variable-length batches, in two modes.

``document`` (the fallback for rows whose length ``cp`` does not divide).  A packed row of ``seq_len`` tokens is a
concatenation of independent documents, so the row is cut into ``cp`` contiguous pieces at document boundaries (balanced
by token count) and every rank runs its piece: no attention or recurrent state ever has to cross ranks.  Limit: a single
document is never split, so ``context_len`` must not exceed ``seq_len / cp``.

``sequence`` (every model family; what crosses ranks depends on the token mixer).  The row is cut into ``cp`` EQUAL
contiguous slices wherever that falls, also inside a document.  Everything but attention is token-local and runs on
the slice.  In attention the keys and values of the row are all-gathered over the group (the ``allgather`` rotate method
of the reference's flag); a rank then attends its own queries to its own slice extended at the front by the part of its
first document that lies on earlier ranks - an ordinary packed-varlen attention problem whose first document is longer
than the slice's share of it, with zero query rows for the borrowed tokens whose outputs are dropped.  The gradient of
the gathered keys / values is reduce-scattered back to their owners by autograd, so a token's dK / dV collect the
contributions of later ranks' queries.  Rotary positions are the tokens' offsets in their whole document.
The gated-linear-attention families pass their recurrent state instead (``ops/gla.py: gla_state_passing``, the counterpart
of fla's context-parallel kernels, fla/ops/cp/chunk_delta_h.py:42-318): a rank runs its slice from a zero state, computes the decay ``A`` and the
state ``B`` its last document leaves behind, all ranks exchange ``(A, B)`` with one differentiable all-gather, every rank
chains its predecessors' pairs into the state that enters its first document (``S_in[j+1] = A_j S_in[j] + B_j`` while
the document goes on) and adds that state's contribution ``scale (q_t * exp(cumsum g)) S_in`` to the rows of its first
document.  A short convolution in front of the recurrence gets the ``conv_size - 1`` rows before the slice from the
previous rank the same way (``ops/conv.py``).  The (gated) delta rule hands on an affine map too, with a full ``dk x dk``
transition; both halves come out of the ordinary operator through writing and reading tokens
(``ops/delta_rule.py: _delta_rule_state_passing``); gated slot attention passes the states of both of its passes and
Mamba-1's selective scan its per-element state (``ops/scan.py``).  Stick-breaking attention needs every earlier key of
the document, like softmax attention, and borrows the rows of its first document that live on earlier ranks
(``borrow_prefix``).

In both modes parameters are sharded over ``dp_shard x cp`` (the ``dp_shard_cp`` group) exactly as the reference sets it
up (flame/models/parallelize_fla.py:72-88), labels are shifted before the cut so no target is lost at a slice border,
and each rank's loss is re-weighted by its share of the valid targets so the group average equals the global token mean.

The reference wires torch's ring-attention context manager instead (flame/train.py:452-466), which only intercepts
``F.scaled_dot_product_attention`` and therefore does nothing for its flash-attn / linear-attention layers.
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


class _AllGatherRows(torch.autograd.Function):
    """``[rows, ...]`` of every rank -> ``[world * rows, ...]`` in rank order; the backward sums every rank's gradient of
    the gathered tensor and hands each rank the rows it owns (reduce-scatter)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group, ctx.dtype = group, x.dtype
        world = dist.get_world_size(group)
        x = x.contiguous()
        if dist.get_backend(group) == "gloo":
            parts = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(parts, x, group=group)
            return torch.cat(parts, 0)
        out = torch.empty(world * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        group = ctx.group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        dy = dy.contiguous()
        rows = dy.shape[0] // world
        if dist.get_backend(group) == "gloo":
            dy = dy.float() if dy.dtype == torch.bfloat16 else dy.clone()
            dist.all_reduce(dy, group=group)
            return dy[rank * rows:(rank + 1) * rows].to(ctx.dtype), None
        out = torch.empty(rows, *dy.shape[1:], dtype=dy.dtype, device=dy.device)
        dist.reduce_scatter_tensor(out, dy, group=group)
        return out, None


class SequenceSlice:
    """What the token mixers need to know about a rank's slice of a row that was cut inside documents.  ``continues[j]``:
    the first document of rank j's slice began on an earlier rank; ``single[j]``: rank j's slice lies inside one
    document (both for every rank of the group: the recurrent families chain their states through them)."""

    def __init__(self, group, lo: int, hi: int, prefix: int, ext_meta: VarlenMeta, rank: int = 0, world: int = 1,
                 continues=None, single=None, max_prefix: int = -1) -> None:
        self.group, self.lo, self.hi, self.prefix, self.ext_meta = group, lo, hi, prefix, ext_meta
        self.rank, self.world = rank, world
        # the longest prefix any rank borrows (same number on every rank): how many trailing rows a rank has to offer;
        # -1 = unknown, offer everything
        self.max_prefix = max_prefix
        self.continues = list(continues) if continues is not None else [False] * world
        self.single = list(single) if single is not None else [False] * world


def borrow_prefix(tensors, sl: SequenceSlice):
    """Row tensors ``[T / cp, ...]`` of this rank's slice -> the same tensors with the rows of the slice's first document
    that live on earlier ranks put in front (``sl.prefix`` rows; one differentiable all-gather per tensor, so the gradient
    of a borrowed row returns to its owner).  A token mixer that is causal and local to a document can then run on the
    extended rows with ``sl.ext_meta`` and drop the first ``sl.prefix`` rows of its output: it recomputes at most one
    document's prefix per rank, which is what makes this the fallback for every mixer without a cheaper hand-over.
    While no document reaches back further than one slice (``sl.max_prefix <= T / cp``, the usual case: documents are at most
    ``context_len`` long) only the last ``max_prefix`` rows of every rank are gathered, not the whole row."""
    p = sl.prefix
    per = sl.hi - sl.lo
    tail = sl.max_prefix
    out = []
    for t in tensors:
        if t is None:
            out.append(None)
            continue
        if 0 <= tail <= per:
            # no document reaches back further than one slice: every rank offers its last ``tail`` rows only, and the
            # prefix is the end of the previous rank's offer
            if tail == 0:
                out.append(t)
                continue
            tails = _AllGatherRows.apply(t[per - tail:].contiguous(), sl.group)          # [world * tail, ...]
            front = tails[sl.rank * tail - p: sl.rank * tail] if p else tails[:0]
            # every rank takes part in the gather's backward collective, also one that borrows nothing
            out.append(torch.cat([front, t], 0) + tails[:0].sum().to(t.dtype) if not p else torch.cat([front, t], 0))
            continue
        full = _AllGatherRows.apply(t.contiguous(), sl.group)
        out.append(full[sl.lo - p:sl.hi].clone())   # the clone lets the gathered row go before the backward pass
    return out


def sequence_parallel_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sl: SequenceSlice, scale: float,
                                window: int = 0) -> torch.Tensor:
    """Attention of this rank's queries ``[T / cp, H, Dh]`` (rotary embedding already applied to q and k) over the keys of
    their documents, wherever those live: see the module docstring."""
    from ..ops.attention import attention
    p = sl.prefix
    k_ext, v_ext = borrow_prefix([k, v], sl)
    q_ext = torch.cat([q.new_zeros(p, *q.shape[1:]), q], 0) if p else q
    o = attention(q_ext.contiguous(), k_ext.contiguous(), v_ext.contiguous(), sl.ext_meta, scale, window)
    return o[p:]


class ContextParallel:
    def __init__(self, dims: ParallelDims, model, mode: str = "auto") -> None:
        self.dims = dims
        self.group = dims.group("cp")
        self.world = dims.cp
        self.rank = dims.local_rank_in("cp")
        self.model = model
        if mode == "auto":
            cfg = getattr(model, "config", None)
            # softmax attention gathers keys / values; the diagonal-decay recurrences (gated linear attention, HGRN2,
            # Mamba2's SSD) hand their state from rank to rank, a short convolution gets its halo rows from the previous rank;
            # every other family borrows the prefix of its first document (``borrow_prefix``), so all of them are cut into
            # equal slices; ``document`` mode remains for rows whose length the group size does not divide
            mode = "sequence"
        if mode not in ("sequence", "document"):
            raise ValueError(f"unknown context-parallel mode {mode!r}")
        self.mode = mode

    def shard_batch(self, ids: torch.Tensor, labels: torch.Tensor, meta: VarlenMeta) -> Tuple[torch.Tensor, torch.Tensor, VarlenMeta]:
        if self.mode == "sequence" and ids.numel() % self.world == 0:
            return self._slice_sequence(ids, labels, meta)
        return self._cut_at_documents(ids, labels, meta)

    def _loss_weight(self, local_shifted: torch.Tensor) -> float:
        n_local = (local_shifted != -100).sum().float()
        n_all = n_local.clone()
        dist.all_reduce(n_all, group=self.group)
        return (n_local * self.world / n_all.clamp_min(1)).item()

    def _slice_sequence(self, ids, labels, meta):
        cu = meta.cu_cpu().tolist()
        T = ids.numel()
        per = T // self.world
        lo, hi = self.rank * per, (self.rank + 1) * per
        flat_ids, flat_labels = ids.reshape(-1), labels.reshape(-1)
        shifted = torch.cat([flat_labels[1:], torch.full_like(flat_labels[:1], -100)])
        # documents that intersect [lo, hi), clipped to the slice
        inner = [c for c in cu if lo < c < hi]
        local_cu = [0] + [c - lo for c in inner] + [per]
        first_start = max(c for c in cu if c <= lo)          # start of the document the slice begins in
        prefix = lo - first_start                            # its tokens that live on earlier ranks
        local_meta = VarlenMeta.from_cu_seqlens(torch.tensor(local_cu, dtype=torch.int32), per, ids.device)
        # rotary positions count from the start of the WHOLE document
        pos = torch.arange(per, dtype=torch.int32)
        starts = torch.tensor(local_cu[:-1], dtype=torch.int32)
        lens = torch.tensor([b - a for a, b in zip(local_cu[:-1], local_cu[1:])])
        off = torch.repeat_interleave(starts, lens)
        pos = pos - off
        pos[: local_cu[1]] += prefix
        local_meta._pos = pos.to(ids.device)
        local_meta._seq_id = torch.repeat_interleave(torch.arange(len(lens), dtype=torch.int32), lens).to(ids.device)
        ext_cu = [0] + [c + prefix for c in local_cu[1:]]
        ext_meta = VarlenMeta.from_cu_seqlens(torch.tensor(ext_cu, dtype=torch.int32), per + prefix, ids.device)
        bounds = set(cu)
        max_prefix = max(j * per - max(c for c in cu if c <= j * per) for j in range(self.world))
        continues = [(j * per) not in bounds for j in range(self.world)]
        single = [not any(j * per < c < (j + 1) * per for c in cu) for j in range(self.world)]
        local_meta.sequence_slice = SequenceSlice(self.group, lo, hi, prefix, ext_meta, self.rank, self.world, continues,
                                                  single, max_prefix)
        local_meta.labels_preshifted = True
        local_shifted = shifted[lo:hi]
        self.loss_weight = self._loss_weight(local_shifted)
        return flat_ids[lo:hi].unsqueeze(0), local_shifted.unsqueeze(0), local_meta

    def _cut_at_documents(self, ids, labels, meta):
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
        local_meta.labels_preshifted = True   # the model takes the targets as they are: nothing is lost at the cut
        self.loss_weight = self._loss_weight(local_shifted)
        return local_ids, local_shifted.unsqueeze(0), local_meta
