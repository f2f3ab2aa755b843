"""Pipeline parallelism: layer ranges per stage, micro-batching of packed rows, GPipe and 1F1B schedules over
point-to-point sends (NCCL on GPUs, gloo on CPUs).

The reference ships a manual stage splitter (flame/models/pipeline_fla.py:28-162) but its trainer refuses to run with
``pipeline_parallel_degree > 1`` (flame/train.py:123-126); here the path is live.  Stage ``s`` of ``S`` keeps a
contiguous range of decoder blocks; the first stage owns the embeddings, the last the final norm and the head.
``pipeline_parallel_split_points`` (names like ``layers.12``) overrides the even split.  A stage boundary carries one
``[tokens, hidden]`` tensor (the residual stream); gradients travel the other way.

Micro-batches: a batch with several rows is split by rows; a single packed varlen row is split at document
boundaries, which is exact because documents are independent.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..components.metrics import logger
from ..ops.varlen import VarlenMeta
from .context_parallel import balanced_cuts
from .dims import ParallelDims


def stage_layer_ranges(num_layers: int, stages: int, split_points: Optional[List[str]] = None) -> List[Tuple[int, int]]:
    if split_points:
        starts = [0] + [int(s.split(".")[-1]) for s in split_points]
        if len(starts) != stages:
            raise ValueError(f"{len(split_points)} split points give {len(starts)} stages, expected {stages}")
        bounds = starts + [num_layers]
    else:
        base, extra = divmod(num_layers, stages)
        bounds = [0]
        for s in range(stages):
            bounds.append(bounds[-1] + base + (1 if s < extra else 0))
    return [(bounds[i], bounds[i + 1]) for i in range(stages)]


def split_into_stage(model, model_config, dims: ParallelDims, job_config) -> Tuple[int, int]:
    """Keeps only this pipeline rank's part of the (meta-device) model; returns its layer range."""
    S, s = dims.pp, dims.local_rank_in("pp")
    pts = list(job_config.experimental.pipeline_parallel_split_points) if job_config is not None else []
    lo, hi = stage_layer_ranges(model_config.num_hidden_layers, S, pts)[s]
    dec = model.decoder
    for i in range(len(dec.layers)):
        if not (lo <= i < hi):
            dec.layers[i] = None
    if s != 0:
        dec.embeddings = None
    if s != S - 1:
        for name in ("norm", "norm_f"):
            if hasattr(dec, name):
                setattr(dec, name, None)
        model.lm_head = None
    if hasattr(dec, "lower_bounds") and s != 0:
        pass  # every stage keeps the (tiny) HGRN2 lower-bound table it needs for its own layers
    model.pp_stage, model.pp_stages = s, S
    logger.info(f"pipeline stage {s}/{S}: layers [{lo}, {hi})")
    return lo, hi


class PipelineRunner:
    def __init__(self, model, engine, dims: ParallelDims, device: torch.device, job_config) -> None:
        self.model, self.engine, self.dims, self.device = model, engine, dims, device
        self.group = dims.group("pp")
        self.ranks = dims.group_ranks("pp")
        self.S = dims.pp
        self.s = dims.local_rank_in("pp")
        self.first, self.last = self.s == 0, self.s == self.S - 1
        ex = job_config.experimental
        self.n_mb = ex.pipeline_parallel_microbatches or self.S
        name = (ex.pipeline_parallel_schedule or "1F1B").lower()
        if name not in ("1f1b", "gpipe"):
            logger.warning(f"pipeline schedule {ex.pipeline_parallel_schedule!r} is not implemented; using 1F1B")
            name = "1f1b"
        self.schedule = name
        self.hidden = model.config.hidden_size
        self.dtype = engine.param_dtype

    # ---- micro-batching ---------------------------------------------------------------------------------------
    def _microbatches(self, batch: Dict[str, torch.Tensor]):
        ids, labels = batch["input_ids"], batch["labels"]
        cu = batch.get("cu_seqlens")
        B, Slen = ids.shape
        out = []
        if cu is None:
            n = min(self.n_mb, B)
            for rows in torch.arange(B).chunk(n):
                out.append((ids[rows], labels[rows], None))
            return out
        cu_list = cu.reshape(-1).tolist()
        n = max(1, min(self.n_mb, len(cu_list) - 1))
        cuts = balanced_cuts(cu_list, n)
        flat_ids, flat_labels = ids.reshape(-1), labels.reshape(-1)
        shifted = torch.cat([flat_labels[1:], torch.full_like(flat_labels[:1], -100)])
        for m in range(n):
            a_doc, b_doc = cuts[m], cuts[m + 1]
            a, b = cu_list[a_doc], cu_list[b_doc]
            if b <= a:
                continue
            lab = torch.cat([torch.full_like(shifted[:1], -100), shifted[a:b - 1]])  # model re-shifts by one
            out.append((flat_ids[a:b].unsqueeze(0), lab.unsqueeze(0),
                        torch.tensor([c - a for c in cu_list[a_doc:b_doc + 1]], dtype=torch.int32)))
        return out

    # ---- p2p ----------------------------------------------------------------------------------------------------
    def _send(self, t: torch.Tensor, to_stage: int):
        return dist.isend(t.contiguous(), dst=self.ranks[to_stage], group=self.group)

    def _recv(self, tokens: int, from_stage: int):
        buf = torch.empty(tokens, self.hidden, dtype=self.dtype, device=self.device)
        return buf, dist.irecv(buf, src=self.ranks[from_stage], group=self.group)

    # ---- one optimizer step's worth of micro-batches -----------------------------------------------------------------
    def forward_backward(self, batch: Dict[str, torch.Tensor], loss_scale: float = 1.0) -> Optional[torch.Tensor]:
        mbs = self._microbatches(batch)
        n = len(mbs)
        total_valid = sum(int((lab[:, 1:] != -100).sum()) for _, lab, _ in mbs)
        fwd_state: List[Optional[tuple]] = [None] * n
        losses = []
        pending = []

        def forward(i: int):
            ids, labels, cu = mbs[i]
            tokens = ids.numel()
            ids_d = ids.to(self.device, non_blocking=True)
            meta = (VarlenMeta.from_cu_seqlens(cu, tokens, self.device) if cu is not None
                    else VarlenMeta.dense(ids.shape[0], ids.shape[1], self.device))
            x_in = None
            if not self.first:
                buf, req = self._recv(tokens, self.s - 1)
                req.wait()
                x_in = buf.requires_grad_(True)
            if self.last:
                lab_d = labels.to(self.device, non_blocking=True)
                valid = int((labels[:, 1:] != -100).sum())
                w = loss_scale * valid / max(total_valid, 1)  # weight of this micro-batch in the step's token mean
                self.model.loss_grad_scale = w
                out = self.model(input_ids=ids_d if self.first else None, inputs_embeds=x_in, labels=lab_d, meta=meta)
                losses.append(out.loss.detach() * w)
                fwd_state[i] = (x_in, out.loss)
            else:
                out = self.model(input_ids=ids_d if self.first else None, inputs_embeds=x_in, meta=meta)
                h = out.hidden_states
                pending.append(self._send(h.detach(), self.s + 1))
                fwd_state[i] = (x_in, h)

        def backward(i: int):
            x_in, y = fwd_state[i]
            fwd_state[i] = None
            if self.last:
                y.backward()
            else:
                buf, req = self._recv(y.shape[0], self.s + 1)
                req.wait()
                torch.autograd.backward(y, buf)
            if not self.first:
                pending.append(self._send(x_in.grad, self.s - 1))

        if self.schedule == "gpipe":
            for i in range(n):
                forward(i)
            for i in range(n):
                backward(i)
        else:  # 1F1B: warm-up forwards, steady state one-forward-one-backward, cool-down backwards
            warm = min(n, self.S - self.s - 1)
            for i in range(warm):
                forward(i)
            f, b = warm, 0
            while f < n:
                forward(f)
                f += 1
                backward(b)
                b += 1
            while b < n:
                backward(b)
                b += 1
        for r in pending:
            r.wait()
        return torch.stack(losses).sum() if losses else None

    def broadcast_loss(self, loss: Optional[torch.Tensor]) -> torch.Tensor:
        t = loss.detach().float().reshape(1) if loss is not None else torch.zeros(1, device=self.device)
        t = t.to(self.device)
        dist.broadcast(t, src=self.ranks[self.S - 1], group=self.group)
        return t[0]
