"""Pipeline parallelism: layer ranges per stage, micro-batching of packed rows, and an executor for the schedules
of ``pp_schedule`` (GPipe, 1F1B, Interleaved1F1B, LoopedBFS, CSV) over point-to-point sends (NCCL on GPUs, gloo on
CPUs).

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
from . import pp_schedule
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


def split_into_stage(model, model_config, dims: ParallelDims, job_config) -> List[Tuple[int, int]]:
    """Keeps only this pipeline rank's stages of the (meta-device) model; returns their layer ranges.

    One stage per rank for GPipe / 1F1B; the looped schedules (Interleaved1F1B, LoopedBFS) and CSV schedules may place
    several stages on a rank, dealt round-robin as torchtitan's ``stage_ids_this_rank`` does in its "loop" style."""
    S_ranks, r = dims.pp, dims.local_rank_in("pp")
    ex = job_config.experimental if job_config is not None else None
    pts = list(ex.pipeline_parallel_split_points) if ex is not None else []
    name = ex.pipeline_parallel_schedule if ex is not None else "1F1B"
    csv_path = (ex.pipeline_parallel_schedule_csv or None) if ex is not None else None
    _, n_stages, owner, key = pp_schedule.resolve(name, csv_path, S_ranks, None, model_config.num_hidden_layers)
    if pts:
        n_stages = len(pts) + 1
        if n_stages % S_ranks:
            raise ValueError(f"{len(pts)} split points give {n_stages} stages, not a multiple of {S_ranks} ranks")
        if csv_path is None:
            owner = pp_schedule.stage_owners(S_ranks, n_stages)
        elif len(owner) != n_stages:
            raise ValueError(f"the schedule CSV has {len(owner)} stages, the split points give {n_stages}")
    ranges = stage_layer_ranges(model_config.num_hidden_layers, n_stages, pts)
    mine = [s for s in range(n_stages) if owner[s] == r]
    keep = set()
    for s in mine:
        keep.update(range(*ranges[s]))
    dec = model.decoder
    for i in range(len(dec.layers)):
        if i not in keep:
            dec.layers[i] = None
    if 0 not in mine:
        dec.embeddings = None
    if n_stages - 1 not in mine:
        for nm in ("norm", "norm_f"):
            if hasattr(dec, nm):
                setattr(dec, nm, None)
        model.lm_head = None
    model.pp_stage_ranges = {s: ranges[s] for s in mine}
    model.pp_owner, model.pp_n_stages, model.pp_schedule_name = owner, n_stages, key
    logger.info(f"pipeline rank {r}/{S_ranks}: stages {mine} of {n_stages} ({key}), layers "
                f"{[ranges[s] for s in mine]}")
    return [ranges[s] for s in mine]


class PipelineRunner:
    """Runs one optimizer step's micro-batches through this rank's stages in the order its schedule gives.

    Sends and receives are posted per peer in the order of ``pp_schedule.pair_message_order`` (sorted by the simulated
    tick at which each boundary tensor is produced), identically on both sides of every pair, so first-in-first-out
    channels match whatever the interleaving; a receive is posted no later than the first send that follows it in that
    order, and waited for only when its consumer runs."""

    def __init__(self, model, engine, dims: ParallelDims, device: torch.device, job_config) -> None:
        self.model, self.engine, self.dims, self.device = model, engine, dims, device
        self.group = dims.group("pp")
        self.ranks = dims.group_ranks("pp")
        self.S = dims.pp
        self.s = dims.local_rank_in("pp")
        ex = job_config.experimental
        self.n_mb = ex.pipeline_parallel_microbatches or self.S
        self.schedule = (ex.pipeline_parallel_schedule or "1F1B")
        self.csv_path = ex.pipeline_parallel_schedule_csv or None
        self.n_stages: int = model.pp_n_stages
        self.owner: List[int] = model.pp_owner
        self.stage_ranges: Dict[int, Tuple[int, int]] = model.pp_stage_ranges
        self.last = (self.n_stages - 1) in self.stage_ranges  # this rank computes the loss
        self.hidden = model.config.hidden_size
        self.dtype = engine.param_dtype
        self._plans: Dict[int, tuple] = {}

    # ---- schedule for a given number of micro-batches ------------------------------------------------------
    def _plan(self, n: int):
        plan = self._plans.get(n)
        if plan is None:
            if self.csv_path:
                sched, n_stages, owner, _ = pp_schedule.resolve(None, self.csv_path, self.S, n, 0)
            else:
                key = self.schedule.lower()
                if key == "interleaved1f1b" and n % self.S:
                    key = "loopedbfs"
                if key in pp_schedule.SINGLE_STAGE and self.n_stages != self.S:
                    key = "loopedbfs"  # split points put several stages on a rank
                sched = pp_schedule.build_schedule(key, self.S, self.n_stages, n)
                n_stages, owner = self.n_stages, self.owner
            if n_stages != self.n_stages or list(owner) != list(self.owner):
                raise ValueError("the pipeline schedule does not match the stages this model was split into")
            order = pp_schedule.pair_message_order(sched, owner, n)
            mine = {}
            for (lo, hi), msgs in order.items():
                if self.s in (lo, hi):
                    mine[hi if lo == self.s else lo] = msgs
            plan = (sched[self.s], mine)
            self._plans[n] = plan
        return plan

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

    # ---- one optimizer step's worth of micro-batches -----------------------------------------------------------------
    def forward_backward(self, batch: Dict[str, torch.Tensor], loss_scale: float = 1.0) -> Optional[torch.Tensor]:
        mbs = self._microbatches(batch)
        n = len(mbs)
        actions, peer_msgs = self._plan(n)
        total_valid = sum(int((lab[:, 1:] != -100).sum()) for _, lab, _ in mbs)
        tokens = [ids.numel() for ids, _, _ in mbs]
        metas: Dict[int, VarlenMeta] = {}
        ptr = {p: 0 for p in peer_msgs}
        index = {p: {(m.kind, m.stage, m.mb): i for i, m in enumerate(msgs)} for p, msgs in peer_msgs.items()}
        recv_req: Dict[tuple, tuple] = {}
        outbox: Dict[tuple, torch.Tensor] = {}
        local: Dict[tuple, torch.Tensor] = {}   # boundary tensors between two stages of this rank
        sends = []
        saved: Dict[Tuple[int, int], tuple] = {}
        losses = []

        def advance(peer: int, key: tuple) -> None:
            """Posts, in pair order, everything up to and including message ``key`` on the channel to ``peer``."""
            msgs, target = peer_msgs[peer], index[peer][key]
            while ptr[peer] <= target:
                msg = msgs[ptr[peer]]
                k = (msg.kind, msg.stage, msg.mb)
                if msg.dst == self.s:
                    buf = torch.empty(tokens[msg.mb], self.hidden, dtype=self.dtype, device=self.device)
                    recv_req[k] = (buf, dist.irecv(buf, src=self.ranks[peer], group=self.group))
                else:
                    t = outbox.pop(k, None)
                    if t is None:
                        raise RuntimeError(f"pipeline schedule asks to send {k} before it was computed")
                    sends.append((t, dist.isend(t, dst=self.ranks[peer], group=self.group)))
                ptr[peer] += 1

        def fetch(kind: str, stage: int, mb: int, src_stage: int) -> torch.Tensor:
            k = (kind, stage, mb)
            peer = self.owner[src_stage]
            if peer == self.s:
                return local.pop(k)
            advance(peer, k)
            buf, req = recv_req.pop(k)
            req.wait()
            return buf

        def emit(kind: str, stage: int, mb: int, dst_stage: int, t: torch.Tensor) -> None:
            k = (kind, stage, mb)
            peer = self.owner[dst_stage]
            if peer == self.s:
                local[k] = t
                return
            outbox[k] = t.contiguous()
            advance(peer, k)

        def meta_of(mb: int) -> VarlenMeta:
            mt = metas.get(mb)
            if mt is None:
                ids, _, cu = mbs[mb]
                mt = (VarlenMeta.from_cu_seqlens(cu, tokens[mb], self.device) if cu is not None
                      else VarlenMeta.dense(ids.shape[0], ids.shape[1], self.device))
                metas[mb] = mt
            return mt

        for act in actions:
            st, mb = act.stage, act.mb
            first, last = st == 0, st == self.n_stages - 1
            lo, hi = self.stage_ranges[st]
            stage_arg = (lo, hi, first, last)
            if act.op == pp_schedule.F:
                ids, labels, _ = mbs[mb]
                x_in = None
                if not first:
                    x_in = fetch("A", st, mb, st - 1).requires_grad_(True)
                ids_d = ids.to(self.device, non_blocking=True) if first else None
                if last:
                    lab_d = labels.to(self.device, non_blocking=True)
                    valid = int((labels[:, 1:] != -100).sum())
                    w = loss_scale * valid / max(total_valid, 1)  # weight of this micro-batch in the step's token mean
                    self.model.loss_grad_scale = w
                    out = self.model(input_ids=ids_d, inputs_embeds=x_in, labels=lab_d, meta=meta_of(mb), stage=stage_arg)
                    losses.append(out.loss.detach() * w)
                    saved[(st, mb)] = (x_in, out.loss)
                else:
                    out = self.model(input_ids=ids_d, inputs_embeds=x_in, meta=meta_of(mb), stage=stage_arg)
                    h = out.hidden_states
                    saved[(st, mb)] = (x_in, h)
                    emit("A", st + 1, mb, st + 1, h.detach())
            else:
                x_in, y = saved.pop((st, mb))
                if last:
                    y.backward()
                else:
                    torch.autograd.backward(y, fetch("G", st, mb, st + 1))
                if not first:
                    emit("G", st - 1, mb, st - 1, x_in.grad)
        for p, msgs in peer_msgs.items():
            if ptr[p] != len(msgs) or recv_req or outbox:
                raise RuntimeError("pipeline step ended with boundary tensors not exchanged")
        for _, r in sends:
            r.wait()
        return torch.stack(losses).sum() if losses else None

    def broadcast_loss(self, loss: Optional[torch.Tensor]) -> torch.Tensor:
        t = loss.detach().float().reshape(1) if loss is not None else torch.zeros(1, device=self.device)
        t = t.to(self.device)
        dist.broadcast(t, src=self.ranks[self.owner[self.n_stages - 1]], group=self.group)
        return t[0]
