"""Sharded-parameter mode of the engine: parameters live as 1/N shards and are gathered around each use.

This is the FSDP2 behaviour the reference configures with ``fully_shard(..., reshard_after_forward=...)`` per block and for
the root (flame/models/parallelize_fla.py:406-467): every rank keeps only its slice of every unit's parameters, the full
parameters of a unit exist only while that unit's forward or backward runs, and the full gradient of a unit exists only
until it has been reduce-scattered.  ``ShardedEngine`` (the resident mode, ``fsdp_reshard_after_forward = never``) keeps
one full bf16 copy and one full fp32 gradient buffer per rank instead; this mode trades a little NVLink traffic per block
for per-GPU memory that falls with the number of ranks.

Layout

* per unit and rank, persistent: bf16 parameter shard (``pshard``, peer-readable), fp32 master / AdamW moments, fp32
  gradient shard - 18 bytes per parameter divided by N;
* staging, independent of the model's depth: two full-unit bf16 buffers and two full-unit fp32 gradient buffers that the
  decoder blocks use in turn (block ``i`` uses buffer ``i % 2``, so the module parameters are fixed views and never have to
  be re-pointed), plus one pair for the root unit (embeddings, final norm, head), which stays gathered for the whole step.

Protocol per step

* before a block's forward (and again before its backward, unless its buffer still holds it): the block's small
  parameters (norm weights, convolution taps, ...) are fetched with a stand-alone peer gather kernel and the rest is left
  *pending*: the first GEMM that reads one of the block's weights runs as ``fb_gemm2_gather_b`` - its copy CTAs pull the
  whole remaining range from the peers' shards while its MMA CTAs start on the rows of the weight that have already
  landed (``csrc/gemm2.cu``).  Anything still pending when the block ends is fetched by the stand-alone kernel;
* before a block's backward its gradient buffer is recycled: wait (bounded, on the device) until every peer has pulled
  the previous owner's gradients, then clear it;
* after a block's backward: reduce-scatter into the fp32 gradient shard (accumulating over micro-batches), on the side
  stream, then tell the peers that this rank is done reading their buffers;
* optimizer: AdamW on the shard writes the bf16 shard in place; a flag tells the peers that the new parameters are there.

With a c10d backend (gloo on CPUs, NCCL when the peer kernels are switched off) the same protocol runs on
``all_gather_into_tensor`` / ``reduce_scatter_tensor``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import gemm as gemm_ops
from ..ops import optim as optim_ops
from .engine import ALIGN, ParamSlot, ShardedEngine, TorchCollectives, Unit, default_unit_plan

CHUNK_SHIFT = 17                      # flags of the fused gather cover 128 KB each
CHUNK_ELEMS = (1 << CHUNK_SHIFT) // 2  # bf16 elements per chunk
SMALL_NUMEL = 65536                   # parameters up to this size are fetched ahead of the block's first GEMM


class ReshardingEngine(ShardedEngine):
    resharding = True

    def __init__(self, *args, policy: str = "default", fuse_gather: bool = True, **kw) -> None:
        self.policy = policy
        self.fuse_gather = fuse_gather
        self.param_version = 0          # bumped by every optimizer step: what a staging buffer holds is stale afterwards
        self._micro = 0                 # micro-batches reduced so far in this step
        self._pending: Optional[gemm_ops.PendingGather] = None
        super().__init__(*args, **kw)
        if self.cpu_offload:
            raise ValueError("sharded-parameter mode does not combine with optimizer-state offload")

    # ------------------------------------------------------------------------------------------------
    def _build(self) -> None:
        plan = default_unit_plan(self.model)
        N = self.shard_world
        mult = N * CHUNK_ELEMS if self.param_dtype == torch.bfloat16 else N * ALIGN
        layouts = []
        total = 0
        for name, named in plan:
            seen: Dict[int, bool] = {}
            uniq = []
            for fqn, p in named:
                if id(p) not in seen:
                    seen[id(p)] = True
                    uniq.append((fqn, p))
            # small parameters first (stable), so that one short gather makes them available before the first GEMM
            ordered = [x for x in uniq if x[1].numel() <= SMALL_NUMEL] + [x for x in uniq if x[1].numel() > SMALL_NUMEL]
            slots, off, small_end = [], 0, 0
            for fqn, p in ordered:
                n = p.numel()
                slots.append(ParamSlot(fqn, tuple(p.shape), off, n, p))
                off += (n + ALIGN - 1) // ALIGN * ALIGN
                if n <= SMALL_NUMEL:
                    small_end = off
            numel = max(mult, (off + mult - 1) // mult * mult)
            layouts.append((name, slots, numel, small_end))
            total += numel
        self.total_numel = total
        blocks = [l for l in layouts if l[0] != "root"]
        max_block = max((l[2] for l in blocks), default=0)
        root_numel = next((l[2] for l in layouts if l[0] == "root"), 0)
        dev, pd = self.device, self.param_dtype
        self.pshard_all = self._alloc(total // N, pd, "pshard")
        # staging: blocks alternate between two buffers, the root unit has its own
        self.cbuf = [torch.zeros(max_block, dtype=pd, device=dev) for _ in range(2)] if max_block else []
        self.gbuf = [self._alloc(max_block, torch.float32, f"gbuf{k}") for k in range(2)] if max_block else []
        self.root_c = torch.zeros(root_numel, dtype=pd, device=dev)
        self.root_g = self._alloc(root_numel, torch.float32, "gbuf_root")
        nflags = max(1, (max(max_block, root_numel) * self.pshard_all.element_size() >> CHUNK_SHIFT) + 1)
        self.cflags = [torch.zeros(nflags, dtype=torch.int32, device=dev) for _ in range(3)]
        self._cbuf_owner: List[Optional[Tuple[str, int]]] = [None, None, None]  # (unit name, parameter version)
        self._gbuf_owner: List[Optional[Unit]] = [None, None, None]
        self._gather_epoch = [0, 0, 0]
        replaced: Dict[int, nn.Parameter] = {}
        base, bi = 0, 0
        for name, slots, numel, small_end in layouts:
            u = Unit(name, slots, numel, N, self.shard_rank)
            u.base, u.sbase, u.small_end = base, base // N, small_end
            if name == "root":
                u.buf = 2
                u.compute, u.grad = self.root_c[:numel], self.root_g[:numel]
            else:
                u.buf = bi % 2
                bi += 1
                u.compute, u.grad = self.cbuf[u.buf][:numel], self.gbuf[u.buf][:numel]
            s = u.shard_size
            u.pshard = self.pshard_all[u.sbase:u.sbase + s]
            u.master = torch.zeros(s, dtype=torch.float32, device=dev)
            u.exp_avg = torch.zeros(s, dtype=torch.float32, device=dev)
            u.exp_avg_sq = torch.zeros(s, dtype=torch.float32, device=dev)
            u.grad_shard = torch.zeros(s, dtype=torch.float32, device=dev)
            u.rs_seq = 0
            u.rs_event = None
            for slot in slots:
                view = u.compute[slot.offset:slot.offset + slot.numel].view(slot.shape)
                newp = nn.Parameter(view, requires_grad=True)
                for attr in ("_no_weight_decay", "_tp", "_tp_replicated", "_fp8"):
                    if hasattr(slot.param, attr):
                        setattr(newp, attr, getattr(slot.param, attr))
                newp.main_grad = u.grad[slot.offset:slot.offset + slot.numel].view(slot.shape)
                replaced[id(slot.param)] = newp
                slot.param = newp
            self.units.append(u)
            base += numel
        for mod in self.model.modules():
            for pname, p in list(mod._parameters.items()):
                if p is not None and id(p) in replaced:
                    mod._parameters[pname] = replaced[id(p)]
        self._unit_by_name = {u.name: u for u in self.units}

    # ---- memory accounting ----------------------------------------------------------------------------------
    def memory_report(self) -> Dict[str, float]:
        """Bytes this rank holds for parameters, gradients and optimizer state."""
        pe = self.pshard_all.element_size()
        sharded = self.pshard_all.numel() * pe + sum(u.shard_size * 16 for u in self.units)  # grad shard + master + 2 moments
        staging = sum(b.numel() * pe for b in self.cbuf) + self.root_c.numel() * pe + \
            sum(b.numel() * 4 for b in self.gbuf) + self.root_g.numel() * 4
        return {"mode": "sharded parameters", "sharded_bytes": float(sharded), "staging_bytes": float(staging),
                "total_bytes": float(sharded + staging), "parameters": float(self.total_numel)}

    # ---- initialisation / state ---------------------------------------------------------------------------
    def init_weights(self, seed: Optional[int] = None) -> None:
        scratch = torch.zeros(self.total_numel, dtype=torch.float32, device=self.device)
        saved = []
        for u in self.units:
            for s_ in u.slots:
                saved.append((s_.param, s_.param.data))
                s_.param.data = scratch[u.base + s_.offset:u.base + s_.offset + s_.numel].view(s_.shape)
        try:
            self.model.init_weights(seed)
        finally:
            for p, d in saved:
                p.data = d
        with torch.no_grad():
            for u in self.units:
                a, b = u.shard_range
                part = scratch[u.base + a:u.base + b]
                u.master.copy_(part)
                u.pshard.copy_(part)
        self._params_changed()

    def _params_changed(self) -> None:
        self.param_version += 1
        self._cbuf_owner = [None, None, None]
        if hasattr(self.collectives, "params_written"):
            self.collectives.params_written(self.param_version)

    @torch.no_grad()
    def refresh_compute(self) -> None:
        for u in self.units:
            u.pshard.copy_(u.master)
        self._params_changed()

    @torch.no_grad()
    def load_full_state(self, tensors, kind: str = "master", strict: bool = True, units=None) -> None:
        for u in (units if units is not None else self.units):
            a, b = u.shard_range
            dst = getattr(u, kind)
            for s in u.slots:
                if s.fqn not in tensors:
                    if strict:
                        raise KeyError(f"missing {s.fqn} in checkpoint")
                    continue
                src = tensors[s.fqn].reshape(-1).to(device=self.device, dtype=torch.float32)
                lo, hi = max(a, s.offset), min(b, s.offset + s.numel)
                if lo < hi:
                    dst[lo - a:hi - a].copy_(src[lo - s.offset:hi - s.offset])
            if kind == "master":
                u.pshard.copy_(u.master)
        if kind == "master":
            self._params_changed()

    # ---- gathering parameters -----------------------------------------------------------------------------
    def _flush_pending(self) -> None:
        """Whatever part of a unit no GEMM has fetched is fetched now, by the stand-alone kernel."""
        pend, self._pending = self._pending, None
        gemm_ops.set_pending_gather(None)
        if pend is not None and not pend.done:
            self.collectives.gather_params(pend.unit, pend.lo, pend.hi)

    def ensure_params(self, u: Unit) -> None:
        """After this call the kernels launched next on this stream may read ``u``'s parameters (except the part that the
        pending fused gather brings in together with the first GEMM that touches it)."""
        want = (u.name, self.param_version)
        if self._cbuf_owner[u.buf] == want:
            return
        self._flush_pending()
        self._cbuf_owner[u.buf] = want
        nbytes = u.numel * u.compute.element_size()
        fused = (self.fuse_gather and self.shard_world > 1 and getattr(self.collectives, "can_fuse_gather", False)
                 and u.name != "root")
        if not fused:
            self.collectives.gather_params(u, 0, nbytes)
            return
        small = u.small_end * u.compute.element_size()
        if small:
            self.collectives.gather_params(u, 0, small)
        self._gather_epoch[u.buf] += 1
        self._pending = self.collectives.make_pending(u, small, nbytes, self.cflags[u.buf], self._gather_epoch[u.buf])
        gemm_ops.set_pending_gather(self._pending)

    def _prepare_grad_buffer(self, u: Unit) -> None:
        prev = self._gbuf_owner[u.buf]
        if prev is u and getattr(u, "_grad_ready_for", None) == (self.param_version, self._micro):
            return
        if prev is not None and prev.rs_event is not None:
            torch.cuda.current_stream().wait_event(prev.rs_event)   # this rank's own pull out of the buffer
        if prev is not None and prev.rs_seq > 0 and hasattr(self.collectives, "wait_pulled"):
            self.collectives.wait_pulled(prev)                     # every peer's pull out of this rank's buffer
        u.grad.zero_()
        self._gbuf_owner[u.buf] = u
        u._grad_ready_for = (self.param_version, self._micro)

    # ---- hooks ------------------------------------------------------------------------------------------------
    def install_backward_hooks(self) -> None:
        if self._hooks_installed:
            return
        from ..models.modeling import get_blocks
        blocks = [b for b in get_blocks(self.model) if b is not None]
        root = self._unit_by_name.get("root")

        def model_pre(mod, args, kwargs=None):
            if root is not None:
                self.ensure_params(root)
            return None

        self.model.register_forward_pre_hook(model_pre)
        for blk in blocks:
            u = self._unit_by_name.get(f"layers.{blk.layer_idx}")
            if u is None:
                continue

            def pre_hook(mod, args, _u=u):
                self.ensure_params(_u)
                x = args[0]
                if torch.is_grad_enabled() and isinstance(x, torch.Tensor) and x.requires_grad:
                    x.register_hook(lambda g, __u=_u: self._on_unit_backward_done(__u, g))
                return None

            def post_hook(mod, args, out, _u=u):
                self._flush_pending()
                if torch.is_grad_enabled():
                    for t in (out if isinstance(out, (tuple, list)) else (out,)):
                        if isinstance(t, torch.Tensor) and t.requires_grad:
                            t.register_hook(lambda g, __u=_u: self._before_unit_backward(__u))
                return None

            blk.register_forward_pre_hook(pre_hook)
            blk.register_forward_hook(post_hook)
        self._hooks_installed = True

    def _before_unit_backward(self, u: Unit):
        self.ensure_params(u)
        self._prepare_grad_buffer(u)
        return None

    def _on_unit_backward_done(self, u: Unit, g: torch.Tensor):
        # (a pending gather at this point belongs to the NEXT block's backward, whose hook ran just before this one)
        if not u.reduced:
            self._reduce_unit(u)
        return None

    # ---- step ---------------------------------------------------------------------------------------------------
    def zero_grad(self) -> None:
        for u in self.units:
            u.reduced = False
        self._norm_zeroed = False
        self._micro = 0
        self._mb_calls = 0
        if hasattr(self.collectives, "begin_step"):
            self.collectives.begin_step()
        root = self._unit_by_name.get("root")
        if root is not None:
            self._prepare_grad_buffer(root)   # the head's gradient is formed during the forward pass

    def set_last_microbatch(self, flag: bool) -> None:
        """The trainer calls this once before every micro-batch: the second and later calls of a step mark the boundary
        after which block gradients are reduced again and ADDED to the gradient shards."""
        self._mb_calls = getattr(self, "_mb_calls", 0) + 1
        if self._mb_calls > 1:
            self.next_microbatch()
        self._last_microbatch = flag

    def next_microbatch(self) -> None:
        """Called between the micro-batches of one step: the blocks' gradients were reduced into the shards already."""
        self._micro += 1
        for u in self.units:
            if u.name != "root":
                u.reduced = False

    def _reduce_unit(self, u: Unit) -> None:
        self._fold_autograd_grads(u)
        self._zero_norm_once()
        accumulate = self._micro > 0 and u.name != "root"
        u.rs_seq += 1
        if self.comm_stream is not None and self.shard_world > 1:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self.collectives.reduce_scatter_avg(u, self.shard_world, accumulate=accumulate,
                                                    want_norm=self._last_microbatch)
                u.rs_event = self.comm_stream.record_event()
        else:
            self.collectives.reduce_scatter_avg(u, self.shard_world, accumulate=accumulate, want_norm=self._last_microbatch)
        u.reduced = True

    @torch.no_grad()
    def step(self, lr: float, grad_scale: float = 1.0) -> None:
        self._flush_pending()
        for u in self.units:
            if not u.reduced:
                self._reduce_unit(u)
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        if self.replica_reducer is not None:
            for u in self.units:
                self.replica_reducer(u.grad_shard)
        if self.commit_gate is not None and not self.commit_gate():
            self.voided_steps += 1
            return
        o = self.optim
        optim_ops.latch_status(self.ctrl)
        if self._norm_scratch is None and self.device.type == "cuda":
            self._norm_scratch = torch.empty(2048, dtype=torch.float32, device=self.device)
        if not getattr(self.collectives, "norm_fused", False) or self.shard_world == 1:
            self.ctrl[optim_ops.CTRL_NORM_SQ] = 0
            for u in self.units:
                optim_ops.sumsq_accumulate(u.grad_shard, self.ctrl[optim_ops.CTRL_NORM_SQ:optim_ops.CTRL_NORM_SQ + 1],
                                           self._norm_scratch, accumulate=True)
        self._all_reduce_norm()
        for u in self.units:
            lowp = u.pshard if (self.param_dtype == torch.bfloat16 or self.device.type != "cuda") else None
            optim_ops.adamw_step(u.master, u.exp_avg, u.exp_avg_sq, u.grad_shard, lowp, self.ctrl, lr, o.beta1, o.beta2,
                                 o.eps, o.kernel_weight_decay, o.max_norm, o.skip_nan_inf, grad_scale)
            if lowp is None:
                u.pshard.copy_(u.master)
        optim_ops.adamw_finalize(self.ctrl, o.max_norm, o.skip_nan_inf, grad_scale)
        self._params_changed()


class TorchReshardCollectives(TorchCollectives):
    """The sharded-parameter protocol on c10d collectives (gloo on CPUs, NCCL when the peer kernels are switched off)."""

    can_fuse_gather = False
    norm_fused = False

    def gather_params(self, u: Unit, lo: int, hi: int) -> None:
        world = dist.get_world_size(self.group) if self.group is not None else 1
        if world == 1:
            u.compute.copy_(u.pshard)
            return
        if self._gloo:
            parts = [torch.empty_like(u.pshard) for _ in range(world)]
            dist.all_gather(parts, u.pshard.clone(), group=self.group)
            torch.cat(parts, out=u.compute)
        else:
            dist.all_gather_into_tensor(u.compute, u.pshard, group=self.group)

    def reduce_scatter_avg(self, unit: Unit, world: int, accumulate: bool = False, want_norm: bool = True) -> None:
        a, b = unit.shard_range
        if world == 1 or self.group is None:
            part = unit.grad[a:b]
        elif self._gloo:
            dist.all_reduce(unit.grad, group=self.group)
            part = unit.grad[a:b] / world
        else:
            part = torch.empty_like(unit.grad_shard)
            dist.reduce_scatter_tensor(part, unit.grad, op=dist.ReduceOp.AVG, group=self.group)
        if self.replicate_group is not None:
            part = part.clone()
            dist.all_reduce(part, group=self.replicate_group)
            part /= dist.get_world_size(self.replicate_group)
        if accumulate:
            unit.grad_shard.add_(part)
        else:
            unit.grad_shard.copy_(part)
