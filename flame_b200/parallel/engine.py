"""Sharded data-parallel training engine (FSDP / HSDP / DDP semantics on flat buffers).

What the reference gets from FSDP2 (``fully_shard`` per block + root with bf16 parameters and fp32 gradient
reduction, flame/models/parallelize_fla.py:406-486) plus the fused AdamW, gradient clipping and NaN skipping of
its trainer (flame/train.py:509-528) is provided here by one engine built for 180 GB devices:

* Parameters are grouped into **units** (one per decoder block, one root unit for embeddings / final norm /
  head).  A unit owns one flat compute-dtype buffer (the model's parameters are views into it, projections that
  are evaluated together sit back to back so they form one GEMM operand) and one flat fp32 gradient buffer
  (``param.main_grad`` views; weight-gradient GEMMs accumulate straight into it).
* Each data-parallel-shard rank owns a contiguous 1/N slice of every unit: fp32 master weights and both AdamW
  moments exist only for that slice.
* The unsharded compute buffers stay resident (a 7B model is 13.5 GB in bf16), so parameters are gathered
  once per step, right after the optimizer, instead of before every block's forward and backward.
* Per step and unit: reduce-scatter(avg) of the fp32 gradients -> sum of squares of the local slice ->
  (after one scalar all-reduce) AdamW with the clip coefficient and the NaN/Inf skip decided on the device ->
  compute-dtype parameters written back and gathered.  The reduce-scatter of a unit is issued from a backward
  hook as soon as that unit's gradients are complete and runs on a side stream.

The collective steps go through a ``Collectives`` backend: ``TorchCollectives`` (NCCL / gloo) or the peer-memory
kernels of ``flame_b200.parallel.peer``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import optim as optim_ops
from .dims import ParallelDims

ALIGN = 64  # elements; keeps every parameter 128-byte aligned in bf16 (TMA needs 16 bytes)


@dataclass
class OptimConfig:
    lr: float = 8e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_norm: float = 1.0
    skip_nan_inf: bool = False
    name: str = "AdamW"

    def __post_init__(self) -> None:
        if self.name not in ("AdamW", "Adam"):
            raise NotImplementedError(f"Optimizer {self.name} not added.")  # torchtitan/components/optimizer.py:304-310

    @property
    def kernel_weight_decay(self) -> float:
        """What the update kernels take: ``weight_decay`` for AdamW (decoupled), its negative for Adam (L2 through the
        gradient, the rule of ``torch.optim.Adam``)."""
        return self.weight_decay if self.name == "AdamW" else -self.weight_decay


@dataclass
class ParamSlot:
    fqn: str
    shape: Tuple[int, ...]
    offset: int  # element offset inside the unit's flat buffers
    numel: int
    param: nn.Parameter = field(repr=False, default=None)


class Unit:
    def __init__(self, name: str, slots: List[ParamSlot], numel: int, shard_world: int, shard_rank: int) -> None:
        self.name, self.slots = name, slots
        self.numel = numel  # padded to a multiple of shard_world * ALIGN
        self.shard_size = numel // shard_world
        self.shard_rank = shard_rank
        self.compute: torch.Tensor = None
        self.grad: torch.Tensor = None
        self.master: torch.Tensor = None
        self.exp_avg: torch.Tensor = None
        self.exp_avg_sq: torch.Tensor = None
        self.grad_shard: torch.Tensor = None
        self.reduced = False

    @property
    def shard_range(self) -> Tuple[int, int]:
        a = self.shard_rank * self.shard_size
        return a, a + self.shard_size

    def compute_shard(self) -> torch.Tensor:
        a, b = self.shard_range
        return self.compute[a:b]


class Collectives:
    """Collective steps the engine needs; implementations must be deterministic in their summation order."""

    def reduce_scatter_avg(self, unit: Unit, world: int) -> None:
        raise NotImplementedError

    def all_gather_params(self, unit: Unit, world: int) -> None:
        raise NotImplementedError


class TorchCollectives(Collectives):
    """c10d collectives over the shard group (NCCL on GPUs, gloo on CPUs)."""

    def __init__(self, group: Optional[dist.ProcessGroup], replicate_group: Optional[dist.ProcessGroup] = None) -> None:
        self.group, self.replicate_group = group, replicate_group
        self._gloo = group is not None and dist.get_backend(group) == "gloo"

    def reduce_scatter_avg(self, unit: Unit, world: int) -> None:
        if world == 1 or self.group is None:
            unit.grad_shard = unit.grad  # alias: nothing to reduce
        elif self._gloo:
            dist.all_reduce(unit.grad, group=self.group)
            a, b = unit.shard_range
            unit.grad_shard.copy_(unit.grad[a:b]).div_(world)
        else:
            dist.reduce_scatter_tensor(unit.grad_shard, unit.grad, op=dist.ReduceOp.AVG, group=self.group)
        if self.replicate_group is not None:
            dist.all_reduce(unit.grad_shard, group=self.replicate_group)
            unit.grad_shard.div_(dist.get_world_size(self.replicate_group))

    def all_gather_params(self, unit: Unit, world: int) -> None:
        if world == 1 or self.group is None:
            return
        if self._gloo:
            parts = [torch.empty_like(unit.compute_shard()) for _ in range(world)]
            dist.all_gather(parts, unit.compute_shard().clone(), group=self.group)
            for r, p in enumerate(parts):
                unit.compute[r * unit.shard_size:(r + 1) * unit.shard_size].copy_(p)
        else:
            dist.all_gather_into_tensor(unit.compute, unit.compute_shard().clone(), group=self.group)


def default_unit_plan(model: nn.Module) -> List[Tuple[str, List[Tuple[str, nn.Parameter]]]]:
    """One unit per decoder block, and a root unit with everything else (embeddings, final norm, head)."""
    from ..models.modeling import get_blocks
    blocks = get_blocks(model)
    prefix = model.base_model_prefix
    claimed = set()
    units = []
    for i, blk in enumerate(blocks):
        if blk is None:
            continue
        named = [(f"{prefix}.layers.{i}.{n}", p) for n, p in blk.named_parameters()]
        for _, p in named:
            claimed.add(id(p))
        units.append((f"layers.{i}", named))
    root = [(n, p) for n, p in model.named_parameters() if id(p) not in claimed]
    units.append(("root", root))
    return units


class ShardedEngine:
    def __init__(self, model: nn.Module, dims: ParallelDims, device: torch.device, param_dtype: torch.dtype,
                 optim: OptimConfig, collectives: Optional[Collectives] = None,
                 allocator: Optional[Callable[[int, torch.dtype, str], torch.Tensor]] = None,
                 overlap: bool = True, cpu_offload: bool = False) -> None:
        self.model, self.dims, self.device, self.param_dtype, self.optim = model, dims, device, param_dtype, optim
        # optimizer-state offload (``training.enable_cpu_offload``): the fp32 master weights and both AdamW moments
        # (12 of the 16-18 bytes a parameter costs) live in pinned host memory and pass through two device staging
        # sets, one unit at a time, while the update kernel of the previous unit runs
        self.cpu_offload = cpu_offload and device.type == "cuda"
        self._stage: List[List[torch.Tensor]] = []
        self._stage_free: List[Optional[torch.cuda.Event]] = [None, None]
        self._copy_stream = torch.cuda.Stream(device=device) if self.cpu_offload else None
        self.shard_world = dims.group_size("dp_shard_cp") if dims._ranks else 1
        self.shard_rank = dims.local_rank_in("dp_shard_cp") if dims._ranks else 0
        self.collectives = collectives or TorchCollectives(dims.group("dp_shard_cp"), dims.group("dp_replicate"))
        self._alloc = allocator or (lambda n, dt, tag: torch.zeros(n, dtype=dt, device=device))
        self.units: List[Unit] = []
        self.ctrl = torch.zeros(optim_ops.CTRL_SIZE, dtype=torch.float32, device=device)
        self._norm_scratch: Optional[torch.Tensor] = None
        self.overlap = overlap and device.type == "cuda"
        self.comm_stream = torch.cuda.Stream(device=device) if self.overlap else None
        self.replica_reducer = None   # callable(tensor): in-place average over fault-tolerant replica groups
        self.commit_gate = None       # callable() -> bool: False voids the step (no update is applied)
        self.voided_steps = 0
        self._last_microbatch = True
        self._hooks_installed = False
        self._norm_groups: List[Optional[dist.ProcessGroup]] = []
        self._build()

    # ------------------------------------------------------------------------------------------------
    def _build(self) -> None:
        plan = default_unit_plan(self.model)
        total = 0
        layouts = []
        for name, named in plan:
            slots, off = [], 0
            seen: Dict[int, ParamSlot] = {}
            for fqn, p in named:
                if id(p) in seen:  # tied parameter: one slot
                    continue
                n = p.numel()
                slot = ParamSlot(fqn, tuple(p.shape), off, n, p)
                seen[id(p)] = slot
                slots.append(slot)
                off += (n + ALIGN - 1) // ALIGN * ALIGN
            mult = self.shard_world * ALIGN
            numel = max(mult, (off + mult - 1) // mult * mult)
            layouts.append((name, slots, numel))
            total += numel
        # one allocation per kind for the whole model; units are slices (keeps peer mappings to two buffers)
        compute_all = self._alloc(total, self.param_dtype, "compute")
        grad_all = self._alloc(total, torch.float32, "grad")
        self.compute_all, self.grad_all = compute_all, grad_all
        base = 0
        replaced: Dict[int, nn.Parameter] = {}
        for name, slots, numel in layouts:
            u = Unit(name, slots, numel, self.shard_world, self.shard_rank)
            u.base = base
            u.compute = compute_all[base:base + numel]
            u.grad = grad_all[base:base + numel]
            s = u.shard_size
            if self.cpu_offload:
                u.master, u.exp_avg, u.exp_avg_sq = (torch.zeros(s, dtype=torch.float32).pin_memory() for _ in range(3))
            else:
                u.master = torch.zeros(s, dtype=torch.float32, device=self.device)
                u.exp_avg = torch.zeros(s, dtype=torch.float32, device=self.device)
                u.exp_avg_sq = torch.zeros(s, dtype=torch.float32, device=self.device)
            u.grad_shard = torch.zeros(s, dtype=torch.float32, device=self.device) if self.shard_world > 1 else u.grad
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
        # swap the module tree's parameters for the views
        for mod in self.model.modules():
            for pname, p in list(mod._parameters.items()):
                if p is not None and id(p) in replaced:
                    mod._parameters[pname] = replaced[id(p)]
        self.total_numel = total

    def memory_report(self) -> Dict[str, float]:
        """Bytes this rank holds for parameters, gradients and optimizer state."""
        pe = self.compute_all.element_size()
        sharded = sum(u.shard_size * (12 + (4 if self.shard_world > 1 else 0)) for u in self.units)
        full = self.total_numel * (pe + 4)
        return {"mode": "resident parameters", "sharded_bytes": float(sharded), "staging_bytes": float(full),
                "total_bytes": float(sharded + full), "parameters": float(self.total_numel)}

    def init_weights(self, seed: Optional[int] = None) -> None:
        """Initialise identically on every rank, in fp32: the parameters are pointed at an fp32 scratch buffer while the
        model's initialiser runs, the master slices take those values exactly and the compute buffers their rounding, so
        master == fp32 init and compute == bf16(master) (the reference initialises fp32 parameters and casts for compute
        only, flame/train.py:279-281 under FSDP2 mixed precision)."""
        if self.param_dtype == torch.float32:
            self.model.init_weights(seed)
            self.sync_master_from_compute()
            return
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
                full = scratch[u.base:u.base + u.numel]
                u.compute.copy_(full)
                a, b = u.shard_range
                u.master.copy_(full[a:b])

    @torch.no_grad()
    def sync_master_from_compute(self) -> None:
        for u in self.units:
            u.master.copy_(u.compute_shard())

    # ------------------------------------------------------------------------------------------------
    def install_backward_hooks(self) -> None:
        """Issue a unit's gradient reduction as soon as the gradient w.r.t. that block's input exists."""
        if self._hooks_installed or self.dims.tp_enabled or self.dims.pp_enabled:
            return  # with tp / pp the reductions are issued from step(), after the replicated gradients were summed
        from ..models.modeling import get_blocks
        blocks = [b for b in get_blocks(self.model) if b is not None]
        unit_of = {u.name: u for u in self.units}
        for blk in blocks:
            u = unit_of.get(f"layers.{blk.layer_idx}")
            if u is None:
                continue

            def pre_hook(mod, args, _u=u):
                x = args[0]
                if torch.is_grad_enabled() and isinstance(x, torch.Tensor) and x.requires_grad:
                    x.register_hook(lambda g, __u=_u: self._on_unit_backward_done(__u, g))
                return None

            blk.register_forward_pre_hook(pre_hook)
        self._hooks_installed = True

    def _on_unit_backward_done(self, u: Unit, g: torch.Tensor):
        if self._last_microbatch and not u.reduced:
            self._reduce_unit(u)
        return None

    def set_last_microbatch(self, flag: bool) -> None:
        self._last_microbatch = flag

    # ------------------------------------------------------------------------------------------------
    def zero_grad(self) -> None:
        self.grad_all.zero_()
        for u in self.units:
            u.reduced = False
        self._norm_zeroed = False
        if hasattr(self.collectives, "begin_step"):
            self.collectives.begin_step()

    def _zero_norm_once(self) -> None:
        # a backend that accumulates the norm inside its reduce-scatter needs ctrl[0] cleared before the first unit
        if not getattr(self, "_norm_zeroed", False):
            self.ctrl[optim_ops.CTRL_NORM_SQ:optim_ops.CTRL_NORM_SQ + 1].zero_()
            self._norm_zeroed = True

    def _fold_autograd_grads(self, u: Unit) -> None:
        """Ops without a kernel path (the CPU configuration, PyTorch fall-backs) hand their weight gradients to autograd;
        move those into the flat fp32 buffer the kernels accumulate into."""
        for s_ in u.slots:
            g = s_.param.grad
            if g is not None:
                s_.param.main_grad.add_(g.to(torch.float32))
                s_.param.grad = None

    def _reduce_unit(self, u: Unit) -> None:
        self._fold_autograd_grads(u)
        self._zero_norm_once()
        if self.comm_stream is not None and self.shard_world > 1:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self.collectives.reduce_scatter_avg(u, self.shard_world)
        else:
            self.collectives.reduce_scatter_avg(u, self.shard_world)
        u.reduced = True

    @torch.no_grad()
    def step(self, lr: float, grad_scale: float = 1.0) -> None:
        """Reduce what is not reduced yet, form the global gradient norm, update, re-gather parameters."""
        tp_group = self.dims.group("tp")
        if tp_group is not None:
            # parameters replicated across the tensor-parallel group (norm weights, low-rank gate input) saw only a part
            # of the tokens / heads on each rank: sum their gradients before anything else
            for u in self.units:
                if u.reduced:
                    continue
                self._fold_autograd_grads(u)
                for s_ in u.slots:
                    if getattr(s_.param, "_tp_replicated", False):
                        dist.all_reduce(u.grad[s_.offset:s_.offset + s_.numel], group=tp_group)
        for u in self.units:
            if not u.reduced:
                self._reduce_unit(u)
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        if self.replica_reducer is not None:
            # fault-tolerant replica groups: average the (already sharded) gradients over the groups of this step's
            # quorum, then apply the update only if every group got through the step
            for u in self.units:
                self.replica_reducer(u.grad_shard if self.shard_world > 1 else u.grad)
        if self.commit_gate is not None and not self.commit_gate():
            self.voided_steps += 1
            return
        o = self.optim
        # a bounded device wait that ran out earlier in this step (a peer that never signalled, a stalled pipeline) left
        # the status word set: latch it on the device so that the update kernels below apply nothing
        optim_ops.latch_status(self.ctrl)
        if self._norm_scratch is None and self.device.type == "cuda":
            self._norm_scratch = torch.empty(2048, dtype=torch.float32, device=self.device)
        if not getattr(self.collectives, "norm_fused", False) or self.shard_world == 1:
            self.ctrl[optim_ops.CTRL_NORM_SQ] = 0
            for u in self.units:
                optim_ops.sumsq_accumulate(u.grad_shard if self.shard_world > 1 else self._local_slice(u.grad, u),
                                           self.ctrl[optim_ops.CTRL_NORM_SQ:optim_ops.CTRL_NORM_SQ + 1],
                                           self._norm_scratch, accumulate=True)
        if tp_group is not None:
            self._discount_replicated_norm()
        self._all_reduce_norm()
        if self.cpu_offload:
            self._offloaded_update(lr, grad_scale)
            optim_ops.adamw_finalize(self.ctrl, o.max_norm, o.skip_nan_inf, grad_scale)
            for u in self.units:
                self.collectives.all_gather_params(u, self.shard_world)
            return
        if getattr(self.collectives, "fused_optimizer", False) and self.shard_world > 1:
            for u in self.units:
                self.collectives.adamw_and_publish(u, lr, o, grad_scale)
            optim_ops.adamw_finalize(self.ctrl, o.max_norm, o.skip_nan_inf, grad_scale)
            self.collectives.publish_done()
            return
        for u in self.units:
            g = u.grad_shard if self.shard_world > 1 else u.grad
            lowp = u.compute_shard() if (self.param_dtype == torch.bfloat16 or self.device.type != "cuda") else None
            optim_ops.adamw_step(u.master, u.exp_avg, u.exp_avg_sq, g, lowp, self.ctrl, lr, o.beta1, o.beta2, o.eps,
                                 o.kernel_weight_decay, o.max_norm, o.skip_nan_inf, grad_scale)
            if lowp is None:
                u.compute_shard().copy_(u.master)
        optim_ops.adamw_finalize(self.ctrl, o.max_norm, o.skip_nan_inf, grad_scale)
        for u in self.units:
            self.collectives.all_gather_params(u, self.shard_world)

    def _offloaded_update(self, lr: float, grad_scale: float) -> None:
        """AdamW with host-resident state: unit i's state travels host -> staging set i % 2 on the copy stream while
        the update of unit i - 1 runs, and travels back as soon as its own update is done."""
        o = self.optim
        if not self._stage:
            n = max(u.shard_size for u in self.units)
            self._stage = [[torch.empty(n, dtype=torch.float32, device=self.device) for _ in range(3)] for _ in range(2)]
        main, copy = torch.cuda.current_stream(), self._copy_stream
        for i, u in enumerate(self.units):
            n, bufs = u.shard_size, self._stage[i % 2]
            host = (u.master, u.exp_avg, u.exp_avg_sq)
            with torch.cuda.stream(copy):
                if self._stage_free[i % 2] is not None:
                    copy.wait_event(self._stage_free[i % 2])  # the write-back that used this set has finished
                for b, h in zip(bufs, host):
                    b[:n].copy_(h, non_blocking=True)
                ready = copy.record_event()
            main.wait_event(ready)
            g = u.grad_shard if self.shard_world > 1 else u.grad
            lowp = u.compute_shard() if self.param_dtype == torch.bfloat16 else None
            optim_ops.adamw_step(bufs[0][:n], bufs[1][:n], bufs[2][:n], g, lowp, self.ctrl, lr, o.beta1, o.beta2, o.eps,
                                 o.kernel_weight_decay, o.max_norm, o.skip_nan_inf, grad_scale)
            if lowp is None:
                u.compute_shard().copy_(bufs[0][:n])
            done = main.record_event()
            with torch.cuda.stream(copy):
                copy.wait_event(done)
                for b, h in zip(bufs, host):
                    h.copy_(b[:n], non_blocking=True)
                self._stage_free[i % 2] = copy.record_event()
        main.wait_stream(copy)  # the host copies are complete before anything reads them (checkpoints, the next step)

    def _local_slice(self, t: torch.Tensor, u: Unit) -> torch.Tensor:
        return t

    def _discount_replicated_norm(self) -> None:
        """Every tensor-parallel rank holds the same gradient for replicated parameters; the sum over the tp group would
        count it tp times, so each rank contributes only 1/tp of it."""
        P = self.dims.tp
        rep = torch.zeros((), dtype=torch.float32, device=self.device)
        for u in self.units:
            a, b = u.shard_range if self.shard_world > 1 else (0, u.numel)
            g = u.grad_shard if self.shard_world > 1 else u.grad
            for s_ in u.slots:
                if not getattr(s_.param, "_tp_replicated", False):
                    continue
                lo, hi = max(a, s_.offset), min(b, s_.offset + s_.numel)
                if lo < hi:
                    rep = rep + g[lo - a:hi - a].float().pow(2).sum()
        self.ctrl[optim_ops.CTRL_NORM_SQ] -= rep * (P - 1) / P

    def _all_reduce_norm(self) -> None:
        sl = self.ctrl[optim_ops.CTRL_NORM_SQ:optim_ops.CTRL_NORM_SQ + 1]
        g = self.dims.group("dp_shard_cp")
        if g is not None:
            dist.all_reduce(sl, group=g)
        for name in ("tp", "pp"):
            grp = self.dims.group(name)
            if grp is not None:
                dist.all_reduce(sl, group=grp)

    # ---- replica-level fault tolerance ---------------------------------------------------------------------
    def replica_state_tensors(self) -> List[torch.Tensor]:
        """Everything a replica group that joins late must copy from an up-to-date one, in a fixed order."""
        out = [self.ctrl]
        for u in self.units:
            out += [u.master, u.exp_avg, u.exp_avg_sq]
        return out

    @torch.no_grad()
    def refresh_compute(self) -> None:
        """Rebuilds the low-precision parameters from the master weights (after ``replica_state_tensors`` changed)."""
        for u in self.units:
            u.compute_shard().copy_(u.master)
            self.collectives.all_gather_params(u, self.shard_world)

    def check_status(self, sync: bool = False) -> None:
        """Raises ``KernelError`` when a kernel of an earlier step recorded a wait that ran out.  Without ``sync`` this
        reads one pinned host word and never touches the stream; the step in which the wait failed applied no update
        (see ``step``), so the parameters are those of the last good step when this raises."""
        if self.device.type != "cuda":
            return
        from ..ops import _lib
        if _lib.available():
            _lib.assert_status_ok(sync=sync)

    def aborted_steps(self) -> int:
        return int(self.ctrl[optim_ops.CTRL_ABORTED])

    # ---- read-outs (host syncs: call only when logging) -------------------------------------------------
    def grad_norm(self) -> float:
        return float(self.ctrl[optim_ops.CTRL_NORM])

    def skipped_steps(self) -> int:
        return int(self.ctrl[optim_ops.CTRL_SKIPPED])

    def applied_steps(self) -> int:
        return int(self.ctrl[optim_ops.CTRL_STEP])

    # ---- state dicts -----------------------------------------------------------------------------------
    def _gather_flat(self, shard: torch.Tensor, u: Unit) -> torch.Tensor:
        if self.shard_world == 1:
            return shard
        if shard.device != self.device:
            shard = shard.to(self.device)  # offloaded optimizer state: gather through the device
        full = torch.empty(u.numel, dtype=shard.dtype, device=shard.device)
        g = self.dims.group("dp_shard_cp")
        if dist.get_backend(g) == "gloo":
            parts = [torch.empty_like(shard) for _ in range(self.shard_world)]
            dist.all_gather(parts, shard.contiguous(), group=g)
            torch.cat(parts, out=full)
        else:
            dist.all_gather_into_tensor(full, shard.contiguous(), group=g)
        return full

    def owns_unit(self, index: int) -> bool:
        """Checkpoint ownership: unit ``index`` is written by shard rank ``index % shard_world`` (of the first replica
        and, for tensors that tensor parallelism does not split, of tensor-parallel rank 0)."""
        if self.dims._ranks and self.dims.dp_replicate_enabled and self.dims.local_rank_in("dp_replicate") != 0:
            return False
        return index % self.shard_world == self.shard_rank

    @torch.no_grad()
    def full_state(self, kind: str = "master", partition: bool = False, to_host: bool = False,
                   dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
        """``{fqn: full tensor}`` for ``kind`` in master | exp_avg | exp_avg_sq.  Collective: every rank takes part in the
        gather of every unit (one unit at a time on the device).  With ``partition`` a rank keeps only the units it owns
        (``owns_unit``), so the copies that survive the call add up to ONE model over the whole job instead of one per
        rank; without it every rank gets everything."""
        out = {}
        tp_group = self.dims.group("tp")
        tp_rank = self.dims.local_rank_in("tp") if tp_group is not None else 0
        for i, u in enumerate(self.units):
            full = self._gather_flat(getattr(u, kind), u)
            mine = (not partition) or self.owns_unit(i)
            for s in u.slots:
                tp = getattr(s.param, "_tp", None)
                split = tp is not None and tp_group is not None
                if not mine and not split:
                    continue
                t = full[s.offset:s.offset + s.numel].view(s.shape)
                if split:
                    parts = [torch.empty_like(t) for _ in range(tp[2])]
                    dist.all_gather(parts, t.contiguous(), group=tp_group)
                    t = torch.cat(parts, dim=tp[0])
                if not mine or (partition and tp_rank != 0):
                    continue
                if dtype is not None:
                    t = t.to(dtype)
                out[s.fqn] = t.cpu() if to_host else t.clone()
            del full
        return out

    def unit_fqns(self) -> List[List[str]]:
        return [[s.fqn for s in u.slots] for u in self.units]

    def full_shape(self, s: ParamSlot) -> Tuple[int, ...]:
        """Shape of the parameter as a checkpoint holds it (tensor-parallel shards concatenated)."""
        tp = getattr(s.param, "_tp", None)
        if tp is None or self.dims.group("tp") is None:
            return tuple(s.shape)
        shp = list(s.shape)
        shp[tp[0]] *= tp[2]
        return tuple(shp)

    @torch.no_grad()
    def load_full_state(self, tensors: Dict[str, torch.Tensor], kind: str = "master", strict: bool = True,
                        units: Optional[List[Unit]] = None) -> None:
        """Inverse of ``full_state``: every rank passes the full tensors and keeps its slice (``units``: only these)."""
        for u in (units if units is not None else self.units):
            a, b = u.shard_range
            dst = getattr(u, kind)
            for s in u.slots:
                if s.fqn not in tensors:
                    if strict:
                        raise KeyError(f"missing {s.fqn} in checkpoint")
                    continue
                src_t = tensors[s.fqn]
                tp = getattr(s.param, "_tp", None)
                if tp is not None and src_t.shape[tp[0]] == s.shape[tp[0]] * tp[2]:
                    src_t = src_t.narrow(tp[0], tp[1] * s.shape[tp[0]], s.shape[tp[0]])
                src = src_t.reshape(-1).to(device=self.device, dtype=torch.float32)
                lo, hi = max(a, s.offset), min(b, s.offset + s.numel)
                if lo < hi:
                    dst[lo - a:hi - a].copy_(src[lo - s.offset:hi - s.offset])
                if kind == "master":
                    u.compute[s.offset:s.offset + s.numel].copy_(src)

    def named_slots(self) -> Iterable[Tuple[Unit, ParamSlot]]:
        for u in self.units:
            for s in u.slots:
                yield u, s

    def optimizer_scalars(self) -> Dict[str, float]:
        c = self.ctrl.detach().cpu().tolist()
        return {"step": c[optim_ops.CTRL_STEP], "skipped": c[optim_ops.CTRL_SKIPPED]}

    def load_optimizer_scalars(self, d: Dict[str, float]) -> None:
        self.ctrl[optim_ops.CTRL_STEP] = float(d.get("step", 0))
        self.ctrl[optim_ops.CTRL_SKIPPED] = float(d.get("skipped", 0))
