"""Peer-memory collectives for the sharded engine (``csrc/comm.cu``).

The flat gradient buffer, the flat parameter buffer and a small flag array are allocated in symmetric memory
(``torch.distributed._symmetric_memory`` does the allocation and the handle exchange); after the rendezvous every
rank holds device pointers to every peer's copies and the kernels move data with plain loads and stores over
NVLink:

* reduce-scatter = each rank *pulls* its slice from all peers in rank order and averages (deterministic), emitting
  the slice's sum of squares for the gradient norm in the same pass;
* all-gather = the AdamW kernel *pushes* its updated bf16 slice into every peer's parameter buffer.

Cross-rank ordering uses one flag word per (unit, source rank) carrying the step number, written with
release/system scope and polled with a bound (``_lib.set_peer_wait_seconds``; the trainer uses the start-up timeout for
the first step and the training timeout afterwards).  A wait that runs out sets the library status word; the engine
latches that word into the optimizer's control vector before the update kernels, which then apply nothing, and
``ShardedEngine.check_status`` raises on the host at the next step boundary instead of training on partial sums.
"""
from __future__ import annotations

from ctypes import c_double, c_float, c_int, c_longlong, c_void_p
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib, optim as optim_ops
from .dims import ParallelDims
from .engine import Collectives, Unit

vp, i32, i64, f32, f64 = c_void_p, c_int, c_longlong, c_float, c_double
_lib.register("fb_peer_max_ranks", [])
_lib.register("fb_peer_rs_parts", [])
_lib.register("fb_peer_signal", [vp, i32, i32, i32, i32, vp])
_lib.register("fb_peer_wait", [vp, i32, i32, i32, f64, vp])
_lib.register("fb_peer_reduce_scatter", [vp, i32, i64, i64, vp, vp, vp, vp])
_lib.register("fb_peer_adamw_push", [vp, vp, vp, vp, vp, i32, i64, i64, f32, f32, f32, f32, f32, f32, i32, vp, f32, vp])
_lib.register("fb_peer_reduce_scatter_acc", [vp, i32, i64, i64, vp, vp, vp, i32, vp])
_lib.register("fb_peer_gather_flat", [vp, i32, i64, vp, i64, i64, vp])



class PeerCollectives(Collectives):
    fused_optimizer = True  # the engine hands the AdamW step to ``adamw_and_publish``

    def __init__(self, dims: ParallelDims, device: torch.device) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        self.symm_mem = symm_mem
        self.dims, self.device = dims, device
        self.group = dims.group("dp_shard_cp")
        assert self.group is not None, "peer collectives need a shard group of at least two ranks"
        # HSDP: the shard group reduces over peer memory, the slices are then averaged over the replicate group (NCCL);
        # the gradient norm can no longer be taken inside the reduce-scatter kernel, it is formed from the averaged slices
        self.replicate_group = dims.group("dp_replicate") if dims.dp_replicate_enabled else None
        self.norm_fused = self.replicate_group is None
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        L = _lib.lib()
        self.max_ranks = int(L.fb_peer_max_ranks())
        if self.world > self.max_ranks:
            raise RuntimeError(f"peer collectives support up to {self.max_ranks} ranks")
        self._handles: Dict[str, object] = {}
        self._tensors: Dict[str, torch.Tensor] = {}
        self._ptr_arrays: Dict[str, torch.Tensor] = {}
        self.nslots = 0
        self.epoch = 0
        self.engine = None
        self._partials = torch.empty(int(L.fb_peer_rs_parts()), dtype=torch.float32, device=device)

    # ---- allocation -----------------------------------------------------------------------------------
    def allocate(self, n: int, dtype: torch.dtype, tag: str) -> torch.Tensor:
        t = self.symm_mem.empty(n, dtype=dtype, device=self.device)
        t.zero_()
        h = self.symm_mem.rendezvous(t, self.group)
        self._handles[tag], self._tensors[tag] = h, t
        ptrs = [int(p) for p in h.buffer_ptrs]
        self._ptr_arrays[tag] = (torch.tensor(ptrs, dtype=torch.int64).numpy().astype("uint64"), ptrs)
        return t

    def attach(self, engine) -> None:
        """Called once the engine's units exist: allocates the flag array (one slot per unit + one for parameters)."""
        self.engine = engine
        nu = len(engine.units)
        # slots: [0, nu) "gradients of unit i are final", nu "parameters written", (nu, 2 nu] "done pulling unit i"
        self.nslots = 2 * nu + 1
        flags = self.allocate(self.nslots * self.max_ranks, torch.int32, "flags")
        self.flags = flags
        self.unit_slot = {id(u): i for i, u in enumerate(engine.units)}
        self.param_slot = nu
        self.pulled_slot = {id(u): nu + 1 + i for i, u in enumerate(engine.units)}
        self._param_version = 0
        self._param_waited = 0
        self._unit_shard_ptrs: Dict[int, object] = {}
        torch.cuda.synchronize()
        dist.barrier(group=self.group, device_ids=[self.device.index])

    def _ptrs(self, tag: str) -> int:
        return self._ptr_arrays[tag][0].ctypes.data

    # ---- step protocol ----------------------------------------------------------------------------------
    def begin_step(self) -> None:
        self.epoch += 1

    def reduce_scatter_avg(self, unit: Unit, world: int, accumulate: bool = False, want_norm: bool = True) -> None:
        """Runs on the current stream: signal "unit gradients final", wait for all peers, pull + average."""
        L = _lib.lib()
        st = _lib.stream_ptr()
        slot = self.unit_slot[id(unit)]
        eng = self.engine
        sharded = getattr(eng, "resharding", False)
        seq = unit.rs_seq if sharded else self.epoch
        _lib.check(L.fb_peer_signal(self._ptrs("flags"), self.world, self.rank, slot, seq, st), "fb_peer_signal")
        _lib.check(L.fb_peer_wait(self.flags.data_ptr(), self.world, slot, seq, _lib.peer_wait_seconds(), st), "fb_peer_wait")
        if sharded:
            # the full gradients of the unit sit in a recycled staging buffer (same buffer, same offset on every rank)
            tag = "gbuf_root" if unit.name == "root" else f"gbuf{unit.buf}"
            off = self.rank * unit.shard_size
        else:
            tag, off = "grad", unit.base + self.rank * unit.shard_size
        norm_ptr = eng.ctrl[optim_ops.CTRL_NORM_SQ:].data_ptr() if (want_norm and self.norm_fused) else 0
        rc = L.fb_peer_reduce_scatter_acc(self._ptrs(tag), self.world, off, unit.shard_size, unit.grad_shard.data_ptr(),
                                          self._partials.data_ptr(), norm_ptr, 1 if accumulate else 0, st)
        _lib.check(rc, "fb_peer_reduce_scatter")
        _lib.count_launch(4)
        if self.replicate_group is not None:
            dist.all_reduce(unit.grad_shard, group=self.replicate_group)
            unit.grad_shard.div_(dist.get_world_size(self.replicate_group))
        if sharded:
            # this rank no longer reads the peers' buffers for this unit: they may recycle them
            _lib.check(L.fb_peer_signal(self._ptrs("flags"), self.world, self.rank, self.pulled_slot[id(unit)], seq, st),
                       "fb_peer_signal")
            _lib.count_launch()

    # ---- sharded-parameter mode (parallel/resharding.py) -------------------------------------------------------
    can_fuse_gather = True

    def wait_pulled(self, unit: Unit) -> None:
        """Current stream waits (bounded) until every peer finished pulling ``unit``'s gradients out of this rank."""
        _lib.check(_lib.lib().fb_peer_wait(self.flags.data_ptr(), self.world, self.pulled_slot[id(unit)], unit.rs_seq,
                                           _lib.peer_wait_seconds(), _lib.stream_ptr()), "fb_peer_wait")
        _lib.count_launch()

    def params_written(self, version: int) -> None:
        """This rank's bf16 shards hold parameter version ``version`` (stream-ordered after the optimizer kernels)."""
        self._param_version = version
        _lib.check(_lib.lib().fb_peer_signal(self._ptrs("flags"), self.world, self.rank, self.param_slot, version,
                                             _lib.stream_ptr()), "fb_peer_signal")
        _lib.count_launch()

    def _await_params(self) -> None:
        if self._param_waited < self._param_version:
            _lib.check(_lib.lib().fb_peer_wait(self.flags.data_ptr(), self.world, self.param_slot, self._param_version,
                                               _lib.peer_wait_seconds(), _lib.stream_ptr()), "fb_peer_wait")
            _lib.count_launch()
            self._param_waited = self._param_version

    def _shard_ptrs(self, unit: Unit):
        arr = self._unit_shard_ptrs.get(id(unit))
        if arr is None:
            import numpy as np
            esz = unit.pshard.element_size()
            arr = np.array([p + unit.sbase * esz for p in self._ptr_arrays["pshard"][1]], dtype=np.uint64)
            self._unit_shard_ptrs[id(unit)] = arr
        return arr

    def gather_params(self, unit: Unit, lo: int, hi: int) -> None:
        """Bytes [lo, hi) of the unit's flat parameter buffer <- the ranks' shards, stand-alone kernel."""
        self._await_params()
        ptrs = self._shard_ptrs(unit)
        rc = _lib.lib().fb_peer_gather_flat(ptrs.ctypes.data, self.world, unit.shard_size * unit.pshard.element_size(),
                                            unit.compute.data_ptr(), lo, hi, _lib.stream_ptr())
        _lib.check(rc, "fb_peer_gather_flat")
        _lib.count_launch()

    def make_pending(self, unit: Unit, lo: int, hi: int, flags: torch.Tensor, epoch: int):
        from ..ops.gemm import PendingGather
        from .resharding import CHUNK_SHIFT
        self._await_params()
        return PendingGather(unit, unit.compute.data_ptr(), lo, hi, self._shard_ptrs(unit), self.world, self.rank,
                             unit.shard_size * unit.pshard.element_size(), CHUNK_SHIFT, flags, epoch,
                             self.engine._flush_pending)

    # norm_fused (set in __init__): the reduce-scatter already accumulated the slice's sum of squares into ctrl[0]

    def adamw_and_publish(self, unit: Unit, lr: float, o, grad_scale: float) -> None:
        L = _lib.lib()
        off = unit.base + self.rank * unit.shard_size
        rc = L.fb_peer_adamw_push(unit.master.data_ptr(), unit.exp_avg.data_ptr(), unit.exp_avg_sq.data_ptr(),
                                  unit.grad_shard.data_ptr(), self._ptrs("compute"), self.world, off, unit.shard_size,
                                  lr, o.beta1, o.beta2, o.eps, o.kernel_weight_decay, o.max_norm, 1 if o.skip_nan_inf else 0,
                                  self.engine.ctrl.data_ptr(), grad_scale, _lib.stream_ptr())
        _lib.check(rc, "fb_peer_adamw_push")
        _lib.count_launch()

    def publish_done(self) -> None:
        """All units pushed: tell the peers, and wait until every peer's pushes into this rank have landed."""
        L = _lib.lib()
        st = _lib.stream_ptr()
        _lib.check(L.fb_peer_signal(self._ptrs("flags"), self.world, self.rank, self.param_slot, self.epoch, st), "fb_peer_signal")
        _lib.check(L.fb_peer_wait(self.flags.data_ptr(), self.world, self.param_slot, self.epoch, _lib.peer_wait_seconds(), st), "fb_peer_wait")
        _lib.count_launch(2)

    def all_gather_params(self, unit: Unit, world: int) -> None:
        return  # done by adamw_and_publish

    def gather_params_now(self, unit: Unit, world: int) -> None:
        """Outside the optimizer step (after a replica group copied its state from another one) nothing has pushed the
        slices to the peers, so the compute buffers are completed with a plain c10d all-gather."""
        dist.all_gather_into_tensor(unit.compute, unit.compute_shard().clone(), group=self.group)
