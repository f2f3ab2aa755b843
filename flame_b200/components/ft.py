"""Replica-level fault tolerance: quorum, managed gradient all-reduce, commit vote, live recovery.

The reference wraps torchft (torchtitan/components/ft/manager.py:32-168): every *replica group* is a training job of
its own (its own ``torchrun`` world, sharded inside with FSDP), a lighthouse decides per step which replica groups
take part, gradients are averaged across the participating groups through a process group that is rebuilt whenever
the membership changes, the optimizer step is applied only if every participant got through the step without an
error, and a group that (re)joins behind the others first copies the state of an up-to-date group.

This module provides the same roles without torchft:

* ``Lighthouse``: a thread next to a ``TCPStore`` server.  Replicas write heartbeats; once per step each replica
  files a request ``req/<round>/<id>`` carrying its committed step; the lighthouse answers with ``dec/<round>``:
  the sorted member list (every replica with a fresh heartbeat that asked in time, at least ``min_replicas``), the
  highest committed step and which member holds it.  One decision per round, read by all, so members never disagree.
  ``python -m flame_b200.components.ft --port P`` runs one standalone.
* ``FTManager`` (one per replica group, driven by the group's rank 0 and mirrored to its other ranks through the
  group's own default process group): ``start_step`` obtains the decision and rebuilds the cross-replica process
  group (gloo over a ``PrefixStore`` of the round, no default group involved) when the members changed;
  ``allreduce`` averages a tensor over the members and records a failure instead of raising; ``should_commit``
  is a MIN-vote over the members; ``recover`` broadcasts the up-to-date member's optimizer state to the others.

Failures are detected on the host: a replica that stops writing heartbeats drops out of the next decision, and a
collective that does not finish within ``timeout`` marks the step as failed (nothing is applied, the next step asks
for a new quorum).  A replica leaves only between steps.
"""
from __future__ import annotations

import argparse
import json
import threading
import time
from datetime import timedelta
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from .metrics import logger


class Lighthouse:
    """Decides the quorum of every round.  ``store`` must be the server side (or any client) of the shared TCPStore."""

    def __init__(self, store: dist.Store, group_size: int, min_replicas: int = 1, heartbeat_timeout: float = 2.0,
                 join_timeout: float = 1.0, poll: float = 0.01) -> None:
        self.store, self.n, self.min = store, group_size, max(1, min_replicas)
        self.hb_timeout, self.join_timeout, self.poll = heartbeat_timeout, join_timeout, poll
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.round = 0
        store.set("round", "0")

    def start(self) -> "Lighthouse":
        self._thread = threading.Thread(target=self._run, name="ft-lighthouse", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def _fresh(self, rid: int, now: float) -> bool:
        key = f"hb/{rid}"
        if not self.store.check([key]):
            return False
        return now - float(self.store.get(key).decode()) < self.hb_timeout

    def _run(self) -> None:
        first_request: Optional[float] = None
        while not self._stop.is_set():
            k = self.round
            now = time.time()
            asked: Dict[int, int] = {}
            for rid in range(self.n):
                key = f"req/{k}/{rid}"
                if self.store.check([key]):
                    asked[rid] = int(json.loads(self.store.get(key).decode())["step"])
            if asked and first_request is None:
                first_request = now
            live = {rid for rid in range(self.n) if self._fresh(rid, now)}
            members = sorted(r for r in asked if r in live)
            waiting_for = live - set(asked)
            timed_out = first_request is not None and now - first_request > self.join_timeout
            if len(members) >= self.min and (not waiting_for or timed_out):
                max_step = max(asked[r] for r in members)
                src = min(r for r in members if asked[r] == max_step)
                self.store.set(f"dec/{k}", json.dumps({"members": members, "steps": {str(r): asked[r] for r in members},
                                                       "max_step": max_step, "src": src}))
                self.round = k + 1
                self.store.set("round", str(self.round))
                first_request = None
                continue
            time.sleep(self.poll)


class FTManager:
    def __init__(self, store: dist.Store, replica_id: int, group_size: int, device: torch.device = torch.device("cpu"),
                 timeout: float = 10.0, heartbeat_interval: float = 0.1, local_group: Optional[dist.ProcessGroup] = None,
                 local_rank: int = 0, backend: str = "gloo", heartbeat_store: Optional[dist.Store] = None) -> None:
        # The heartbeat thread needs a connection of its own: a store client serialises its calls, so a main thread
        # blocked in ``wait`` for a decision would otherwise hold back the very heartbeats that keep it in the quorum.
        self.store, self.rid, self.n, self.device = store, replica_id, group_size, device
        self._hb_store = heartbeat_store if heartbeat_store is not None else store
        self.timeout, self.backend = timeout, backend
        self.local_group, self.local_rank = local_group, local_rank
        self.members: List[int] = []
        self.pg: Optional[dist.ProcessGroup] = None
        self.decision: Dict = {}
        self.errored = False
        self.quorum_id = -1
        self.reconfigurations = 0
        self._stop = threading.Event()
        self._hb: Optional[threading.Thread] = None
        if local_rank == 0:
            self._beat()
            self._hb = threading.Thread(target=self._heartbeat, args=(heartbeat_interval,), name="ft-heartbeat", daemon=True)
            self._hb.start()

    # ---- liveness ---------------------------------------------------------------------------------------------
    def _beat(self) -> None:
        self._hb_store.set(f"hb/{self.rid}", repr(time.time()))

    def _heartbeat(self, interval: float) -> None:
        while not self._stop.wait(interval):
            try:
                self._beat()
            except Exception:  # the store went away: nothing left to report to
                return

    def shutdown(self) -> None:
        """Leaves the job between steps: heartbeats stop, the next decision is taken without this replica."""
        self._stop.set()
        if self._hb is not None:
            self._hb.join(timeout=2)
        self.pg = None

    # ---- quorum -----------------------------------------------------------------------------------------------
    def _ask(self, step: int) -> Dict:
        deadline = time.time() + self.timeout
        while True:
            k = int(self.store.get("round").decode())
            self.store.set(f"req/{k}/{self.rid}", json.dumps({"step": step}))
            left = max(0.05, deadline - time.time())
            self.store.wait([f"dec/{k}"], timedelta(seconds=left))
            dec = json.loads(self.store.get(f"dec/{k}").decode())
            dec["round"] = k
            if self.rid in dec["members"]:
                return dec
            if time.time() > deadline:
                raise TimeoutError(f"replica {self.rid} was not admitted to a quorum within {self.timeout}s")

    def start_step(self, step: int) -> Dict:
        """Quorum for this step attempt; ``step`` is the number of steps this replica has committed.  Returns the
        decision (``members``, ``max_step``, ``src``, ``heal``: whether this replica must recover first)."""
        self.errored = False
        if self.local_rank == 0:
            dec = self._ask(step)
            payload = [dec]
        else:
            payload = [None]
        if self.local_group is not None:
            dist.broadcast_object_list(payload, src=dist.get_global_rank(self.local_group, 0), group=self.local_group)
        dec = payload[0]
        if dec["members"] != self.members:
            self._reconfigure(dec)
        self.decision = dec
        dec["heal"] = dec["steps"][str(self.rid)] < dec["max_step"]
        return dec

    def _reconfigure(self, dec: Dict) -> None:
        members = dec["members"]
        self.members, self.quorum_id = list(members), dec["round"]
        self.reconfigurations += 1
        self.pg = None
        if len(members) > 1:
            prefix = dist.PrefixStore(f"pg/{dec['round']}/{self.local_rank}", self.store)
            rank = members.index(self.rid)
            if self.backend == "gloo":
                self.pg = dist.ProcessGroupGloo(prefix, rank, len(members), timedelta(seconds=self.timeout))
            else:
                opts = dist.ProcessGroupNCCL.Options()
                opts._timeout = timedelta(seconds=self.timeout)
                self.pg = dist.ProcessGroupNCCL(prefix, rank, len(members), opts)
        logger.info(f"fault tolerance: replica {self.rid} joins quorum {dec['round']} with members {members}")

    def num_participants(self) -> int:
        return max(1, len(self.members))

    # ---- managed collectives ----------------------------------------------------------------------------------
    def _run(self, fn: Callable[[], "dist.Work"]) -> bool:
        if self.errored:
            return False
        try:
            work = fn()
            ok = work.wait(timedelta(seconds=self.timeout))
            if ok is False:
                raise RuntimeError("collective reported failure")
            return True
        except Exception as e:  # a member died or timed out: the step is void, the next quorum sorts it out
            logger.warning(f"fault tolerance: cross-replica collective failed on replica {self.rid}: {e}")
            self.errored = True
            self.pg = None
            self.members = []  # forces a new process group at the next quorum, whoever is in it
            return False

    def allreduce(self, t: torch.Tensor) -> None:
        """In-place average over the participating replicas; on failure the tensor is left as it is and the step is
        marked as failed."""
        if self.pg is None:
            return
        staged = t if (self.backend != "gloo" or not t.is_cuda) else t.detach().to("cpu")
        opts = dist.AllreduceOptions()
        opts.reduceOp = dist.ReduceOp.SUM
        if self._run(lambda: self.pg.allreduce([staged], opts)):
            staged.div_(len(self.members))
            if staged is not t:
                t.copy_(staged)

    def should_commit(self, local_ok: bool = True) -> bool:
        """True only if every member finished the step without an error (a MIN vote over the members)."""
        vote = torch.tensor([1 if (local_ok and not self.errored) else 0], dtype=torch.int32)
        if self.pg is not None and not self.errored:
            opts = dist.AllreduceOptions()
            opts.reduceOp = dist.ReduceOp.MIN
            v = vote if self.backend == "gloo" else vote.to(self.device)
            if self._run(lambda: self.pg.allreduce([v], opts)):
                vote = v.cpu()
            else:
                vote.zero_()
        elif self.errored:
            vote.zero_()
        return self._local_verdict(bool(vote.item()))

    def _local_verdict(self, ok: bool) -> bool:
        """One decision per replica group: every local rank runs its own cross-replica process group, so one rank's
        collective can fail while another's succeeds.  A MIN over the group's ranks makes them all commit, or all void
        the step (and all rebuild their cross-replica group at the next quorum), so the sharded update and the
        collectives inside the group never run on a part of the ranks only."""
        if self.local_group is None or dist.get_world_size(self.local_group) == 1:
            return ok
        v = torch.tensor([1 if ok else 0], dtype=torch.int32,
                         device=self.device if dist.get_backend(self.local_group) == "nccl" else "cpu")
        dist.all_reduce(v, op=dist.ReduceOp.MIN, group=self.local_group)
        agreed = bool(v.item())
        if not agreed and not self.errored:
            self.errored = True
            self.pg = None
            self.members = []
        return agreed

    def recover(self, tensors: List[torch.Tensor]) -> bool:
        """Copies ``tensors`` (same list, same order on every member) from the decision's up-to-date member to every
        member; called by all members of a quorum in which at least one is behind."""
        if self.pg is None:
            return self._local_verdict(not self.errored)
        root = self.members.index(self.decision["src"])
        ok = True
        for t in tensors:
            staged = t if (self.backend != "gloo" or not t.is_cuda) else t.detach().to("cpu")
            opts = dist.BroadcastOptions()
            opts.rootRank = root
            opts.rootTensor = 0
            if not self._run(lambda: self.pg.broadcast([staged], opts)):
                ok = False
                break
            if staged is not t:
                t.copy_(staged)
        # all ranks of the group recovered, or none continues as if it had
        return self._local_verdict(ok)


class SemiSync:
    """Semi-synchronous training over replica groups: LocalSGD and DiLoCo (the modes torchtitan reaches through
    ``maybe_semi_sync_training``, torchtitan/components/ft/manager.py:120-168).

    Between synchronisations every replica group trains on its own (no per-step gradient averaging across groups).
    Every ``sync_steps`` optimizer steps:

    * ``local_sgd``: the fp32 master weights are averaged over the groups;
    * ``diloco``: the pseudo-gradient ``outer - master`` (what the inner steps changed since the last synchronisation)
      is averaged over the groups and applied to the outer weights by SGD with (Nesterov) momentum; the inner weights
      restart from the new outer weights.

    ``allreduce`` is the in-place averaging collective of the replica layer (``FTManager.allreduce``); ``failed`` tells
    whether it failed since ``begin``.  A failed synchronisation changes nothing: LocalSGD simply keeps training and
    tries again at the next interval, DiLoCo falls back to the last outer weights, which every group still holds."""

    def __init__(self, engine, method: str, sync_steps: int, allreduce: Callable[[torch.Tensor], None],
                 failed: Callable[[], bool] = lambda: False, outer_lr: float = 0.7, outer_momentum: float = 0.9,
                 nesterov: bool = True) -> None:
        if method not in ("local_sgd", "diloco"):
            raise ValueError(f"unknown semi-synchronous method {method!r} (local_sgd | diloco)")
        if sync_steps < 1:
            raise ValueError("sync_steps must be at least 1")
        self.engine, self.method, self.sync_steps = engine, method, sync_steps
        self.allreduce, self.failed = allreduce, failed
        self.outer_lr, self.mu, self.nesterov = outer_lr, outer_momentum, nesterov
        self.local_steps = 0
        self.syncs = 0
        self.outer: List[torch.Tensor] = []
        self.momentum: List[torch.Tensor] = []
        if method == "diloco":
            self.outer = [u.master.detach().clone() for u in engine.units]
            self.momentum = [torch.zeros_like(u.master) for u in engine.units]

    @torch.no_grad()
    def after_step(self) -> bool:
        """Call after every applied optimizer step; returns True when a synchronisation was carried out."""
        self.local_steps += 1
        if self.local_steps < self.sync_steps:
            return False
        self.local_steps = 0
        units = self.engine.units
        if self.method == "local_sgd":
            avg = [u.master.detach().clone() for u in units]
            for t in avg:
                self.allreduce(t)
            if self.failed():
                return False
            for u, t in zip(units, avg):
                u.master.copy_(t)
        else:
            pseudo = [o - u.master for o, u in zip(self.outer, units)]
            for t in pseudo:
                self.allreduce(t)
            if self.failed():
                for u, o in zip(units, self.outer):   # back to the last weights all groups agree on
                    u.master.copy_(o)
                self.engine.refresh_compute()
                return False
            for o, m, g, u in zip(self.outer, self.momentum, pseudo, units):
                m.mul_(self.mu).add_(g)
                step = g.add(m, alpha=self.mu) if self.nesterov else m
                o.add_(step, alpha=-self.outer_lr)
                u.master.copy_(o)
        self.engine.refresh_compute()
        self.syncs += 1
        return True


def connect(addr: str, replica_id: int, timeout: float = 30.0) -> dist.Store:
    """Client connection to the lighthouse's store at ``host:port``."""
    host, port = addr.rsplit(":", 1)
    return dist.TCPStore(host, int(port), is_master=False, timeout=timedelta(seconds=timeout), wait_for_workers=False)


def main() -> None:
    ap = argparse.ArgumentParser(description="Standalone fault-tolerance lighthouse (TCPStore server + quorum thread)")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=29510)
    ap.add_argument("--group-size", type=int, required=True)
    ap.add_argument("--min-replicas", type=int, default=1)
    ap.add_argument("--heartbeat-timeout", type=float, default=5.0)
    ap.add_argument("--join-timeout", type=float, default=5.0)
    args = ap.parse_args()
    store = dist.TCPStore(args.host, args.port, is_master=True, wait_for_workers=False)
    Lighthouse(store, args.group_size, args.min_replicas, args.heartbeat_timeout, args.join_timeout).start()
    logger.info(f"lighthouse listening on {args.host}:{args.port} for {args.group_size} replica groups")
    while True:
        time.sleep(3600)


if __name__ == "__main__":
    main()
