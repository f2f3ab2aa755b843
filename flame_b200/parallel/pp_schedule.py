"""Pipeline schedules as data: who runs which (stage, micro-batch) forward or backward, in what order.

The reference picks a torch ``PipelineSchedule`` class by name, or loads a CSV of per-rank actions
(torchtitan/distributed/pipeline_parallel.py:36-123 ``build_pipeline_schedule``, ``stage_ids_this_rank``).  Here a
schedule is a plain list of ``Action`` per pipeline rank, produced by ``build_schedule`` (GPipe, 1F1B,
Interleaved1F1B, LoopedBFS) or ``parse_schedule_csv``; ``simulate`` replays it with unit-time actions, which both
validates it (every input is produced before it is consumed, nothing deadlocks) and yields the tick at which each
boundary tensor comes into being.  ``pair_message_order`` sorts the tensors that cross each pair of ranks by that
tick: the executor in ``pipeline.py`` posts its sends and receives per peer in exactly this order on both sides, so
point-to-point channels that match messages first-in-first-out (NCCL, gloo) can neither mismatch nor deadlock,
whatever the interleaving of forward and backward traffic.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

F, B = "F", "B"


@dataclass(frozen=True)
class Action:
    op: str      # "F" forward, "B" backward (input and weight gradients together)
    stage: int   # global stage index, 0 .. n_stages - 1
    mb: int      # micro-batch index

    def __str__(self) -> str:
        return f"{self.stage}{self.op}{self.mb}"


Schedule = List[List[Action]]
SINGLE_STAGE = ("gpipe", "1f1b")
MULTI_STAGE = ("interleaved1f1b", "loopedbfs")


def stage_ids_this_rank(rank: int, pp: int, n_stages: int, style: str = "loop") -> Tuple[int, ...]:
    """Stages of one rank: ``loop`` deals stages round-robin (rank r gets r, r + pp, ...), ``v`` folds them back so
    that rank r gets r and n_stages - 1 - r (two stages per rank), as torchtitan's helper of the same name does."""
    if n_stages % pp:
        raise ValueError(f"{n_stages} stages do not divide over {pp} pipeline ranks")
    per = n_stages // pp
    if style == "loop":
        return tuple(rank + k * pp for k in range(per))
    if style == "v":
        if per != 2:
            raise ValueError("the V style needs exactly two stages per rank")
        return (rank, n_stages - 1 - rank)
    raise ValueError(f"unknown stage placement {style!r}")


def stage_owners(pp: int, n_stages: int, style: str = "loop") -> List[int]:
    owner = [0] * n_stages
    for r in range(pp):
        for s in stage_ids_this_rank(r, pp, n_stages, style):
            owner[s] = r
    return owner


def build_schedule(name: str, pp: int, n_stages: int, n_mb: int, style: str = "loop") -> Schedule:
    """Per-rank action lists for a named schedule.  Names are case-insensitive and follow torch's classes:
    ``GPipe``, ``1F1B`` (one stage per rank), ``Interleaved1F1B``, ``LoopedBFS`` (several stages per rank)."""
    key = name.lower()
    if key in SINGLE_STAGE and n_stages != pp:
        raise ValueError(f"schedule {name} runs one stage per rank, got {n_stages} stages on {pp} ranks")
    out: Schedule = []
    for r in range(pp):
        stages = stage_ids_this_rank(r, pp, n_stages, style)
        acts: List[Action] = []
        if key == "gpipe":
            acts += [Action(F, r, m) for m in range(n_mb)]
            acts += [Action(B, r, m) for m in range(n_mb)]
        elif key == "1f1b":
            warm = min(n_mb, pp - r - 1)
            acts += [Action(F, r, m) for m in range(warm)]
            for k in range(n_mb - warm):
                acts.append(Action(F, r, warm + k))
                acts.append(Action(B, r, k))
            acts += [Action(B, r, m) for m in range(n_mb - warm, n_mb)]
        elif key == "loopedbfs":
            for s in stages:
                acts += [Action(F, s, m) for m in range(n_mb)]
            for s in reversed(stages):
                acts += [Action(B, s, m) for m in range(n_mb)]
        elif key == "interleaved1f1b":
            if style != "loop":
                raise ValueError("Interleaved1F1B places stages round-robin")
            if n_mb % pp:
                raise ValueError(f"Interleaved1F1B needs a micro-batch count that is a multiple of {pp}, got {n_mb}")
            V = len(stages)
            total = n_mb * V

            def fwd(k: int) -> Action:
                return Action(F, stages[(k // pp) % V], (k // (pp * V)) * pp + k % pp)

            def bwd(k: int) -> Action:
                return Action(B, stages[V - 1 - (k // pp) % V], (k // (pp * V)) * pp + k % pp)

            warm = min(total, (pp - r - 1) * 2 + (V - 1) * pp)
            acts += [fwd(k) for k in range(warm)]
            for k in range(total - warm):
                acts.append(fwd(warm + k))
                acts.append(bwd(k))
            acts += [bwd(k) for k in range(total - warm, total)]
        else:
            raise ValueError(f"unknown pipeline schedule {name!r}; known: GPipe, 1F1B, Interleaved1F1B, LoopedBFS, or a CSV")
        out.append(acts)
    return out


_CELL = re.compile(r"^(\d+)([A-Za-z_]+)(\d+)$")


def parse_schedule_csv(text: str) -> Schedule:
    """One line per pipeline rank, comma-separated cells ``<stage><op><micro-batch>`` as written by torch's schedule
    dumps: ``F`` forward, ``B`` full backward; a split backward (``I`` input gradient then ``W`` weight gradient) is
    run as one backward at the ``I`` cell.  Empty cells (bubbles) are skipped; communication cells are rejected, the
    executor derives communication itself."""
    sched: Schedule = []
    for line in text.strip().splitlines():
        acts: List[Action] = []
        for cell in line.strip().split(","):
            cell = cell.strip()
            if not cell:
                continue
            m = _CELL.match(cell)
            if not m:
                raise ValueError(f"cannot parse schedule cell {cell!r}")
            stage, op, mb = int(m.group(1)), m.group(2).upper(), int(m.group(3))
            if op == "F":
                acts.append(Action(F, stage, mb))
            elif op in ("B", "I"):
                acts.append(Action(B, stage, mb))
            elif op == "W":
                continue
            else:
                raise ValueError(f"schedule cell {cell!r}: only compute actions (F, B, I, W) are accepted")
        sched.append(acts)
    return sched


def format_schedule_csv(sched: Schedule) -> str:
    return "\n".join(",".join(str(a) for a in acts) for acts in sched) + "\n"


def infer_layout(sched: Schedule) -> Tuple[int, List[int]]:
    """(number of stages, owner rank of each stage) of a schedule; every stage must live on exactly one rank."""
    owner: Dict[int, int] = {}
    for r, acts in enumerate(sched):
        for a in acts:
            if owner.setdefault(a.stage, r) != r:
                raise ValueError(f"stage {a.stage} appears on ranks {owner[a.stage]} and {r}")
    n = max(owner) + 1 if owner else 0
    if sorted(owner) != list(range(n)):
        raise ValueError(f"stages are not 0..{n - 1}: {sorted(owner)}")
    return n, [owner[s] for s in range(n)]


def simulate(sched: Schedule, n_stages: int, n_mb: int) -> Dict[Action, int]:
    """Finish tick of every action under unit durations; raises ``ValueError`` if an action is missing or repeated,
    or if the ranks end up waiting for one another."""
    want = {Action(op, s, m) for op in (F, B) for s in range(n_stages) for m in range(n_mb)}
    have = [a for acts in sched for a in acts]
    if len(have) != len(set(have)) or set(have) != want:
        missing, extra = want - set(have), set(have) - want
        raise ValueError(f"schedule does not run every (stage, micro-batch) exactly once forward and backward: "
                         f"missing {sorted(map(str, missing))[:4]}, unexpected {sorted(map(str, extra))[:4]}, "
                         f"{len(have) - len(set(have))} repeated")

    def deps(a: Action) -> List[Action]:
        if a.op == F:
            return [Action(F, a.stage - 1, a.mb)] if a.stage > 0 else []
        d = [Action(F, a.stage, a.mb)]
        if a.stage < n_stages - 1:
            d.append(Action(B, a.stage + 1, a.mb))
        return d

    done: Dict[Action, int] = {}
    ptr = [0] * len(sched)
    free_at = [0] * len(sched)
    remaining = len(have)
    while remaining:
        progressed = False
        for r, acts in enumerate(sched):
            while ptr[r] < len(acts):
                a = acts[ptr[r]]
                ds = deps(a)
                if any(d not in done for d in ds):
                    break
                start = max([free_at[r]] + [done[d] for d in ds])
                done[a] = start + 1
                free_at[r] = start + 1
                ptr[r] += 1
                remaining -= 1
                progressed = True
        if not progressed:
            stuck = [str(acts[ptr[r]]) for r, acts in enumerate(sched) if ptr[r] < len(acts)]
            raise ValueError(f"schedule deadlocks: ranks wait at {stuck}")
    return done


@dataclass(frozen=True)
class Message:
    kind: str   # "A" activation entering `stage`, "G" gradient of the output of `stage`
    stage: int  # the consuming stage
    mb: int
    src: int
    dst: int


def pair_message_order(sched: Schedule, owner: Sequence[int], n_mb: int) -> Dict[Tuple[int, int], List[Message]]:
    """For every unordered pair of ranks (lo, hi): the boundary tensors that cross between them, both directions, in
    the order in which both sides must post them."""
    n_stages = len(owner)
    ticks = simulate(sched, n_stages, n_mb)
    pairs: Dict[Tuple[int, int], List[Tuple[int, int, str, int, int, Message]]] = {}
    for s in range(n_stages):
        for m in range(n_mb):
            if s > 0 and owner[s - 1] != owner[s]:
                msg = Message("A", s, m, owner[s - 1], owner[s])
                t = ticks[Action(F, s - 1, m)]
                pairs.setdefault((min(msg.src, msg.dst), max(msg.src, msg.dst)), []).append((t, msg.src, "A", s, m, msg))
            if s < n_stages - 1 and owner[s + 1] != owner[s]:
                msg = Message("G", s, m, owner[s + 1], owner[s])
                t = ticks[Action(B, s + 1, m)]
                pairs.setdefault((min(msg.src, msg.dst), max(msg.src, msg.dst)), []).append((t, msg.src, "G", s, m, msg))
    return {k: [x[-1] for x in sorted(v, key=lambda x: x[:-1])] for k, v in pairs.items()}


def bubble_fraction(sched: Schedule, n_stages: int, n_mb: int) -> float:
    """Idle share of the pipeline under unit-time actions (for logging and tests)."""
    ticks = simulate(sched, n_stages, n_mb)
    span = max(ticks.values())
    busy = sum(len(a) for a in sched)
    return 1.0 - busy / (span * len(sched))


def resolve(name: Optional[str], csv_path: Optional[str], pp: int, n_mb: Optional[int], n_layers: int,
            layers_per_stage: Optional[int] = None) -> Tuple[Schedule, int, List[int], str]:
    """(schedule, n_stages, stage owners, resolved name) from the job's flags, mirroring the reference's builder: a
    CSV wins over the name; multi-stage schedules get two stages per rank unless ``layers_per_stage`` says otherwise;
    when Interleaved1F1B does not fit the micro-batch count the looped breadth-first schedule is used instead."""
    if csv_path:
        with open(csv_path) as fh:
            sched = parse_schedule_csv(fh.read())
        if len(sched) != pp:
            raise ValueError(f"{csv_path}: {len(sched)} rows for {pp} pipeline ranks")
        n_stages, owner = infer_layout(sched)
        csv_mb = max(a.mb for acts in sched for a in acts) + 1
        if n_mb is None:
            n_mb = csv_mb
        if csv_mb != n_mb:
            raise ValueError(f"{csv_path} is written for {csv_mb} micro-batches, the step has {n_mb}")
        simulate(sched, n_stages, n_mb)
        return sched, n_stages, owner, "csv"
    key = (name or "1F1B").lower()
    if n_mb is None:
        n_mb = pp
    if key in SINGLE_STAGE:
        n_stages = pp
    elif key in MULTI_STAGE:
        per = 2
        if layers_per_stage:
            per = max(1, -(-n_layers // layers_per_stage) // pp)
        n_stages = pp * per
        while n_stages > pp and n_stages > n_layers:
            n_stages -= pp
        if key == "interleaved1f1b" and n_mb % pp:
            key = "loopedbfs"
    else:
        raise ValueError(f"unknown pipeline schedule {name!r}; known: GPipe, 1F1B, Interleaved1F1B, LoopedBFS, or a CSV")
    sched = build_schedule(key, pp, n_stages, n_mb)
    return sched, n_stages, stage_owners(pp, n_stages), key
