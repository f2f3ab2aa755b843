"""Pipeline schedules: builders, CSV round trip, the unit-time simulator, and the executor on two gloo ranks.

Mirrors what the reference gets from torch's schedule classes through
torchtitan/distributed/pipeline_parallel.py:36-123 (schedule by name or CSV, looped stage placement)."""
import os

import pytest

from flame_b200.parallel import pp_schedule as ps
from test_trainer_cpu import TINY, _args, _losses_from_log, _torchrun


@pytest.mark.parametrize("name,pp,stages,n_mb", [("GPipe", 4, 4, 8), ("1F1B", 4, 4, 8), ("1F1B", 2, 2, 1),
                                                 ("LoopedBFS", 2, 4, 3), ("Interleaved1F1B", 2, 4, 4),
                                                 ("Interleaved1F1B", 4, 8, 8), ("Interleaved1F1B", 4, 12, 4)])
def test_named_schedules_are_complete_and_deadlock_free(name, pp, stages, n_mb):
    sched = ps.build_schedule(name, pp, stages, n_mb)
    ticks = ps.simulate(sched, stages, n_mb)  # raises on a missing action or a deadlock
    assert len(ticks) == 2 * stages * n_mb
    owner = ps.stage_owners(pp, stages)
    for r, acts in enumerate(sched):
        assert all(owner[a.stage] == r for a in acts)
        assert [ticks[a] for a in acts] == sorted(ticks[a] for a in acts)
    assert ps.parse_schedule_csv(ps.format_schedule_csv(sched)) == sched
    # both sides of every pair see the same message list, and each rank's own sends appear in production order
    order = ps.pair_message_order(sched, owner, n_mb)
    for (lo, hi), msgs in order.items():
        assert all({m.src, m.dst} == {lo, hi} for m in msgs)
        for r in (lo, hi):
            produced = [ticks[ps.Action(ps.F, m.stage - 1, m.mb) if m.kind == "A" else ps.Action(ps.B, m.stage + 1, m.mb)]
                        for m in msgs if m.src == r]
            assert produced == sorted(produced)


def test_interleaving_shrinks_the_bubble():
    one = ps.bubble_fraction(ps.build_schedule("1F1B", 4, 4, 8), 4, 8)
    two = ps.bubble_fraction(ps.build_schedule("Interleaved1F1B", 4, 8, 8), 8, 8)
    assert two < one


def test_stage_placement_styles():
    assert ps.stage_ids_this_rank(1, 4, 8, "loop") == (1, 5)
    assert ps.stage_ids_this_rank(1, 4, 8, "v") == (1, 6)
    with pytest.raises(ValueError):
        ps.stage_ids_this_rank(0, 4, 6)


def test_invalid_schedules_are_rejected():
    with pytest.raises(ValueError, match="deadlock"):
        ps.simulate(ps.parse_schedule_csv("0B0,0F0\n1F0,1B0\n"), 2, 1)
    with pytest.raises(ValueError, match="exactly once"):
        ps.simulate(ps.parse_schedule_csv("0F0,0B0\n1F0\n"), 2, 1)
    with pytest.raises(ValueError, match="compute actions"):
        ps.parse_schedule_csv("0F0,0SEND_F0\n")
    with pytest.raises(ValueError, match="multiple"):
        ps.build_schedule("Interleaved1F1B", 2, 4, 3)
    # a split backward is accepted and folded into one backward
    assert ps.parse_schedule_csv("0F0,0I0,0W0\n")[0] == [ps.Action("F", 0, 0), ps.Action("B", 0, 0)]


def test_looped_schedules_match_single_rank_training(tmp_path):
    """pp=2 with two stages per rank (Interleaved1F1B by name, LoopedBFS from a CSV) reproduces the single-rank loss
    curve of a 4-layer model in fp32."""
    tmp = str(tmp_path)
    four = dict(TINY, num_hidden_layers=4)
    common = ["--training.seq_len", "1024"]

    def args(d, extra):
        a = _args(d, steps=3, extra=common + extra)
        import json
        with open(os.path.join(d, "tiny.json"), "w") as f:
            json.dump(four, f)
        return a

    one = _torchrun(tmp, 1, args(tmp, []), 29751)
    assert one.returncode == 0, one.stderr[-3000:]
    a = _losses_from_log(one.stderr)
    csv = os.path.join(tmp, "bfs.csv")
    with open(csv, "w") as f:
        f.write(ps.format_schedule_csv(ps.build_schedule("LoopedBFS", 2, 4, 4)))
    pp = ["--experimental.pipeline_parallel_degree", "2", "--experimental.pipeline_parallel_microbatches", "4"]
    for name, extra, port in (("il", ["--experimental.pipeline_parallel_schedule", "Interleaved1F1B"], 29752),
                              ("csv", ["--experimental.pipeline_parallel_schedule_csv", csv], 29753)):
        d = os.path.join(tmp, name)
        os.makedirs(d)
        r = _torchrun(d, 2, args(d, pp + extra), port)
        assert r.returncode == 0, r.stderr[-3000:]
        assert "stages [0, 2] of 4" in r.stderr and "stages [1, 3] of 4" in r.stderr
        b = _losses_from_log(r.stderr)
        b = b[::2] if len(b) == 6 else b
        assert len(b) >= 3, (name, b, r.stderr[-2000:])
        for x, y in zip(a, b[:3]):
            assert abs(x - y) < 5e-3, (name, a, b)
