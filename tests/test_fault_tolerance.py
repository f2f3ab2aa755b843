"""Failure detection without faulting any device: injected on the host, or by letting a bounded device wait run out."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_nan_gradient_skips_the_step_and_counts_it():
    """A poisoned gradient (NaN norm) must leave parameters, moments and the step counter untouched."""
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.parallel import OptimConfig, ParallelDims, ShardedEngine
    cfg = ModelConfig("transformer", hidden_size=64, num_hidden_layers=1, num_heads=2, vocab_size=128)
    model = build_model(cfg, device="meta", init=False)
    eng = ShardedEngine(model, ParallelDims(world_size=1), torch.device("cpu"), torch.float32,
                        OptimConfig(lr=1e-2, skip_nan_inf=True))
    eng.init_weights(0)
    ids = torch.randint(3, 128, (1, 32))
    eng.zero_grad()
    model(input_ids=ids, labels=ids).loss.backward()
    eng.step(1e-2)
    before = eng.compute_all.clone()
    eng.zero_grad()
    model(input_ids=ids, labels=ids).loss.backward()
    eng.units[0].grad[3] = float("nan")  # host-side fault injection
    eng.step(1e-2)
    assert torch.equal(eng.compute_all, before)
    assert eng.applied_steps() == 1 and eng.skipped_steps() == 1
    eng.zero_grad()
    model(input_ids=ids, labels=ids).loss.backward()
    eng.step(1e-2)
    assert eng.applied_steps() == 2 and not torch.equal(eng.compute_all, before)


def test_lost_rank_is_detected_by_the_collective_timeout(tmp_path):
    """Rank 1 leaves between steps; rank 0's next collective ends with an error after the short timeout (gloo, CPU)."""
    script = tmp_path / "w.py"
    script.write_text(textwrap.dedent('''
        import os, sys, time, datetime, torch, torch.distributed as dist
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=3))
        rank = dist.get_rank()
        t = torch.ones(4)
        dist.all_reduce(t)                      # step 1: everybody is here
        if rank == 1:
            os._exit(0)                         # leaves between steps, nothing in flight
        try:
            dist.all_reduce(t)                  # step 2: the peer is gone
            print("NO_ERROR")
        except Exception as e:
            print("DETECTED", type(e).__name__)
        os._exit(0)
    '''))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29761", str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=120, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert "DETECTED" in r.stdout, (r.stdout, r.stderr[-2000:])


def test_truncated_checkpoint_is_not_picked_up(tmp_path):
    """A step folder without its .metadata file (interrupted write) is ignored when looking for the latest step."""
    from flame_b200.components.checkpoint import CheckpointManager
    (tmp_path / "checkpoint" / "step-4").mkdir(parents=True)
    (tmp_path / "checkpoint" / "step-4" / ".metadata").write_text("x")
    (tmp_path / "checkpoint" / "step-8").mkdir(parents=True)  # no .metadata: incomplete
    mgr = CheckpointManager.__new__(CheckpointManager)
    mgr.folder = str(tmp_path / "checkpoint")
    assert mgr.find_latest_step() == 4


@pytest.mark.gpu
def test_device_wait_runs_out_and_reports_instead_of_hanging():
    """A peer flag that nothing sets: the bounded wait gives up, the status word says so, the context stays usable."""
    from ctypes import c_double, c_int, c_void_p
    from flame_b200.ops import _lib
    L = _lib.lib()
    L.fb_peer_wait.argtypes = [c_void_p, c_int, c_int, c_int, c_double, c_void_p]
    L.fb_peer_wait.restype = c_int
    _lib.status_clear()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    rc = L.fb_peer_wait(flags.data_ptr(), 2, 0, 1, 0.2, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    st = _lib.status()
    assert (st >> 16) == 5, hex(st)  # ERR_WAIT_PEER
    with pytest.raises(_lib.KernelError):
        _lib.assert_status_ok()
    _lib.status_clear()
    x = torch.ones(8, device="cuda")
    assert float((x * 2).sum()) == 16.0  # the context is alive


@pytest.mark.gpu
def test_step_after_a_failed_wait_applies_nothing_and_the_engine_raises():
    """The trainer's guard: a wait on a flag nobody sets runs out during a step; the optimizer kernels of that step
    leave parameters and moments untouched, and the engine raises at the next status check."""
    from ctypes import c_double, c_int, c_void_p
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.ops import _lib, optim as optim_ops
    from flame_b200.ops.varlen import VarlenMeta
    from flame_b200.parallel import OptimConfig, ParallelDims, ShardedEngine
    dev = torch.device("cuda:0")
    cfg = ModelConfig("transformer", hidden_size=128, num_hidden_layers=1, num_heads=2, vocab_size=512)
    model = build_model(cfg, device="meta", dtype=torch.bfloat16, init=False)
    eng = ShardedEngine(model, ParallelDims(world_size=1), dev, torch.bfloat16, OptimConfig(lr=1e-2))
    eng.init_weights(0)
    ids = torch.randint(3, 512, (1, 512), device=dev)
    meta = VarlenMeta.from_cu_seqlens(torch.tensor([0, 200, 512], dtype=torch.int32), 512, dev)
    _lib.status_clear()

    def one_step():
        eng.zero_grad()
        model(input_ids=ids, labels=ids, meta=meta).loss.backward()
        eng.step(1e-2)

    one_step()
    eng.check_status(sync=True)
    before = [u.master.clone() for u in eng.units]
    bf_before = eng.compute_all.clone()
    L = _lib.lib()
    L.fb_peer_wait.argtypes = [c_void_p, c_int, c_int, c_int, c_double, c_void_p]
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    eng.zero_grad()
    model(input_ids=ids, labels=ids, meta=meta).loss.backward()
    assert L.fb_peer_wait(flags.data_ptr(), 2, 0, 1, 0.2, torch.cuda.current_stream().cuda_stream) == 0
    eng.step(1e-2)
    with pytest.raises(_lib.KernelError, match="another GPU"):
        eng.check_status(sync=True)
    assert eng.aborted_steps() == 1 and eng.applied_steps() == 1
    for u, b in zip(eng.units, before):
        assert torch.equal(u.master, b)
    assert torch.equal(eng.compute_all, bf_before)
    _lib.status_clear()
    one_step()  # the context and the engine are usable again
    eng.check_status(sync=True)
    assert eng.applied_steps() == 2
    assert not torch.equal(eng.units[0].master, before[0])


def test_abort_flag_voids_the_update_on_the_reference_path():
    from flame_b200.ops import optim as optim_ops
    ctrl = torch.zeros(optim_ops.CTRL_SIZE)
    ctrl[optim_ops.CTRL_NORM_SQ] = 4.0
    ctrl[optim_ops.CTRL_ABORT] = 1.0
    p, m, v, g = torch.ones(8), torch.zeros(8), torch.zeros(8), torch.ones(8)
    optim_ops.adamw_step(p, m, v, g, None, ctrl, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1.0, False)
    optim_ops.adamw_finalize(ctrl, 1.0, False)
    assert torch.equal(p, torch.ones(8)) and float(ctrl[optim_ops.CTRL_STEP]) == 0 and float(ctrl[optim_ops.CTRL_ABORTED]) == 1


# ---------------------------------------------------------------------------------------------------------------
# replica groups: quorum, managed all-reduce, commit vote, live recovery (host-side failures only, gloo on CPU)
# ---------------------------------------------------------------------------------------------------------------
_REPLICA = textwrap.dedent("""
    import sys, time, torch
    import torch.distributed as dist
    from flame_b200.components.ft import FTManager, connect
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.parallel import OptimConfig, ParallelDims, ShardedEngine

    addr, rid, n, steps, leave_after = sys.argv[1], *map(int, sys.argv[2:6])
    wait_key = sys.argv[6]
    store = connect(addr, rid)
    cfg = ModelConfig("transformer", hidden_size=64, num_hidden_layers=1, num_heads=2, vocab_size=128)
    model = build_model(cfg, device="meta", init=False)
    eng = ShardedEngine(model, ParallelDims(world_size=1), torch.device("cpu"), torch.float32, OptimConfig(lr=1e-2))
    eng.init_weights(rid if wait_key == "fresh" else 0)   # a fresh joiner starts from different weights on purpose
    ft = FTManager(store, rid, n, timeout=20.0, heartbeat_store=connect(addr, rid))
    eng.replica_reducer, eng.commit_gate = ft.allreduce, ft.should_commit
    if wait_key != "fresh":
        store.wait(["go"])                                 # all three start together
    gen = torch.Generator().manual_seed(100 + rid)
    step, sizes = 0, []
    while step < steps:
        if wait_key not in ("none", "fresh") and step == 4:
            store.wait([wait_key])                         # the test holds the survivors here until the joiner is up
        dec = ft.start_step(step)
        sizes.append(len(dec["members"]))
        if min(dec["steps"].values()) < dec["max_step"]:
            assert ft.recover(eng.replica_state_tensors())
            if dec["heal"]:
                eng.refresh_compute()
                step = dec["max_step"]
                print(f"HEALED {rid} to {step}", flush=True)
                if step >= steps:
                    break
        ids = torch.randint(3, 128, (1, 32), generator=gen)
        eng.zero_grad()
        model(input_ids=ids, labels=ids).loss.backward()
        before = eng.voided_steps
        eng.step(1e-2)
        if eng.voided_steps != before:
            print(f"VOIDED {rid} at {step}", flush=True)
            continue
        step += 1
        if step == leave_after:
            ft.shutdown()                                  # leaves between steps, nothing in flight
            print(f"LEFT {rid} at {step}", flush=True)
            sys.exit(0)
    ck = float(sum(u.master.double().sum() for u in eng.units))
    print(f"DONE {rid} step {step} checksum {ck:.9f} sizes {sizes} reconf {ft.reconfigurations}", flush=True)
    ft.shutdown()
""")


def _spawn(addr, rid, n, steps, leave_after, wait_key):
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    return subprocess.Popen([sys.executable, "-c", _REPLICA, addr, str(rid), str(n), str(steps), str(leave_after), wait_key],
                            cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)


def test_replica_groups_survive_a_departure_and_heal_a_joiner():
    """Three replica groups average gradients; group 2 leaves after two steps, the other two carry on as a quorum of
    two; a fresh group 2 (different weights, step 0) joins, copies the survivors' state and finishes in lockstep."""
    import re
    from datetime import timedelta
    import torch.distributed as dist
    from flame_b200.components.ft import Lighthouse
    port = 29771
    store = dist.TCPStore("127.0.0.1", port, is_master=True, timeout=timedelta(seconds=60), wait_for_workers=False)
    lh = Lighthouse(store, 3, min_replicas=1, heartbeat_timeout=1.0, join_timeout=1.0).start()
    addr = f"127.0.0.1:{port}"
    try:
        procs = [_spawn(addr, 0, 3, 8, -1, "joiner_up"), _spawn(addr, 1, 3, 8, -1, "joiner_up"),
                 _spawn(addr, 2, 3, 8, 2, "none")]
        import time
        t0 = time.time()
        while not store.check(["hb/0", "hb/1", "hb/2"]):
            assert time.time() - t0 < 200, "the replicas never came up"
            time.sleep(0.05)
        store.set("go", "1")
        out2, _ = procs[2].communicate(timeout=240)
        assert "LEFT 2 at 2" in out2, out2
        t0 = time.time()
        joiner = _spawn(addr, 2, 3, 8, -1, "fresh")
        # release the survivors only once the JOINER is beating (the last beat of the group that left can still be
        # fresh: only a beat written after the spawn counts), so that it is part of a later quorum
        while float(store.get("hb/2").decode()) <= t0:
            assert time.time() - t0 < 200, "the joiner never came up"
            time.sleep(0.05)
        store.set("joiner_up", "1")
        outs = [p.communicate(timeout=240)[0] for p in (procs[0], procs[1], joiner)]
    finally:
        lh.stop()
    done = [re.search(r"DONE (\d) step (\d+) checksum ([-0-9.]+) sizes (\[[^\]]*\]) reconf (\d+)", o) for o in outs]
    assert all(done), outs
    assert {m.group(2) for m in done} == {"8"}
    # all three end with the same weights: same quorums, same averaged gradients, joiner healed from the survivors
    assert len({m.group(3) for m in done}) == 1, [m.group(0) for m in done]
    assert "HEALED 2 to" in outs[2]
    sizes0 = eval(done[0].group(4))
    assert sizes0[0] == 3 and 2 in sizes0 and sizes0[-1] == 3, sizes0   # 3 -> 2 after the departure -> 3 again
    assert int(done[0].group(5)) >= 3


_LOCAL_RANKS = textwrap.dedent("""
    import os, sys, torch
    from datetime import timedelta
    import torch.distributed as dist
    from flame_b200.components.ft import FTManager, connect

    addr, rid, lrank, lport = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{lport}", rank=lrank, world_size=2,
                            timeout=timedelta(seconds=60))
    ft = FTManager(connect(addr, rid), rid, 2, timeout=3.0, local_group=dist.group.WORLD, local_rank=lrank,
                   heartbeat_store=connect(addr, rid))

    class Broken:
        def allreduce(self, *a, **k):
            raise RuntimeError("injected: this rank's cross-replica link is down")

    step = 0
    for attempt in range(4):
        dec = ft.start_step(step)
        if attempt == 0 and rid == 0 and lrank == 1:
            ft.pg = Broken()                       # host-side failure on ONE local rank of ONE replica group
        t = torch.full((4,), float(rid + 1))
        ft.allreduce(t)
        ok = ft.should_commit()
        print(f"ATTEMPT {attempt} rid {rid} lrank {lrank} commit {ok} value {t[0].item():.2f}", flush=True)
        if ok:
            step += 1
    print(f"END rid {rid} lrank {lrank} step {step}", flush=True)
    ft.shutdown()
    dist.destroy_process_group()
""")


def test_all_local_ranks_of_a_replica_group_take_the_same_commit_decision():
    """Two replica groups of two ranks each.  The cross-replica collective of one local rank fails on the host; the
    other local rank's succeeds.  Both ranks of both groups must void that step together and commit the later ones."""
    import re
    from datetime import timedelta
    import torch.distributed as dist
    from flame_b200.components.ft import Lighthouse
    port = 29775
    store = dist.TCPStore("127.0.0.1", port, is_master=True, timeout=timedelta(seconds=60), wait_for_workers=False)
    lh = Lighthouse(store, 2, min_replicas=2, heartbeat_timeout=5.0, join_timeout=20.0).start()
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    try:
        procs = [subprocess.Popen([sys.executable, "-c", _LOCAL_RANKS, f"127.0.0.1:{port}", str(rid), str(lr), str(29780 + rid)],
                                  cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                 for rid in range(2) for lr in range(2)]
        outs = [p.communicate(timeout=300)[0] for p in procs]
    finally:
        lh.stop()
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
    for o in outs:
        got = re.findall(r"ATTEMPT (\d) rid \d lrank \d commit (True|False) value ([0-9.]+)", o)
        assert [g[1] for g in got] == ["False", "True", "True", "True"], o
        assert all(g[2] == "1.50" for g in got[1:]), o      # the average of 1 and 2 once the groups were rebuilt
        assert "END" in o and "step 3" in o, o


def test_trainer_runs_two_fault_tolerant_replica_groups(tmp_path):
    """``--fault_tolerance.enable`` through the trainer: two single-process replica groups on different data end with
    the same weights."""
    import re
    from datetime import timedelta
    import torch.distributed as dist
    from flame_b200.components.ft import Lighthouse
    from test_trainer_cpu import _args
    port = 29773
    store = dist.TCPStore("127.0.0.1", port, is_master=True, timeout=timedelta(seconds=60), wait_for_workers=False)
    lh = Lighthouse(store, 2, min_replicas=2, heartbeat_timeout=5.0, join_timeout=30.0).start()
    try:
        procs = []
        for rid in range(2):
            d = os.path.join(str(tmp_path), f"r{rid}")
            os.makedirs(d)
            args = _args(d, steps=3, extra=["--fault_tolerance.enable", "--fault_tolerance.replica_id", str(rid),
                                           "--fault_tolerance.group_size", "2"])
            env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2",
                       FLAME_FT_LIGHTHOUSE=f"127.0.0.1:{port}", FLAME_FT_TIMEOUT="60")
            procs.append(subprocess.Popen([sys.executable, "-m", "flame_b200.train", *args], cwd=ROOT, env=env,
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        outs = [p.communicate(timeout=400)[0] for p in procs]
    finally:
        lh.stop()
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
    sums = [re.search(r"ends at step 3 with parameter checksum ([-0-9.]+)", o) for o in outs]
    assert all(sums), outs[0][-2000:]
    assert sums[0].group(1) == sums[1].group(1)
    losses = [re.findall(r"step:\s+1\s+loss:\s+([0-9.]+)", o) for o in outs]
    assert losses[0] and losses[1] and losses[0][0] != losses[1][0]   # different data per replica group


def test_local_sgd_and_diloco_synchronise_simulated_replica_groups():
    """Two replica groups simulated in one process: the cross-group averaging collective is a function that averages the
    same tensor of both engines.  LocalSGD: masters equal the mean after a synchronisation.  DiLoCo: the outer step
    follows SGD with Nesterov momentum on the averaged pseudo-gradient, and a failed synchronisation restores the last
    outer weights."""
    from flame_b200.components.ft import SemiSync
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.parallel import OptimConfig, ParallelDims, ShardedEngine

    def make(seed_data):
        cfg = ModelConfig("transformer", hidden_size=64, num_hidden_layers=1, num_heads=2, vocab_size=128)
        model = build_model(cfg, device="meta", init=False)
        eng = ShardedEngine(model, ParallelDims(world_size=1), torch.device("cpu"), torch.float32, OptimConfig(lr=1e-2))
        eng.init_weights(0)
        gen = torch.Generator().manual_seed(seed_data)
        return model, eng, gen

    def train(model, eng, gen, n):
        for _ in range(n):
            ids = torch.randint(3, 128, (1, 32), generator=gen)
            eng.zero_grad()
            model(input_ids=ids, labels=ids).loss.backward()
            eng.step(1e-2)

    for method in ("local_sgd", "diloco"):
        (ma, ea, ga), (mb, eb, gb) = make(1), make(2)
        fail = {"now": False}
        sa = SemiSync(ea, method, 3, lambda t: None, lambda: fail["now"], outer_lr=0.5, outer_momentum=0.9)
        sb = SemiSync(eb, method, 3, lambda t: None, lambda: fail["now"], outer_lr=0.5, outer_momentum=0.9)
        start = [u.master.clone() for u in ea.units]
        train(ma, ea, ga, 3), train(mb, eb, gb, 3)
        assert not torch.equal(ea.units[0].master, eb.units[0].master)
        # the averaging collective of each group is emulated by handing it the mean over both groups, in call order
        if method == "local_sgd":
            mean = [(x.master + y.master) / 2 for x, y in zip(ea.units, eb.units)]
            it_a, it_b = iter(mean), iter(mean)
            sa.allreduce = lambda t: t.copy_(next(it_a))
            sb.allreduce = lambda t: t.copy_(next(it_b))
            sa.local_steps = sb.local_steps = 2
            assert sa.after_step() and sb.after_step()
            for x, y, m in zip(ea.units, eb.units, mean):
                assert torch.allclose(x.master, m) and torch.equal(x.master, y.master)
        else:
            pg = [((o - x.master) + (o - y.master)) / 2 for o, x, y in zip(start, ea.units, eb.units)]
            it_a, it_b = iter(pg), iter(pg)
            sa.allreduce = lambda t: t.copy_(next(it_a))
            sb.allreduce = lambda t: t.copy_(next(it_b))
            sa.local_steps = sb.local_steps = 2
            assert sa.after_step() and sb.after_step()
            # first outer step: momentum = g, Nesterov step = g + mu g, outer = start - lr (1 + mu) g
            for o, g, x, y in zip(start, pg, ea.units, eb.units):
                want = o - 0.5 * (1 + 0.9) * g
                assert torch.allclose(x.master, want, atol=1e-6) and torch.equal(x.master, y.master)
            # a failed synchronisation: inner progress is dropped, weights return to the last outer weights
            outer_now = [o.clone() for o in sa.outer]
            train(ma, ea, ga, 3)
            fail["now"] = True
            sa.allreduce = lambda t: None
            sa.local_steps = 2
            assert not sa.after_step()
            for u, o in zip(ea.units, outer_now):
                assert torch.equal(u.master, o)
            fail["now"] = False
        assert torch.equal(ea.units[0].compute.float(), ea.units[0].master)   # compute buffers were refreshed
