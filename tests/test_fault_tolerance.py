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
