"""Two-GPU checks (skipped with fewer devices): peer-memory collectives against NCCL collectives."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(nproc: int, peer: bool, port: int, worker: str = "multi_gpu_worker.py", **extra_env) -> dict:
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", worker)]
    env = dict(os.environ, PYTHONPATH=ROOT, FLAME_B200_PEER="1" if peer else "0", **extra_env)
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-4000:])
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_collectives_match_nccl():
    a = _run(2, True, 29741)
    b = _run(2, False, 29742)
    assert a["backend"] == "PeerCollectives" and b["backend"] == "TorchCollectives"
    # every rank holds identical parameters after the step
    assert max(a["checksums"]) - min(a["checksums"]) == 0
    assert max(b["checksums"]) - min(b["checksums"]) == 0
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) / abs(y) < 2e-2
    assert all(x == x and x < 12 for x in a["losses"])
    assert abs(a["grad_norm"] - b["grad_norm"]) / b["grad_norm"] < 5e-2


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_tensor_parallel_kernels_and_tp2_training():
    r = _run(2, True, 29743, "tp_gpu_worker.py")
    assert r["fused"]
    assert r["allgather_gemm_err"] < 1e-2 and r["allgather_gemm_mn_err"] < 1e-2 and r["gemm_reduce_scatter_err"] < 1e-2
    for x, y in zip(r["losses"]["tp"], r["losses"]["single"]):
        assert abs(x - y) / y < 2e-2
    assert abs(r["tp_grad_norm"] - r["single_grad_norm"]) / r["single_grad_norm"] < 5e-2


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_parameter_mode_matches_resident_mode():
    """Parameters sharded between uses (peer gather fused into each block's first GEMM, recycled gradient staging) give
    the loss curve of the resident mode; with and without the fusion, with gradient accumulation, with checkpointing."""
    base = _run(2, True, 29744, FLAME_TEST_ACCUM="2")
    assert base["engine"] == "ShardedEngine"
    for port, env in ((29745, {}), (29746, {"FLAME_B200_FUSED_GATHER": "0"}), (29747, {"FLAME_TEST_AC": "full"}),
                      (29748, {"FLAME_B200_PEER": "0"})):
        peer = env.pop("FLAME_B200_PEER", "1") == "1"
        r = _run(2, peer, port, FLAME_TEST_RESHARD="default", FLAME_TEST_ACCUM="2", **env)
        assert r["engine"] == "ReshardingEngine", r
        for x, y in zip(r["losses"], base["losses"]):
            assert abs(x - y) / abs(y) < 5e-3, (env, r["losses"], base["losses"])
        assert abs(r["grad_norm"] - base["grad_norm"]) / base["grad_norm"] < 5e-2
        assert abs(r["checksums"][0] - r["checksums"][1]) == 0
        # 18 bytes per parameter over 2 ranks (plus padding to whole 128 KB chunks) against 6 + 16 / 2 bytes resident
        assert r["memory"]["sharded_bytes"] < 0.75 * base["memory"]["total_bytes"]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_hsdp_on_peer_kernels_matches_nccl():
    """dp_replicate 2 x dp_shard 2: the shard groups reduce and publish over peer memory, the slices are averaged over
    the replicate group; same losses, gradient norm and (on every rank) parameters as the c10d path."""
    a = _run(4, True, 29751, FLAME_TEST_REPLICATE="2")
    b = _run(4, False, 29752, FLAME_TEST_REPLICATE="2")
    assert a["backend"] == "PeerCollectives" and b["backend"] == "TorchCollectives"
    assert max(a["checksums"]) - min(a["checksums"]) == 0
    assert max(b["checksums"]) - min(b["checksums"]) == 0
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) / abs(y) < 2e-2
    assert abs(a["grad_norm"] - b["grad_norm"]) / b["grad_norm"] < 5e-2


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("family", ["transformer", "gla", "delta_net"])
def test_context_parallel_inside_documents_matches_one_gpu(tmp_path, family):
    """The trainer on one GPU against cp = 2 on two, rows of 4096 tokens with documents of up to 3072 (so the cut at 2048
    falls inside documents), bf16 kernels: softmax attention gathers keys / values, gla hands its recurrent state and
    the convolution's halo rows over, the delta rule its (transition, state) pair.  Same seed, same loss curve."""
    import test_trainer_cpu as t
    cfgs = {
        "transformer": dict(t.TINY),
        "gla": dict(t.TINY, model_type="gla", num_heads=2, expand_k=0.5, expand_v=1, use_gk=True, use_gv=False, attn_mode="chunk",
                    use_short_conv=True),
        "delta_net": dict(t.TINY, model_type="delta_net", num_heads=2, use_short_conv=True, use_gate=False, qk_norm="l2",
                          attn_mode="chunk"),
    }
    port = {"transformer": 29811, "gla": 29813, "delta_net": 29815}[family]

    def launch(d, nproc, extra, port):
        os.makedirs(d, exist_ok=True)
        args = t._args(d, steps=4, extra=["--training.seq_len", "4096", "--training.context_len", "3072", *extra])
        with open(os.path.join(d, "tiny.json"), "w") as f:
            json.dump(cfgs[family], f)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
               "127.0.0.1", "--master-port", str(port), "-m", "flame_b200.train", *args]
        r = subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-3000:]
        return t._losses_from_log(r.stderr)

    one = launch(str(tmp_path / "one"), 1, [], port)
    two = launch(str(tmp_path / "two"), 2, ["--experimental.context_parallel_degree", "2"], port + 1)
    two = two[::2] if len(two) == 8 else two
    assert len(one) == 4 and len(two) >= 4
    for x, y in zip(one, two[:4]):
        assert abs(x - y) < 2e-3, (one, two)
