"""Worker for the multi-GPU tests (launched by torch.distributed.run): trains a small Transformer for a few steps
with the backend chosen by FLAME_B200_PEER and prints the losses and a parameter checksum from rank 0."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    from flame_b200.config_manager import JobConfig
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.ops import _lib
    from flame_b200.parallel.dims import ParallelDims
    from flame_b200.parallel.engine import OptimConfig
    from flame_b200.parallel.parallelize import parallelize
    import bench

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    policy = os.environ.get("FLAME_TEST_RESHARD", "never")
    accum = int(os.environ.get("FLAME_TEST_ACCUM", "1"))
    job = JobConfig().parse_args(["--model.config", bench.MODEL_JSON, "--model.tokenizer_path", "synthetic",
                                  "--activation_checkpoint.mode", os.environ.get("FLAME_TEST_AC", "none"),
                                  "--training.fsdp_reshard_after_forward", policy])
    replicate = int(os.environ.get("FLAME_TEST_REPLICATE", "1"))
    dims = ParallelDims(dp_replicate=replicate, dp_shard=-1, world_size=world).build_mesh(rank)
    cfg = ModelConfig("transformer", hidden_size=512, num_hidden_layers=3, num_heads=8, vocab_size=32000,
                      max_position_embeddings=8192)
    model = build_model(cfg, device="meta", dtype=torch.bfloat16, init=False)
    runner = parallelize(model, cfg, dims, job, dev, torch.bfloat16, OptimConfig(lr=1e-3, max_norm=1.0, skip_nan_inf=True))
    eng = runner.engine
    eng.init_weights(7)
    model.train()
    bench.SEQ_LEN = 8192
    batches = bench.make_batches(5 * accum, rank)
    losses = []
    fused = 0
    from flame_b200.ops import gemm as gemm_ops
    for i in range(5):
        eng.zero_grad()
        loss = 0.0
        for m in range(accum):
            eng.set_last_microbatch(m == accum - 1)
            loss = loss + runner.forward_backward(batches[i * accum + m], 1.0 / accum)
        eng.step(1e-3)
        avg, _ = runner.reduce_loss(loss)
        losses.append(avg)
    torch.cuda.synchronize()
    _lib.assert_status_ok()
    # identical on every rank: the sum over ranks of the master slices' checksums (both modes shard them alike in size)
    local = torch.tensor([float(sum(u.master.double().abs().sum() for u in eng.units))], dtype=torch.float64, device=dev)
    dist.all_reduce(local)
    checksum = float(local)
    if hasattr(eng, "compute_all"):
        checksum = float(eng.compute_all.float().abs().sum())
    gn = eng.grad_norm()
    sums = [None] * world
    dist.all_gather_object(sums, checksum)
    if rank == 0:
        print("RESULT " + json.dumps({"losses": losses, "checksums": sums, "grad_norm": gn,
                                      "backend": type(eng.collectives).__name__, "engine": type(eng).__name__,
                                      "memory": eng.memory_report(),
                                      "launches": _lib.launches()}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
