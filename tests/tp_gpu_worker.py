"""Worker for the two-GPU tensor-parallel test: fused collective GEMMs against c10d + matmul, then a short tp=2 run."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


def main() -> None:
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.ops import _lib
    from flame_b200.parallel.dims import ParallelDims
    from flame_b200.parallel.engine import OptimConfig, ShardedEngine
    from flame_b200.parallel.tensor_parallel import TPContext, apply_tensor_parallel

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    dims = ParallelDims(dp_shard=1, tp=world, world_size=world).build_mesh(rank)
    out = {}
    tp = TPContext(dims, dev)
    rows, K, N = 2048, 1024, 1536
    assert tp.ensure_buffers(rows, max(K, N)), "symmetric memory is required for the fused tensor-parallel kernels"
    torch.manual_seed(100 + rank)
    x_s = torch.randn(rows, K, device=dev, dtype=torch.bfloat16)
    torch.manual_seed(7)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    errs = []
    for it in range(3):  # repeated calls exercise buffer alternation and epochs
        y, x_full = tp.allgather_gemm(x_s, w, False, N)
        ref_full = tp.all_gather_rows(x_s)
        errs.append(max(rel(x_full, ref_full), rel(y, ref_full.float() @ w.float().t())))
    out["allgather_gemm_err"] = max(errs)
    a = torch.randn(rows * world, K, device=dev, dtype=torch.bfloat16) * 0.1
    errs = []
    for it in range(3):
        y_s = tp.gemm_reduce_scatter(a, w, False, N)
        full = a.float() @ w.float().t()
        dist.all_reduce(full)
        errs.append(rel(y_s, full[rank * rows:(rank + 1) * rows]))
    out["gemm_reduce_scatter_err"] = max(errs)
    wt = w.t().contiguous()  # [K, N] storage: the "b_mn" form used by the backward passes
    y2, _ = tp.allgather_gemm(x_s, wt, True, N)
    out["allgather_gemm_mn_err"] = rel(y2, tp.all_gather_rows(x_s).float() @ w.float().t())
    torch.cuda.synchronize()
    _lib.assert_status_ok()

    # short training run: tp=2 against the same model without tp (same seed), bf16
    kw = dict(hidden_size=512, num_hidden_layers=2, num_heads=8, vocab_size=4096, max_position_embeddings=8192)
    losses = {}
    for name, use_tp in (("tp", True), ("single", False)):
        cfg = ModelConfig("transformer", **kw)
        m = build_model(cfg, device="meta", dtype=torch.bfloat16, init=False)
        if use_tp:
            apply_tensor_parallel(m, cfg, dims)
            d = dims
        else:
            d = ParallelDims(world_size=1)
        eng = ShardedEngine(m, d, dev, torch.bfloat16, OptimConfig(lr=1e-3, max_norm=1.0))
        eng.init_weights(11)
        m.train()
        g = torch.Generator().manual_seed(3)
        ls = []
        for step in range(4):
            ids = torch.randint(3, 4096, (1, 4096), generator=g).to(dev)
            cu = torch.tensor([0, 1500, 1501, 4096], dtype=torch.int32)
            eng.zero_grad()
            o = m(input_ids=ids, labels=ids, cu_seqlens=cu)
            o.loss.backward()
            eng.step(1e-3)
            ls.append(float(o.loss))
        losses[name] = ls
        out[name + "_grad_norm"] = eng.grad_norm()
    out["losses"] = losses
    out["fused"] = bool(tp.fused)
    torch.cuda.synchronize()
    _lib.assert_status_ok()
    if rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
