"""Timings and roofline fractions of the fused compute + communication kernels (one process per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29555 \
        -m flame_b200.tools.commbench [--iters 20] [--out summary.json]

Measured, per kernel, with CUDA events on the launching stream after warm-up, a barrier before every timed iteration,
a 256 MiB L2 flush in between, and the MAXIMUM over ranks of the median:

* ``peer_reduce_scatter``   data-parallel gradient reduce-scatter (+ norm partials) of one 12.6 M-parameter unit
* ``peer_adamw_push``       AdamW on the slice + bf16 publication into every peer
* ``peer_gather_flat``      stand-alone sharded-parameter all-gather of one unit
* ``gemm2_gather_b``        the same all-gather fused into the unit's first GEMM (65,536 x 3072 x 1024), against the plain GEMM
* ``gemm2_allgather_a``     tensor-parallel all-gather -> GEMM, against the plain GEMM on gathered rows
* ``gemm2_scatter_rows``    tensor-parallel GEMM -> reduce-scatter (scatter + slot sum), against the plain GEMM

For every kernel: the bytes that have to cross NVLink per rank, the time, bytes / time against the measured peer-copy
bandwidth of this pool (770 GB/s per direction; 900 GB/s nominal) and, for the GEMM-carrying kernels, TFLOP/s against the
measured bf16 peak.  The roofline time of a fused kernel is the slower of (FLOPs / peak) and (NVLink bytes / link
bandwidth); ``roofline_fraction`` = that time / measured time.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

LINK_MEASURED, LINK_NOMINAL = 770e9, 900e9


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from flame_b200.ops import _lib, gemm as gemm_ops, optim as optim_ops
    from flame_b200.parallel.dims import ParallelDims
    from flame_b200.parallel.engine import OptimConfig, Unit
    from flame_b200.parallel.peer import PeerCollectives
    from flame_b200.parallel.resharding import CHUNK_SHIFT
    from flame_b200.tools.opbench import peaks
    _, flops_peak, peak_label = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    L = _lib.lib()

    def timed(fn, iters=args.iters, warmup=3) -> float:
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            torch.cuda.synchronize()
            dist.barrier(device_ids=[local])
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t) * 1e-3

    results = []

    def record(name, seconds, link_bytes, flops=0.0, plain_seconds=None, note=""):
        t_link, t_flop = link_bytes / LINK_MEASURED, flops / flops_peak
        row = {"kernel": name, "ranks": world, "ms": round(seconds * 1e3, 4), "nvlink_bytes_per_rank": int(link_bytes),
               "nvlink_gbs": round(link_bytes / seconds / 1e9, 1),
               "fraction_of_measured_770": round(link_bytes / seconds / LINK_MEASURED, 3),
               "fraction_of_nominal_900": round(link_bytes / seconds / LINK_NOMINAL, 3),
               "roofline_fraction": round(max(t_link, t_flop) / seconds, 3), "note": note}
        if flops:
            row["tflops"] = round(flops / seconds / 1e12, 1)
            row["tflops_fraction_" + peak_label.replace(" ", "_")] = round(flops / seconds / flops_peak, 3)
        if plain_seconds is not None:
            row["plain_gemm_ms"] = round(plain_seconds * 1e3, 4)
            row["plain_gemm_tflops"] = round(flops / plain_seconds / 1e12, 1)
        results.append(row)

    dims = ParallelDims(dp_shard=-1, world_size=world).build_mesh(rank)
    pc = PeerCollectives(dims, dev)
    # ---- a unit the size of one transformer_340M block: 12.6 M parameters ------------------------------------------
    chunk_elems = (1 << CHUNK_SHIFT) // 2
    numel = (12_600_000 + world * chunk_elems - 1) // (world * chunk_elems) * (world * chunk_elems)
    shard = numel // world
    grad = pc.allocate(numel, torch.float32, "grad")
    compute = pc.allocate(numel, torch.bfloat16, "compute")
    pshard = pc.allocate(shard, torch.bfloat16, "pshard")
    grad.normal_()
    pshard.normal_()

    class _Eng:
        units = []
        ctrl = torch.zeros(optim_ops.CTRL_SIZE, dtype=torch.float32, device=dev)
        resharding = False

    u = Unit("layers.0", [], numel, world, rank)
    u.base, u.sbase, u.buf = 0, 0, 0
    u.grad, u.compute, u.pshard = grad, compute, pshard
    u.master, u.exp_avg, u.exp_avg_sq = (torch.zeros(shard, device=dev) for _ in range(3))
    u.grad_shard = torch.zeros(shard, device=dev)
    u.rs_seq = 0
    eng = _Eng()
    eng.units = [u]
    pc.attach(eng)
    eng._flush_pending = lambda: None

    def rs():
        pc.begin_step()
        pc.reduce_scatter_avg(u, world)

    t = timed(rs)
    record("peer_reduce_scatter_kernel (+ signal / wait / norm)", t, shard * 4 * (world - 1),
           note=f"fp32 unit of {numel:,} elements; every rank pulls its 1/{world} slice from the {world - 1} peers")
    o = OptimConfig(lr=1e-4)
    eng.ctrl[optim_ops.CTRL_NORM_SQ] = 1.0

    def push():
        pc.begin_step()
        pc.adamw_and_publish(u, 1e-4, o, 1.0)
        pc.publish_done()

    t = timed(push)
    record("peer_adamw_push_kernel (+ signal / wait)", t, shard * 2 * (world - 1),
           note="AdamW on the slice; the bf16 result is stored into every peer's parameter buffer")

    pc.params_written(1)

    def gather():
        pc.gather_params(u, 0, numel * 2)

    t = timed(gather)
    record("peer_gather_flat_kernel", t, shard * 2 * (world - 1), note="stand-alone sharded-parameter all-gather of the unit")

    # fused: the gather rides on the block's first GEMM (qkv projection of transformer_340M: 65,536 x 3072 x 1024)
    M, N, K = 65536, 3072, 1024
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w_off = 1 << 20   # the weight lies 2 MiB into the unit, after the small parameters
    w = compute[w_off:w_off + N * K].view(N, K)
    y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    flags = torch.zeros((numel * 2 >> CHUNK_SHIFT) + 1, dtype=torch.int32, device=dev)
    epoch = [0]

    def fused():
        epoch[0] += 1
        pend = pc.make_pending(u, 0, numel * 2, flags, epoch[0])
        gemm_ops.set_pending_gather(pend)
        gemm_ops.gemm_nt(x, w, out=y)
        assert pend.done

    t_plain = timed(lambda: gemm_ops.gemm_nt(x, w, out=y))
    t = timed(fused)
    record("gemm2_bf16_kernel, flat gather mode (fb_gemm2_gather_b)", t, shard * 2 * (world - 1), 2.0 * M * N * K, t_plain,
           note="all-gather of the whole unit fused into its first GEMM; the plain GEMM reads an already gathered weight")

    # ---- tensor-parallel fused kernels --------------------------------------------------------------------------
    if world >= 2:
        from flame_b200.parallel.tensor_parallel import TPContext
        tdims = ParallelDims(dp_shard=1, tp=world, world_size=world).build_mesh(rank)
        tp = TPContext(tdims, dev)
        rows, Kt, Nt = 8192 // world, 4096, 11008 // world // 8 * 8
        if tp.ensure_buffers(rows, max(Kt, 4096)):
            xs = torch.randn(rows, Kt, device=dev, dtype=torch.bfloat16)
            wt = torch.randn(Nt, Kt, device=dev, dtype=torch.bfloat16) * 0.02
            x_full = torch.randn(rows * world, Kt, device=dev, dtype=torch.bfloat16)
            t_plain = timed(lambda: gemm_ops.gemm_nt(x_full, wt))
            t = timed(lambda: tp.allgather_gemm(xs, wt, False, Nt))
            record("gemm2_bf16_kernel, row gather mode (fb_gemm2_allgather_a)", t, rows * Kt * 2 * (world - 1),
                   2.0 * rows * world * Nt * Kt, t_plain, note=f"GLA-7B up projection shard: {rows * world} x {Nt} x {Kt}")
            a = torch.randn(rows * world, Nt, device=dev, dtype=torch.bfloat16)
            wd = torch.randn(4096, Nt, device=dev, dtype=torch.bfloat16) * 0.02
            t_plain = timed(lambda: gemm_ops.gemm_nt(a, wd))
            t = timed(lambda: tp.gemm_reduce_scatter(a, wd, False, 4096))
            record("gemm2_bf16_kernel, row scatter mode (fb_gemm2_scatter_rows) + slot sum", t,
                   rows * 4096 * 2 * (world - 1), 2.0 * rows * world * 4096 * Nt, t_plain,
                   note=f"GLA-7B down projection shard: {rows * world} x 4096 x {Nt}; bf16 partial rows go to their owners")
    torch.cuda.synchronize()
    _lib.assert_status_ok()
    if rank == 0:
        out = {"ranks": world, "link_reference": "770 GB/s per direction measured on this pool, 900 GB/s nominal",
               "compute_reference": f"{flops_peak / 1e12:.0f} TFLOP/s bf16 {peak_label}", "kernels": results}
        print(json.dumps(out, indent=1))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(out, f, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
