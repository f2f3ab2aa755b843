"""Headline benchmark: training tokens/s of the flagship recipe on N B200s of one node.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 10 --warmup 3

Recipe (the reference's flagship, flame README "Transformer-340M"): configs/transformer_340M.json, bf16 parameters with
fp32 master weights / AdamW / gradient reduction, FSDP over all GPUs, per-GPU batch 1 x seq_len 65536 packed
variable-length documents (uniform 64..4096 tokens, EOS-joined, context_len 4096), gradient clipping 1.0, NaN/Inf skip.
Synthetic tokens, random-init weights.  Every step is a full training step: forward, backward, gradient reduction,
clipping, optimizer update, parameter re-gather.

Two numbers are measured per run:
* ``value``: K steps timed on the device with CUDA events (batches already resident on the GPU), max over ranks;
* ``e2e``: K steps through the trainer's ``Runner.forward_backward`` + ``engine.step`` with, every step, the
  host->device copy of that step's batch from pinned memory and a device->host read of the loss.

``--impl reference`` runs the unmodified reference trainer installed under ``baseline/_ref`` on the same recipe.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SEQ_LEN = 65536
CONTEXT_LEN = 4096
MODEL_JSON = os.path.join(ROOT, "configs", "transformer_340M.json")

# The named configurations of the baseline table.  ``--config X`` fills in the flags below it; a flag given explicitly
# wins.  t340m (the default) is the flagship recipe and is what a bare ``python bench.py --gpus N`` measures.
PRESETS = {
    "t340m": dict(model="transformer_340M", seq_len=65536, batch_size=1, varlen=True, tp=1, pp=1, ac="none"),
    "gdn1b": dict(model="gated_deltanet_1B", seq_len=65536, batch_size=1, varlen=True, tp=1, pp=1, ac="selective",
                  ac_option="mixer"),
    "sba340m": dict(model="sba_340m", seq_len=4096, batch_size=8, varlen=False, tp=1, pp=1, ac="none"),
    "gla7b_tp2": dict(model="gla_7B", seq_len=8192, batch_size=1, varlen=True, tp=2, pp=1, ac="none"),
    "gla7b_pp2": dict(model="gla_7B", seq_len=8192, batch_size=1, varlen=True, tp=1, pp=2, ac="none"),
}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_batches(n: int, rank: int, seed: int = 42, batch_size: int = 1, varlen: bool = True):
    """``n`` batches built by the trainer's own synthetic stream + collator (pinned host memory): one packed row with
    document boundaries (``varlen``), or ``batch_size`` rows of ``SEQ_LEN`` tokens without boundaries."""
    import torch
    from flame_b200.data import DataCollatorForLanguageModeling, SimpleTokenizer, SyntheticTokenDataset
    tok = SimpleTokenizer(32000, bos_token_id=None, eos_token_id=2)
    ds = SyntheticTokenDataset(SEQ_LEN, 32000, 64, 4096, eos_token_id=2, seed=seed, rank=rank)
    coll = DataCollatorForLanguageModeling(tok, context_len=CONTEXT_LEN if varlen else None, varlen=varlen)
    out = []
    it = iter(ds)
    for _ in range(n):
        b = coll([next(it) for _ in range(batch_size if not varlen else 1)])
        out.append({k: (v.pin_memory() if torch.cuda.is_available() else v) for k, v in b.items()})
    return out


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist
    from flame_b200.config_manager import JobConfig
    from flame_b200.models import ModelConfig, build_model
    from flame_b200.ops import _lib
    from flame_b200.parallel.dims import ParallelDims
    from flame_b200.parallel.engine import OptimConfig
    from flame_b200.parallel.parallelize import parallelize

    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    job = JobConfig().parse_args([
        "--model.config", MODEL_JSON, "--model.tokenizer_path", "synthetic", "--training.dataset", "synthetic",
        "--training.batch_size", str(args.batch_size), "--training.seq_len", str(SEQ_LEN),
        "--training.context_len", str(CONTEXT_LEN), *(["--training.varlen"] if args.varlen else []),
        "--training.skip_nan_inf", "--training.max_norm", "1.0", "--optimizer.lr", "3e-4",
        "--optimizer.eps", "1e-15", "--activation_checkpoint.mode", args.ac,
        "--activation_checkpoint.selective_ac_option", args.ac_option,
        "--training.tensor_parallel_degree", str(args.tp), "--experimental.pipeline_parallel_degree", str(args.pp),
        "--experimental.pipeline_parallel_microbatches", str(max(args.batch_size, args.pp)),
        "--training.fsdp_reshard_after_forward", args.reshard,
        *(["--training.enable_cpu_offload"] if args.cpu_offload else []),
        *(["--model.converters", "float8"] if args.float8 else [])])
    dims = ParallelDims(dp_shard=-1, tp=args.tp, pp=args.pp, world_size=world).build_mesh(rank)
    nd = args.tp * args.pp  # ranks that share one data stream
    cfg = ModelConfig.from_pretrained(MODEL_JSON)
    model = build_model(cfg, device="meta", dtype=torch.bfloat16, init=False)
    if args.float8:
        from flame_b200.train import apply_model_converters
        apply_model_converters(model, job)
    optim = OptimConfig(lr=3e-4, eps=1e-15, max_norm=1.0, skip_nan_inf=True)
    runner = parallelize(model, cfg, dims, job, dev, torch.bfloat16, optim)
    engine = runner.engine
    engine.init_weights(42)
    model.train()

    K, W = args.steps, args.warmup
    # ranks of one tensor-parallel / pipeline group read the same rows
    batches = make_batches(W + K, dims.dp_rank if dims.dp_enabled else 0, batch_size=args.batch_size, varlen=args.varlen)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > L2 (126 MB)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(device_ids=[local_rank])
            torch.cuda.synchronize()

    def step_e2e(b):
        engine.zero_grad()
        engine.set_last_microbatch(True)
        loss = runner.forward_backward(b, 1.0)  # pinned host -> device copy happens inside
        engine.step(3e-4)
        # device -> host read of the step's result (pipeline ranks without the last stage hold no loss)
        return float(loss) if loss is not None else float(engine.ctrl[4])

    # ---------------- end to end through the public API ----------------
    losses = [step_e2e(b) for b in batches[:W]]
    sync_all()
    t0 = time.perf_counter()
    for b in batches[W:]:
        losses.append(step_e2e(b))
    sync_all()
    e2e_s = time.perf_counter() - t0
    h2d = sum(v.numel() * v.element_size() for v in batches[0].values())

    # ---------------- device-timed: batches resident on the GPU ----------------
    dev_batches = [{k: v.to(dev) for k, v in b.items()} for b in batches[W:]]
    from flame_b200.ops.varlen import VarlenMeta
    if args.varlen:
        metas = [VarlenMeta.from_cu_seqlens(b["cu_seqlens"].reshape(-1), SEQ_LEN, dev) for b in batches[W:]]
    else:
        metas = [VarlenMeta.dense(args.batch_size, SEQ_LEN, dev) for _ in batches[W:]]

    def step_dev(b, meta):
        flush.zero_()
        engine.zero_grad()
        if args.pp > 1:
            runner.forward_backward(b, 1.0)  # the pipeline runner owns the micro-batch schedule
        else:
            model.loss_grad_scale = 1.0
            out = model(input_ids=b["input_ids"], labels=b["labels"], meta=meta)
            out.loss.backward()
        engine.step(3e-4)

    for b, m in list(zip(dev_batches, metas))[: max(W, 3)]:
        step_dev(b, m)
    sync_all()
    _lib.status_clear()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for b, m in zip(dev_batches, metas):
        step_dev(b, m)
    ev1.record()
    sync_all()
    dev_ms = ev0.elapsed_time(ev1)
    launches = _lib.launches() - launches0
    clocks = sampler.stop() if rank == 0 else {}
    _lib.assert_status_ok(sync=False)

    times = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(times[0]), float(times[1])
    tokens = SEQ_LEN * args.batch_size * (world // nd) * K
    mem = torch.cuda.max_memory_allocated(dev) / 2 ** 30
    mem_report = engine.memory_report() if hasattr(engine, "memory_report") else {}
    result = {
        "metric": "train tokens/s", "value": tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8 linear layers (tensor-wise e4m3 / e5m2), bf16 elsewhere" if args.float8 else "bf16",
        "data": "synthetic", "impl": "flame_b200",
        "config": {"name": args.config, "model": args.model, "global_batch": args.batch_size * (world // nd),
                   "seq_len": SEQ_LEN, "context_len": CONTEXT_LEN, "varlen": args.varlen,
                   "parallelism": f"fsdp{world // nd}" + (f"xtp{args.tp}" if args.tp > 1 else "")
                                  + (f"xpp{args.pp}" if args.pp > 1 else ""),
                   "fsdp_reshard_after_forward": args.reshard, "peak_memory_gib": round(mem, 2),
                   "param_grad_optimizer_gib": round(mem_report.get("total_bytes", 0.0) / 2 ** 30, 3),
                   "of_which_unsharded_gib": round(mem_report.get("staging_bytes", 0.0) / 2 ** 30, 3),
                   "optimizer": "AdamW fp32 master, clip 1.0" + (", state in pinned host memory" if args.cpu_offload else ""),
                   "activation_checkpoint": args.ac,
                   "l2": "256 MiB buffer written before every step; per-step working set is tens of GB",
                   "collectives": type(engine.collectives).__name__},
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / K,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "final_loss": losses[-1],
    }
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else {}


def run_reference(args) -> dict:
    from baseline.reference_arm import run as ref_run
    return ref_run(args, SEQ_LEN, CONTEXT_LEN, MODEL_JSON)


def main() -> None:
    global MODEL_JSON, SEQ_LEN
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    # the flags below select the other configs of the baseline table; the defaults are the flagship recipe
    ap.add_argument("--config", default="t340m", choices=sorted(PRESETS), help="a named configuration of the baseline table")
    ap.add_argument("--model", default=None, help="name of a file in configs/ (without .json)")
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--batch-size", type=int, default=None, help="rows per GPU and step")
    ap.add_argument("--varlen", dest="varlen", action="store_true", default=None)
    ap.add_argument("--no-varlen", dest="varlen", action="store_false", help="plain [batch, seq_len] rows, no document boundaries")
    ap.add_argument("--tp", type=int, default=None, help="tensor-parallel degree (the rest of the GPUs shard data)")
    ap.add_argument("--pp", type=int, default=None, help="pipeline-parallel degree")
    ap.add_argument("--ac", default=None, choices=["none", "full", "selective"], help="activation checkpointing mode")
    ap.add_argument("--ac-option", default=None,
                    help="selective option: 'op', 'mixer' (recompute only the chunk pipelines) or every N-th block")
    ap.add_argument("--reshard", default="never", choices=["default", "always", "never"],
                    help="fsdp_reshard_after_forward: never keeps the gathered parameters resident (fastest)")
    ap.add_argument("--cpu-offload", action="store_true", help="optimizer state in pinned host memory")
    ap.add_argument("--float8", action="store_true", help="linear layers on the fp8 GEMM (the result's dtype says so)")
    args = ap.parse_args()
    for key, val in PRESETS[args.config].items():
        if getattr(args, key) is None:
            setattr(args, key, val)
    if args.ac_option is None:
        args.ac_option = "2"
    MODEL_JSON = os.path.join(ROOT, "configs", args.model + ".json")
    SEQ_LEN = args.seq_len
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        try:
            res = run_reference(args)
        except Exception as e:  # the reference arm must never take the benchmark down
            import traceback
            traceback.print_exc()  # the whole error goes to stderr; the JSON line keeps its first and last lines
            lines = [l.strip() for l in str(e).splitlines() if l.strip()]
            brief = (lines[0][:160] + (" ... " + lines[-1][:160] if len(lines) > 1 else "")) if lines else ""
            res = {"impl": "reference", "unavailable": f"{type(e).__name__}: {brief}"}
    else:
        res = run_ours(args)
    if res:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
