"""Memory estimation mode (``--memory_estimation.enabled``): what one rank needs, without training.

The reference hands this to torchtitan's estimator, which builds the model under FakeTensorMode with FSDP and reads a
memory tracker (flame/config_manager.py:824-835).  Here the two parts of the footprint are obtained separately:

* parameters, gradients and optimizer state: EXACT, from a dry build of the engine's flat-buffer layout for the requested
  parallel degrees (``ShardedEngine`` resident mode or ``ReshardingEngine`` sharded-parameter mode) on the meta device;
* activations: with ``--memory_estimation.disable_fake_mode`` on a machine with a GPU, one real training step is run and
  the allocator's peak is reported; otherwise a proxy of the model (same family and switches, two layers, hidden size
  256, a short row) runs on the CPU under ``saved_tensors_hooks``, and the bytes it saves per token, layer and hidden
  unit are scaled to the real sizes (activations grow linearly in all three; quadratic attention buffers of the CPU
  fallback are excluded by keeping the proxy's documents short).  The second figure is an estimate and is labelled so.

    python -m flame_b200.tools.estimate_memory --job.config_file flame_b200/models/fla.toml --model.config configs/transformer_340M.json \
        --training.seq_len 65536 --training.varlen --training.data_parallel_shard_degree 8
"""
from __future__ import annotations

import copy
import json
import os
from typing import Dict

import torch

from ..config_manager import TORCH_DTYPE_MAP, JobConfig
from ..models import ModelConfig, build_model

GiB = float(1 << 30)


def state_bytes(model_config: ModelConfig, shard_degree: int, policy: str, param_dtype: torch.dtype = torch.bfloat16) -> Dict[str, float]:
    """Parameter / gradient / optimizer bytes per rank from a dry build of the engine layout (no allocation of note)."""
    from ..parallel.engine import ShardedEngine
    from ..parallel.resharding import ReshardingEngine
    model = build_model(model_config, device="meta", dtype=param_dtype, init=False)
    sharded = policy in ("default", "always") and shard_degree > 1
    cls = ReshardingEngine if sharded else ShardedEngine
    eng = cls.__new__(cls)
    eng.model, eng.device, eng.param_dtype = model, torch.device("meta"), param_dtype
    eng.shard_world, eng.shard_rank, eng.units = shard_degree, 0, []
    eng.cpu_offload = False
    eng._alloc = lambda n, dt, tag: torch.empty(n, dtype=dt, device="meta")
    eng._build()
    rep = eng.memory_report()
    rep["parameters"] = float(sum(p.numel() for p in model.parameters()))
    return rep


def _saved_bytes(model, ids, cu) -> int:
    total = 0
    seen = set()

    def pack(t):
        nonlocal total
        key = (t.untyped_storage().data_ptr(), t.storage_offset(), tuple(t.shape))
        if not isinstance(t, torch.nn.Parameter) and key not in seen:
            seen.add(key)
            total += t.numel() * t.element_size()
        return t

    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        out = model(input_ids=ids, labels=ids, cu_seqlens=cu)
    out.loss.backward()
    return total


def activation_bytes_estimate(model_config: ModelConfig, tokens: int, bytes_per_element: int = 2) -> float:
    """Saved-activation bytes of one micro-batch, scaled up from a small CPU proxy of the same family."""
    small = copy.deepcopy(model_config)
    h0 = 256
    ratio = h0 / float(model_config.hidden_size)
    small.hidden_size = h0
    for key in ("num_heads", "num_kv_heads", "num_v_heads"):
        v = small.get(key)
        if isinstance(v, int) and v > 0:
            setattr(small, key, max(1, int(round(v * ratio))))
    if small.get("intermediate_size"):
        small.intermediate_size = max(64, int(small.intermediate_size * ratio) // 64 * 64)
    small.vocab_size = 512
    T, doc = 256, 32
    cu = torch.arange(0, T + 1, doc, dtype=torch.int32)
    per_layer = []
    for layers in (1, 3):
        small.num_hidden_layers = layers
        if isinstance(small.get("attn"), dict):
            small.attn = dict(small.attn, layers=[i for i in small.attn.get("layers", []) if i < layers],
                              num_heads=4, num_kv_heads=4)
        m = build_model(small, device="cpu", dtype=torch.float32, init=True, seed=0)
        m.train()
        ids = torch.randint(3, 512, (1, T))
        per_layer.append(_saved_bytes(m, ids, cu))
    block = (per_layer[1] - per_layer[0]) / 2.0            # bytes one decoder block saves for T proxy tokens in fp32
    rest = per_layer[0] - block                             # embeddings, final norm, head
    coeff = block / (T * h0 * 4.0)                          # saved ELEMENTS per token and hidden unit
    blocks = coeff * tokens * model_config.hidden_size * bytes_per_element * model_config.num_hidden_layers
    head = (rest / (T * h0 * 4.0)) * tokens * model_config.hidden_size * bytes_per_element
    return blocks + head


def estimate(job_config: JobConfig, world_size: int = 1) -> Dict[str, float]:
    tr = job_config.training
    cfg = ModelConfig.from_pretrained(job_config.model.config)
    nd = max(1, tr.tensor_parallel_degree) * max(1, job_config.experimental.pipeline_parallel_degree) * \
        max(1, job_config.experimental.context_parallel_degree)
    shard = tr.data_parallel_shard_degree
    if shard in (-1, 0):
        shard = max(1, world_size // (nd * max(1, tr.data_parallel_replicate_degree)))
    dtype = TORCH_DTYPE_MAP[tr.mixed_precision_param]
    rep = state_bytes(cfg, shard, tr.fsdp_reshard_after_forward, dtype)
    tokens = tr.batch_size * tr.seq_len
    ac = job_config.activation_checkpoint.mode
    act = activation_bytes_estimate(cfg, tokens)
    if ac == "full":
        act = act / max(1, cfg.num_hidden_layers) * 2 + tokens * cfg.hidden_size * 2 * cfg.num_hidden_layers
    elif ac == "selective":
        act *= 0.5
    out = {"parameters": rep["parameters"], "shard_degree": float(shard), "mode": rep["mode"],
           "state_gib": rep["total_bytes"] / GiB, "sharded_state_gib": rep["sharded_bytes"] / GiB,
           "staging_or_resident_gib": rep["staging_bytes"] / GiB, "activations_gib_estimate": act / GiB,
           "total_gib_estimate": (rep["total_bytes"] + act) / GiB}
    if job_config.memory_estimation.disable_fake_mode and torch.cuda.is_available():
        out["measured_peak_gib"] = measure_one_step(job_config)
    return out


def measure_one_step(job_config: JobConfig) -> float:
    """One real forward / backward / optimizer step on this GPU; the allocator's peak."""
    from ..parallel.dims import ParallelDims
    from ..parallel.engine import OptimConfig, ShardedEngine
    from ..ops.varlen import VarlenMeta
    tr = job_config.training
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = ModelConfig.from_pretrained(job_config.model.config)
    model = build_model(cfg, device="meta", dtype=torch.bfloat16, init=False)
    eng = ShardedEngine(model, ParallelDims(world_size=1), dev, torch.bfloat16, OptimConfig())
    eng.init_weights(0)
    model.train()
    torch.cuda.reset_peak_memory_stats(dev)
    ids = torch.randint(3, cfg.vocab_size, (tr.batch_size, tr.seq_len), device=dev)
    meta = VarlenMeta.dense(tr.batch_size, tr.seq_len, dev)
    eng.zero_grad()
    model(input_ids=ids, labels=ids, meta=meta).loss.backward()
    eng.step(1e-4)
    torch.cuda.synchronize()
    return torch.cuda.max_memory_allocated(dev) / GiB


def main() -> None:
    cfg = JobConfig().parse_args()
    world = int(os.environ.get("WORLD_SIZE", os.environ.get("NGPU", 1)))
    print(json.dumps(estimate(cfg, world), indent=2))


if __name__ == "__main__":
    main()
