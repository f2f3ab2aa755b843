"""Tensor parallelism with sequence parallelism for packed ``[T, D]`` activations.

Plan (same split as the reference's TP plans, flame/models/parallelize_fla.py:111-280): embeddings row-wise over the
vocabulary with a sequence-sharded output; every norm runs on the rank's ``T / tp`` rows; q/k/v (+ gate projections)
and the MLP's gate/up are column-parallel behind an all-gather of the rows; ``o_proj`` and ``down_proj`` are
row-parallel in front of a reduce-scatter; the head is column-parallel over the vocabulary with a vocabulary-parallel
loss.  Supported families: ``transformer`` and ``gla`` (the two the reference has plans for).

Collective + GEMM pairs run as ONE kernel each on CUDA (``csrc/gemm.cu``):

* all-gather -> GEMM: copy CTAs inside the GEMM launch pull the peers' row shards over NVLink into the local full
  matrix chunk by chunk while the tensor-core CTAs start on the local shard and pick up remote chunks as their flags
  appear (``fb_gemm_allgather_a``);
* GEMM -> reduce-scatter: the epilogue stores each output row straight into the owner rank's receive slot, remote rows
  first (``fb_gemm_scatter_rows``); a small kernel sums the slots.

On CPU (gloo) the same autograd functions use c10d collectives, which is what the world-size-2 plumbing tests run.
"""
from __future__ import annotations

from ctypes import c_double, c_float, c_int, c_longlong, c_void_p
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..components.metrics import logger
from ..ops import _lib
from ..ops.gemm import gemm_nn, gemm_nt, gemm_tn
from ..ops.linear import _adjacent, _cat_view
from .dims import ParallelDims

vp, i32, i64 = c_void_p, c_int, c_longlong
_lib.register("fb_gemm_allgather_a", [vp, i32, i32, i32, i64, vp, vp, vp, i32, vp, vp, i32, i32, i64, i64, i32, vp])
_lib.register("fb_gemm_scatter_rows", [vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i32, vp])
_lib.register("fb_sum_slots", [vp, i32, i64, i64, vp, vp])
_lib.register("fb_peer_signal", [vp, i32, i32, i32, i32, vp])
_lib.register("fb_peer_wait", [vp, i32, i32, i32, c_double, vp])
_lib.register("fb_ce_vp_stats", [vp, vp, vp, i64, i32, i64, i64, i32, vp])
_lib.register("fb_ce_vp_grad", [vp, vp, vp, vp, c_float, i64, i32, i64, i64, i32, vp])

_CTX: Optional["TPContext"] = None


def tp_context() -> Optional["TPContext"]:
    return _CTX


class TPContext:
    """Per-process tensor-parallel state: group, rank, and (on CUDA) the symmetric staging buffers and flags."""

    def __init__(self, dims: ParallelDims, device: torch.device) -> None:
        self.group = dims.group("tp")
        self.world = dims.tp
        self.rank = dims.local_rank_in("tp")
        self.device = device
        self.fused = False
        self.rows = 0
        self.width = 0
        self._epoch = [0, 0, 0, 0]
        self._turn_ag = 0
        self._turn_rs = 0

    # ---- fused path set-up (lazy: needs the row count of a micro-batch) ----------------------------------------
    def ensure_buffers(self, rows_per_rank: int, width: int) -> bool:
        if self.device.type != "cuda" or not _lib.available():
            return False
        if rows_per_rank % 128 != 0 or width % 8 != 0:
            return False
        if self.fused and rows_per_rank <= self.rows and width <= self.width:
            return True
        try:
            import torch.distributed._symmetric_memory as symm_mem
            self.rows, self.width = rows_per_rank, width
            self.send, self.recv, self._send_ptrs, self._recv_ptrs = [], [], [], []
            for _ in range(2):
                s = symm_mem.empty(rows_per_rank * width, dtype=torch.bfloat16, device=self.device)
                h = symm_mem.rendezvous(s, self.group)
                self.send.append(s)
                self._send_ptrs.append(torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64).numpy().astype("uint64"))
                r = symm_mem.empty(self.world * rows_per_rank * width, dtype=torch.bfloat16, device=self.device)
                h2 = symm_mem.rendezvous(r, self.group)
                self.recv.append(r)
                self._recv_ptrs.append(torch.tensor([int(p) for p in h2.buffer_ptrs], dtype=torch.int64).numpy().astype("uint64"))
            f = symm_mem.empty(4 * 16, dtype=torch.int32, device=self.device)
            f.zero_()
            hf = symm_mem.rendezvous(f, self.group)
            self.flags = f
            self._flag_ptrs = torch.tensor([int(p) for p in hf.buffer_ptrs], dtype=torch.int64).numpy().astype("uint64")
            self.chunk_flags = [torch.zeros(4096, dtype=torch.int32, device=self.device) for _ in range(2)]
            self._epoch = [0, 0, 0, 0]
            torch.cuda.synchronize()
            dist.barrier(group=self.group, device_ids=[self.device.index])
            self.fused = True
        except Exception as e:  # symmetric memory unavailable: c10d collectives
            logger.warning(f"fused tensor-parallel kernels unavailable ({e!r}); using NCCL collectives")
            self.fused = False
        return self.fused

    # ---- fused all-gather -> GEMM -----------------------------------------------------------------------------
    def allgather_gemm(self, x_s: torch.Tensor, w: torch.Tensor, b_mn: bool, n_out: int) -> tuple:
        """Returns (y [T, n_out], x_full [T, K]).  ``w`` is [n_out, K] (b_mn False) or [K, n_out] (b_mn True)."""
        L = _lib.lib()
        rows, K = x_s.shape
        buf = self._turn_ag
        self._turn_ag ^= 1
        self._epoch[buf] += 1
        ep = self._epoch[buf]
        send = self.send[buf][: rows * K].view(rows, K)
        send.copy_(x_s)
        st = _lib.stream_ptr()
        _lib.check(L.fb_peer_signal(self._flag_ptrs.ctypes.data, self.world, self.rank, buf, ep, st), "fb_peer_signal")
        T = rows * self.world
        x_full = torch.empty(T, K, dtype=x_s.dtype, device=x_s.device)
        y = torch.empty(T, n_out, dtype=x_s.dtype, device=x_s.device)
        rc = L.fb_gemm_allgather_a(self._send_ptrs[buf].ctypes.data, self.world, self.rank, rows, K, x_full.data_ptr(),
                                   self.chunk_flags[buf].data_ptr(), self.flags.data_ptr() + buf * 16 * 4, ep, w.data_ptr(),
                                   y.data_ptr(), n_out, K, w.stride(0), y.stride(0), 1 if b_mn else 0, st)
        _lib.check(rc, "fb_gemm_allgather_a")
        _lib.count_launch(2)
        return y, x_full

    # ---- fused GEMM -> reduce-scatter ---------------------------------------------------------------------------
    def gemm_reduce_scatter(self, a: torch.Tensor, w: torch.Tensor, b_mn: bool, n_out: int) -> torch.Tensor:
        """a [T, K] (local partial operand), ``w`` as above -> y_s [T / world, n_out] summed over the ranks."""
        L = _lib.lib()
        T, K = a.shape
        rows = T // self.world
        buf = self._turn_rs
        self._turn_rs ^= 1
        slot = 2 + buf
        self._epoch[slot] += 1
        ep = self._epoch[slot]
        st = _lib.stream_ptr()
        rc = L.fb_gemm_scatter_rows(a.data_ptr(), w.data_ptr(), self._recv_ptrs[buf].ctypes.data, self.world, self.rank, rows,
                                    n_out, K, a.stride(0), w.stride(0), n_out, 1 if b_mn else 0, st)
        _lib.check(rc, "fb_gemm_scatter_rows")
        _lib.check(L.fb_peer_signal(self._flag_ptrs.ctypes.data, self.world, self.rank, slot, ep, st), "fb_peer_signal")
        _lib.check(L.fb_peer_wait(self.flags.data_ptr(), self.world, slot, ep, _lib.peer_wait_seconds(), st), "fb_peer_wait")
        out = torch.empty(rows, n_out, dtype=a.dtype, device=a.device)
        rc = L.fb_sum_slots(self.recv[buf].data_ptr(), self.world, rows * n_out, rows * n_out, out.data_ptr(), st)
        _lib.check(rc, "fb_sum_slots")
        _lib.count_launch(4)
        return out

    # ---- c10d fall-backs ----------------------------------------------------------------------------------------
    def all_gather_rows(self, x_s: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(x_s) for _ in range(self.world)]
        dist.all_gather(parts, x_s.contiguous(), group=self.group)
        return torch.cat(parts, 0)

    def reduce_scatter_rows(self, y: torch.Tensor) -> torch.Tensor:
        y = y.contiguous()
        rows = y.shape[0] // self.world
        if dist.get_backend(self.group) == "gloo":
            dist.all_reduce(y, group=self.group)
            return y[self.rank * rows:(self.rank + 1) * rows].clone()
        out = torch.empty(rows, *y.shape[1:], dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out, y, group=self.group)
        return out

    def all_reduce(self, t: torch.Tensor, op=dist.ReduceOp.SUM) -> torch.Tensor:
        dist.all_reduce(t, op=op, group=self.group)
        return t


# --------------------------------------------------------------------------------------------------------------
# autograd functions
# --------------------------------------------------------------------------------------------------------------
def _weights_view(weights: Sequence[torch.Tensor]) -> Optional[torch.Tensor]:
    ws = [w.detach() for w in weights]
    if len(ws) == 1:
        return ws[0]
    return _cat_view(ws) if _adjacent(ws) else None


class _AllGatherLinear(torch.autograd.Function):
    """y = all_gather_rows(x_s) @ cat(weights).T with column-parallel weights; backward reduce-scatters dx."""

    @staticmethod
    def forward(ctx, x_s, *weights):
        tp = tp_context()
        n_out = sum(w.shape[0] for w in weights)
        wcat = _weights_view(weights)
        if wcat is None:
            wcat = torch.cat([w.detach() for w in weights], 0)
        if tp.ensure_buffers(x_s.shape[0], x_s.shape[1]) and x_s.dtype == torch.bfloat16:
            y, x_full = tp.allgather_gemm(x_s, wcat, False, n_out)
        else:
            x_full = tp.all_gather_rows(x_s)
            y = gemm_nt(x_full, wcat)
        ctx.save_for_backward(x_full, *weights)
        return y

    @staticmethod
    def backward(ctx, dy):
        tp = tp_context()
        x_full, *weights = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        wcat = _weights_view(weights)
        if wcat is None:
            wcat = torch.cat([w.detach() for w in weights], 0)
        K = x_full.shape[1]
        if tp.fused and dy.dtype == torch.bfloat16 and tp.ensure_buffers(x_full.shape[0] // tp.world, K):
            dx_s = tp.gemm_reduce_scatter(dy, wcat, True, K)
        else:
            dx_s = tp.reduce_scatter_rows(gemm_nn(dy, wcat))
        grads = _weight_grads(dy, x_full, weights)
        return (dx_s, *grads)


class _LinearReduceScatter(torch.autograd.Function):
    """y_s = reduce_scatter_rows(a @ weight.T) with a row-parallel weight [out, in / tp]."""

    @staticmethod
    def forward(ctx, a, weight):
        tp = tp_context()
        a = a if a.is_contiguous() else a.contiguous()
        n_out = weight.shape[0]
        if a.dtype == torch.bfloat16 and tp.ensure_buffers(a.shape[0] // tp.world, n_out):
            y_s = tp.gemm_reduce_scatter(a, weight.detach(), False, n_out)
        else:
            y_s = tp.reduce_scatter_rows(gemm_nt(a, weight.detach()))
        ctx.save_for_backward(a, weight)
        return y_s

    @staticmethod
    def backward(ctx, dy_s):
        tp = tp_context()
        a, weight = ctx.saved_tensors
        dy_s = dy_s if dy_s.is_contiguous() else dy_s.contiguous()
        n_in = weight.shape[1]
        if tp.fused and dy_s.dtype == torch.bfloat16 and tp.ensure_buffers(dy_s.shape[0], dy_s.shape[1]):
            da, dy_full = tp.allgather_gemm(dy_s, weight.detach(), True, n_in)
        else:
            dy_full = tp.all_gather_rows(dy_s)
            da = gemm_nn(dy_full, weight.detach())
        (gw,) = _weight_grads(dy_full, a, [weight])
        return da, gw


def _weight_grads(dy: torch.Tensor, x: torch.Tensor, weights: Sequence[torch.Tensor]) -> List[Optional[torch.Tensor]]:
    grads: List[Optional[torch.Tensor]] = [None] * len(weights)
    mgs = [getattr(w, "main_grad", None) for w in weights]
    if all(m is not None for m in mgs):
        if len(weights) == 1 or _adjacent(mgs):
            mg = mgs[0] if len(weights) == 1 else _cat_view(mgs)
            gemm_tn(dy, x, out=mg, accumulate=True)
        else:
            c = 0
            for w, m in zip(weights, mgs):
                gemm_tn(dy[:, c:c + w.shape[0]], x, out=m, accumulate=True)
                c += w.shape[0]
    else:
        c = 0
        for i, w in enumerate(weights):
            grads[i] = gemm_tn(dy[:, c:c + w.shape[0]], x, out_dtype=torch.float32).to(w.dtype)
            c += w.shape[0]
    return grads


def allgather_linear(x_s: torch.Tensor, weights: Sequence[torch.Tensor]) -> torch.Tensor:
    return _AllGatherLinear.apply(x_s, *weights)


def linear_reduce_scatter(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return _LinearReduceScatter.apply(a, weight)


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_s):
        return tp_context().all_gather_rows(x_s)

    @staticmethod
    def backward(ctx, dy):
        return tp_context().reduce_scatter_rows(dy)


class _ScatterRowsSum(torch.autograd.Function):
    """reduce-scatter of per-rank partial rows (forward), all-gather in backward."""

    @staticmethod
    def forward(ctx, y):
        return tp_context().reduce_scatter_rows(y)

    @staticmethod
    def backward(ctx, dy_s):
        return tp_context().all_gather_rows(dy_s)


# --------------------------------------------------------------------------------------------------------------
# vocabulary-parallel pieces
# --------------------------------------------------------------------------------------------------------------
class _VocabParallelCE(torch.autograd.Function):
    """Mean cross-entropy over vocabulary-sharded logits (max / sum-exp / target logit reduced over the group)."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, ignore_index, grad_scale):
        tp = tp_context()
        if (_lib.available() and logits.is_cuda and logits.dtype == torch.bfloat16 and logits.is_contiguous()
                and logits.shape[1] % 8 == 0):
            return _VocabParallelCE._forward_kernels(ctx, tp, logits, labels.contiguous(), vocab_start, ignore_index,
                                                     grad_scale)
        lf = logits.float()
        m = lf.max(-1).values
        tp.all_reduce(m, dist.ReduceOp.MAX)
        e = (lf - m[:, None]).exp()
        s = e.sum(-1)
        tp.all_reduce(s)
        V = logits.shape[1]
        local = labels - vocab_start
        mine = (local >= 0) & (local < V) & (labels != ignore_index)
        tgt = torch.zeros_like(m)
        idx = local.clamp(0, V - 1)
        tgt[mine] = lf.gather(1, idx[:, None]).squeeze(1)[mine]
        tp.all_reduce(tgt)
        valid = labels != ignore_index
        n = valid.sum().clamp_min(1)
        loss = ((m + s.log() - tgt) * valid).sum() / n
        p = e / s[:, None]
        p[mine, idx[mine]] -= 1.0
        p = p * (valid[:, None].float() * (grad_scale / n))
        ctx.save_for_backward(p.to(logits.dtype))
        return loss

    @staticmethod
    def _forward_kernels(ctx, tp, logits, labels, vocab_start, ignore_index, grad_scale):
        """Two kernels and ONE collective: per-row statistics of the local slice, an all-gather of ``[rows, 3]`` floats,
        then the gradient written in place over the logits (no fp32 copy of the ``[rows, V / tp]`` slice)."""
        L = _lib.lib()
        T, V = logits.shape
        st = _lib.stream_ptr()
        stats = torch.empty(T, 3, dtype=torch.float32, device=logits.device)
        _lib.check(L.fb_ce_vp_stats(logits.data_ptr(), labels.data_ptr(), stats.data_ptr(), T, V, logits.stride(0),
                                    int(vocab_start), ignore_index, st), "fb_ce_vp_stats")
        allst = torch.empty(tp.world, T, 3, dtype=torch.float32, device=logits.device)
        dist.all_gather_into_tensor(allst, stats, group=tp.group)
        m = allst[..., 0].max(0).values
        s = (allst[..., 1] * (allst[..., 0] - m).exp()).sum(0)
        lse = (m + s.log()).contiguous()
        tgt = allst[..., 2].sum(0)
        valid = labels != ignore_index
        n_valid = valid.sum().clamp_min(1).to(torch.int32).reshape(1)
        loss = ((lse - tgt) * valid).sum() / n_valid[0]
        _lib.check(L.fb_ce_vp_grad(logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), n_valid.data_ptr(),
                                   float(grad_scale), T, V, logits.stride(0), int(vocab_start), ignore_index, st),
                   "fb_ce_vp_grad")
        _lib.count_launch(2)
        ctx.save_for_backward(logits)   # now the gradient, in place (the logits of the head are not used again)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        (p,) = ctx.saved_tensors
        return p * dloss.to(p.dtype), None, None, None, None


def vocab_parallel_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, vocab_start: int, ignore_index: int = -100,
                                 grad_scale: float = 1.0) -> torch.Tensor:
    return _VocabParallelCE.apply(logits, labels, vocab_start, ignore_index, grad_scale)


# --------------------------------------------------------------------------------------------------------------
# module surgery
# --------------------------------------------------------------------------------------------------------------
def _shard_param(mod: nn.Module, name: str, dim: int, rank: int, world: int) -> None:
    p = getattr(mod, name)
    shape = list(p.shape)
    assert shape[dim] % world == 0, f"{name}{tuple(shape)} is not divisible by tp={world} on dim {dim}"
    shape[dim] //= world
    newp = nn.Parameter(torch.empty(shape, dtype=p.dtype, device=p.device), requires_grad=True)
    newp._tp = (dim, rank, world)
    for attr in ("_no_weight_decay",):
        if hasattr(p, attr):
            setattr(newp, attr, getattr(p, attr))
    mod._parameters[name] = newp


def _mark_replicated(p: nn.Parameter) -> None:
    p._tp_replicated = True


def apply_tensor_parallel(model, model_config, dims: ParallelDims, job_config=None) -> TPContext:
    """Rewrites the (meta-device) model in place for tensor + sequence parallelism."""
    global _CTX
    mt = model_config.model_type
    if mt not in ("transformer", "gla"):
        raise NotImplementedError(f"tensor parallelism has plans for 'transformer' and 'gla', not for {mt!r}")
    from ..models import layers as Lyr
    from ..models.modules import GatedMLP
    dev = next(model.parameters()).device
    tp = TPContext(dims, torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    _CTX = tp
    r, w = tp.rank, tp.world
    dec = model.decoder
    _shard_param(dec.embeddings, "weight", 0, r, w)
    dec.embeddings.tp = tp
    _shard_param(model.lm_head, "weight", 0, r, w)
    model.tp = tp
    for blk in dec.layers:
        if blk is None:
            continue
        for n in ("attn_norm", "mlp_norm"):
            nm = getattr(blk, n)
            if nm.weight is not None:
                _mark_replicated(nm.weight)
        mlp = blk.mlp
        for n in ("gate_proj", "up_proj"):
            _shard_param(getattr(mlp, n), "weight", 0, r, w)
        _shard_param(mlp.down_proj, "weight", 1, r, w)
        mlp.tp = tp
        attn = blk.attn
        if isinstance(attn, Lyr.Attention):
            assert attn.num_heads % w == 0 and attn.num_kv_heads % w == 0, "heads must divide by the tp degree"
            for n in ("q_proj", "k_proj", "v_proj"):
                _shard_param(getattr(attn, n), "weight", 0, r, w)
            _shard_param(attn.o_proj, "weight", 1, r, w)
            attn.num_heads //= w
            attn.num_kv_heads //= w
            attn.tp = tp
        elif isinstance(attn, Lyr.GatedLinearAttention):
            assert attn.num_heads % w == 0 and attn.num_kv_heads % w == 0
            for n in ("q_proj", "k_proj", "v_proj"):
                _shard_param(getattr(attn, n), "weight", 0, r, w)
            if attn.use_output_gate:
                _shard_param(attn.g_proj, "weight", 0, r, w)
            _mark_replicated(attn.gk_proj[0].weight)
            _shard_param(attn.gk_proj[1], "weight", 0, r, w)
            _shard_param(attn.gk_proj[1], "bias", 0, r, w)
            _shard_param(attn.o_proj, "weight", 1, r, w)
            norm = attn.g_norm_swish_gate if attn.fuse_norm_and_gate else attn.g_norm
            if norm.weight is not None:
                _mark_replicated(norm.weight)
            attn.num_heads //= w
            attn.num_kv_heads //= w
            attn.key_dim //= w
            attn.value_dim //= w
            attn.tp = tp
        else:
            raise NotImplementedError(type(attn).__name__)
    fn = dec.final_norm
    if fn is not None and fn.weight is not None:
        _mark_replicated(fn.weight)
    logger.info(f"Applied tensor parallelism (degree {w}) with sequence-parallel norms and a vocabulary-parallel head")
    return tp
