"""Parallelism degrees and the device mesh.

Same contract as the reference's dependency (torchtitan/distributed/parallel_dims.py:20-234): degrees
``dp_replicate, dp_shard (-1 = whatever is left), cp, tp, pp`` whose product is the world size; mesh dimension
order ``pp, dp_replicate, dp_shard, cp, tp`` with only the dimensions larger than one materialised; derived
groups ``dp`` (data loading), ``dp_shard_cp`` (parameter sharding) and ``dp_cp`` (loss averaging).

Process groups are created directly with ``torch.distributed.new_group`` from the rank's coordinates, so the
same code serves NCCL on GPUs and gloo on CPUs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch.distributed as dist

ORDER = ("pp", "dp_replicate", "dp_shard", "cp", "tp")


@dataclass
class ParallelDims:
    dp_replicate: int = 1
    dp_shard: int = -1
    cp: int = 1
    tp: int = 1
    pp: int = 1
    world_size: int = 1
    enable_loss_parallel: bool = True
    _groups: Dict[str, Optional[dist.ProcessGroup]] = field(default_factory=dict, repr=False)
    _ranks: Dict[str, List[int]] = field(default_factory=dict, repr=False)
    _rank: int = 0

    def __post_init__(self) -> None:
        for name in ("dp_replicate", "cp", "tp", "pp"):
            assert getattr(self, name) >= 1, f"{name} must be >= 1"
        assert self.dp_shard == -1 or self.dp_shard >= 1, "dp_shard must be -1 or >= 1"
        if self.dp_shard == -1:
            rest = self.dp_replicate * self.cp * self.tp * self.pp
            assert self.world_size % rest == 0, f"world size {self.world_size} is not divisible by {rest}"
            self.dp_shard = self.world_size // rest
        prod = self.dp_replicate * self.dp_shard * self.cp * self.tp * self.pp
        assert prod == self.world_size, (
            f"dp_replicate({self.dp_replicate}) * dp_shard({self.dp_shard}) * cp({self.cp}) * tp({self.tp}) * "
            f"pp({self.pp}) != world_size({self.world_size})")

    # ---- properties mirroring the reference -----------------------------------------------------
    @property
    def dp_enabled(self) -> bool:
        return self.dp_replicate > 1 or self.dp_shard > 1

    @property
    def dp_replicate_enabled(self) -> bool:
        return self.dp_replicate > 1

    @property
    def dp_shard_enabled(self) -> bool:
        return self.dp_shard > 1

    @property
    def cp_enabled(self) -> bool:
        return self.cp > 1

    @property
    def tp_enabled(self) -> bool:
        return self.tp > 1

    @property
    def pp_enabled(self) -> bool:
        return self.pp > 1

    @property
    def loss_parallel_enabled(self) -> bool:
        return self.tp > 1 and self.enable_loss_parallel

    @property
    def non_data_parallel_size(self) -> int:
        return self.cp * self.tp * self.pp

    @property
    def seq_len_divisor(self) -> int:
        return self.tp * (self.cp * 2)

    @property
    def dp_degree(self) -> int:
        return self.dp_replicate * self.dp_shard

    def degrees(self) -> Dict[str, int]:
        return {n: getattr(self, n) for n in ORDER}

    # ---- coordinates --------------------------------------------------------------------------------
    def coords(self, rank: int) -> Dict[str, int]:
        out = {}
        rem = rank
        for name in reversed(ORDER):
            d = getattr(self, name)
            out[name] = rem % d
            rem //= d
        return out

    def rank_of(self, coords: Dict[str, int]) -> int:
        r = 0
        for name in ORDER:
            r = r * getattr(self, name) + coords[name]
        return r

    def _group_ranks(self, rank: int, over: Tuple[str, ...]) -> List[int]:
        """Ranks that share this rank's coordinates on every dimension not in ``over``."""
        base = self.coords(rank)
        ranks = []

        def rec(i: int, cur: Dict[str, int]) -> None:
            if i == len(over):
                ranks.append(self.rank_of(cur))
                return
            for v in range(getattr(self, over[i])):
                nxt = dict(cur)
                nxt[over[i]] = v
                rec(i + 1, nxt)

        rec(0, base)
        return sorted(ranks)

    GROUP_DEFS = {
        "pp": ("pp",), "dp_replicate": ("dp_replicate",), "dp_shard": ("dp_shard",), "cp": ("cp",), "tp": ("tp",),
        "dp": ("dp_replicate", "dp_shard"), "dp_shard_cp": ("dp_shard", "cp"),
        "dp_cp": ("dp_replicate", "dp_shard", "cp"),
    }

    def build_mesh(self, rank: Optional[int] = None) -> "ParallelDims":
        """Creates every process group (all ranks must call this in the same order).  A group of size one is
        represented by ``None``."""
        self._rank = dist.get_rank() if (rank is None and dist.is_initialized()) else (rank or 0)
        for name, over in self.GROUP_DEFS.items():
            size = 1
            for o in over:
                size *= getattr(self, o)
            mine: Optional[dist.ProcessGroup] = None
            my_ranks = self._group_ranks(self._rank, over)
            if size > 1 and dist.is_initialized():
                seen = set()
                for r in range(self.world_size):
                    ranks = tuple(self._group_ranks(r, over))
                    if ranks in seen:
                        continue
                    seen.add(ranks)
                    g = dist.new_group(list(ranks))
                    if self._rank in ranks:
                        mine = g
            self._groups[name] = mine
            self._ranks[name] = my_ranks
        return self

    def group(self, name: str) -> Optional[dist.ProcessGroup]:
        return self._groups.get(name)

    def group_ranks(self, name: str) -> List[int]:
        return self._ranks.get(name, [self._rank])

    def group_size(self, name: str) -> int:
        return len(self.group_ranks(name))

    def local_rank_in(self, name: str) -> int:
        return self.group_ranks(name).index(self._rank)

    @property
    def dp_rank(self) -> int:
        return self.local_rank_in("dp") if self._ranks else 0
