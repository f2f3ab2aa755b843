from .dims import ParallelDims
from .engine import OptimConfig, ShardedEngine

__all__ = ["ParallelDims", "OptimConfig", "ShardedEngine"]
