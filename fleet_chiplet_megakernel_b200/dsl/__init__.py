"""The Fleet task DSL over ``PersistentKernel`` (python/mirage/mpk/dsl of the reference): a graph session,
op functions and decorators that carry scheduling metadata."""
from .graph import Graph, Tensor
from .ops import (rmsnorm, embed, linear, linear_silu, silu_mul, silu_mul_linear, argmax, paged_attention_split_kv,
                  paged_attention)
from .cost_model import select_strategy, select_k_splits
from .decorators import task, distribute, affinity, get_meta, strategy_from_meta
from .types import Tile, Partition, Chunk

__all__ = ["Graph", "Tensor", "rmsnorm", "embed", "linear", "linear_silu", "silu_mul", "silu_mul_linear", "argmax",
           "paged_attention_split_kv", "paged_attention", "select_strategy", "select_k_splits", "task", "distribute",
           "affinity", "get_meta", "strategy_from_meta", "Tile", "Partition", "Chunk"]
