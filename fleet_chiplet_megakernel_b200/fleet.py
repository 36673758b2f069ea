"""``fleet``: the task-specification API of the reference (python/mirage/mpk/fleet.py) on the B200 runtime.

    import fleet_chiplet_megakernel_b200.fleet as fleet

    @fleet.task(level="gpu", tiling="split_k")            # the reference's level="xcd" is accepted too
    def down_proj(x, w, out, res):
        return fleet.ops.linear(x, w, out, residual=res, strategy=fleet.strategy_from_meta(fleet.get_meta(down_proj)))

    g = fleet.Graph(mpk)
    x = g.input(tensor, "x"); out = g.intermediate((tokens, hidden), name="out")
"""
from .dsl.decorators import task, distribute, affinity, get_meta, strategy_from_meta
from .dsl.types import Tile, Partition, Chunk
from .dsl.graph import Graph, Tensor
from .dsl import ops
from .dsl.cost_model import select_strategy, select_k_splits

__all__ = ["task", "distribute", "affinity", "get_meta", "strategy_from_meta", "Tile", "Partition", "Chunk", "Graph",
           "Tensor", "ops", "select_strategy", "select_k_splits"]
