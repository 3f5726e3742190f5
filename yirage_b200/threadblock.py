"""TBGraph: thread-block graph wrapper (python/yirage/threadblock.py).  On the persistent
kernel path a thread-block graph is only a list of operands with their grid partition
maps, so that is all this wrapper forwards."""
from .core import CyTBGraph, DTensor


class TBGraph:
    def __init__(self, graph: CyTBGraph):
        self.cygraph = graph

    def new_input(self, dtensor: DTensor, input_map: tuple, forloop_dim: int,
                  store_in_dmem: bool = False):
        return self.cygraph.new_input(dtensor, input_map, forloop_dim, store_in_dmem)

    @property
    def grid_dim(self):
        return self.cygraph.grid_dim

    @property
    def block_dim(self):
        return self.cygraph.block_dim
