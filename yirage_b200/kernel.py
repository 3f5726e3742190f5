"""KNGraph: the kernel-graph surface (`yirage.new_kernel_graph()`), as in
python/yirage/kernel.py:249-321,584,1260-1284.

Two uses survive on the B200 path:
  * the micro-graphs of the reference benchmarks (benchmark/rmsnorm.py,
    benchmark/gated_mlp.py): new_input / rms_norm / matmul / silu / mul / mark_output,
    then superoptimize() and a call with torch tensors.  The search is gone: superoptimize
    matches the graph against the hand-written fused kernels (micrograph.py) and fails
    loudly when nothing matches;
  * the persistent-kernel builders, which go through customized() / register_task() /
    attach_* / shuffle_tensors and end in generate_task_graph().
"""
from typing import List, Optional

import torch

from .core import (CyKNGraph, CyTBGraph, DTensor, bfloat16, convert_torch_type_to_dtype, dtype,
                   float16)
from .lowering import RegisteredTask
from .threadblock import TBGraph


def check_stride(dims, strides, layout="row-major"):
    curr_stride = 1
    if layout == "row-major":
        for i in range(len(dims) - 1, -1, -1):
            if strides[i] != curr_stride:
                return False
            curr_stride *= dims[i]
    elif layout == "column-major":
        for i in range(len(dims)):
            if strides[i] != curr_stride:
                return False
            curr_stride *= dims[i]
    return True


class KNGraph:
    def __init__(self, graph: CyKNGraph):
        self.cygraph = graph
        self._is_compiled = False
        self.run = None
        self._valid_cuda_kernels = False
        self._cached_results = None
        self.visualizer = None
        self.backend = "cuda"
        self._executor = None
        self._task_graph_hook = None   # set by PersistentKernel

    # ------------------------------------------------------------------ graph building
    def new_input(self, dims: tuple, strides: tuple = None, dtype: dtype = float16) -> DTensor:
        if strides is not None:
            assert len(dims) == len(strides)
            assert check_stride(dims, strides, "row-major") | check_stride(
                dims, strides, "column-major")
        return self.cygraph.new_input(dims, strides, dtype)

    def mark_output(self, A: DTensor, strides: tuple = None):
        return self.cygraph.mark_output(A, strides)

    def matmul(self, A: DTensor, B: DTensor) -> DTensor:
        return self.cygraph.matmul(A, B)

    def rms_norm(self, A: DTensor, normalized_shape: tuple):
        return self.cygraph.rms_norm(A, normalized_shape)

    def silu(self, A: DTensor):
        return self.cygraph.silu(A)

    def mul(self, A: DTensor, B: DTensor):
        return self.cygraph.mul(A, B)

    def add(self, A: DTensor, B: DTensor):
        return self.cygraph.add(A, B)

    def customized(self, inputs: List[DTensor], bgraph: TBGraph) -> List[DTensor]:
        return self.cygraph.customized(inputs, bgraph.cygraph)

    # ------------------------------------------------------------ persistent-kernel hooks
    def attach_torch_tensor(self, t: DTensor, torch_tensor: torch.Tensor, name: str):
        t.kind, t.name, t.torch_tensor = "torch", name, torch_tensor

    def attach_cuda_tensor(self, t: DTensor, name: str):
        t.kind, t.name = "cuda", name

    def attach_nvshmem_tensor(self, t: DTensor, name: str):
        t.kind, t.name = "nvshmem", name

    def fuse_tensors(self, inputs: List[DTensor], fused_dim: int, num_groups: int, name: str = None):
        raise NotImplementedError("fuse_tensors is not on the decode hot path; use shuffle_tensors")

    def shuffle_tensors(self, inputs: List[DTensor], shuffled_dim: int, num_groups: int,
                        name: str = None):
        """New tensor whose rows interleave the inputs group by group
        (src/kernel/graph.cc:398-437); materialised at compile time."""
        assert shuffled_dim == 0
        first = inputs[0]
        for t in inputs:
            if t.num_dims != first.num_dims or t.dims[1:] != first.dims[1:] or t.dtype != first.dtype:
                raise ValueError("shuffle_tensors: inputs must agree on all but dimension 0")
            if t.dims[0] % num_groups:
                raise ValueError("shuffle_tensors: rows must be divisible by num_groups")
        dims = (sum(t.dims[0] for t in inputs),) + tuple(first.dims[1:])
        out = self.cygraph.new_input(dims, None, first.dtype)
        out.kind, out.name = "shuffled", name
        out.sources, out.num_groups = list(inputs), num_groups
        return out

    def register_task(self, bgraph: TBGraph, task_type: str, params: Optional[List[int]] = None,
                      **attrs):
        cy: CyTBGraph = bgraph.cygraph
        # validates the partition maps the way TBInputOp does (input_loader.cc:84-110)
        for inp in cy.inputs:
            cy.tile_dims(inp)
        self.cygraph.tasks.append(RegisteredTask(
            task_type, [inp.dtensor for inp in cy.inputs], cy.grid_dim, cy.block_dim,
            list(params or []), dict(attrs)))

    def generate_task_graph(self, num_gpus: int, my_gpu_id: int):
        if self._task_graph_hook is None:
            raise RuntimeError("generate_task_graph needs a PersistentKernel around the graph")
        return self._task_graph_hook(num_gpus, my_gpu_id)

    # ---------------------------------------------------------------- micro-graph execution
    def superoptimize(self, **kwargs):
        """The reference searches for a fast muGraph here (kernel.py:584-1247).  The B200
        build has no search: the graph is matched against the fused kernels that exist and
        compiled into a one-pass task graph.  Unknown keyword arguments of the reference
        signature (config, backend, warmup_iters, ...) are accepted and ignored."""
        from .micrograph import MicroGraphExecutor
        self._executor = MicroGraphExecutor(self.cygraph)
        self._is_compiled = True
        self._valid_cuda_kernels = True
        return self

    def compile(self, **kwargs):
        return self.superoptimize(**kwargs)

    def valid_kernels(self):
        assert self._is_compiled, "Should check kernel validness after compilation"
        return self._valid_cuda_kernels

    def __call__(self, **kwargs):
        if self._executor is None:
            self.superoptimize()
        inputs = kwargs.get("inputs", [])
        return self._executor.run(inputs, stream=kwargs.get("stream", None))

    cuda_call = __call__
