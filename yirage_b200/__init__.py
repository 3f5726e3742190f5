"""yirage_b200: a B200-native (sm_100a) implementation of the persistent-kernel LLM decode
path behind YiRage's Python surface.

Exports the names the reference package exports for this path
(python/yirage/__init__.py:35-38,76-85): dtypes, DTensor, new_kernel_graph,
new_threadblock_graph, KNGraph, TBGraph, PersistentKernel, get_configurations_from_gpu,
speculative.  The search (`superoptimize` proper), the backend registry and the transpilers
of the reference are not part of this package.
"""
from . import core, global_config as _gc, kernel, lowering, persistent_kernel, speculative, threadblock, utils
from .core import (CyKNGraph, CyTBGraph, DTensor, bfloat16, convert_torch_type_to_dtype, dtype,
                   float16, float32, float64, int8, int16, int32, int64, uint8, uint16, uint32,
                   uint64)
from .global_config import global_config
from .kernel import KNGraph
from .persistent_kernel import PersistentKernel
from .threadblock import TBGraph
from .utils import get_configurations_from_gpu, get_shared_memory_capacity
from .version import __version__


class InputNotFoundError(Exception):
    """Raised when cannot find input tensors"""


def set_gpu_device_id(device_id: int):
    global_config.gpu_device_id = device_id


def bypass_compile_errors(value: bool = True):
    global_config.bypass_compile_errors = value


def new_kernel_graph():
    return KNGraph(CyKNGraph())


def new_threadblock_graph(grid_dim: tuple, block_dim: tuple, forloop_range: int,
                          reduction_dimx: int):
    return TBGraph(CyTBGraph(grid_dim, block_dim, forloop_range, reduction_dimx))


def get_available_backends():
    return ["cuda"]


def is_backend_available(name):
    return name == "cuda"


def get_default_backend():
    return "cuda"
