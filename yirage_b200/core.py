"""Graph IR objects behind the Python surface: dtype, DTensor, the kernel graph and the
thread-block graph.  Plain Python stand-ins for the reference's Cython layer
(python/yirage/_cython/core.pyx: dtype :60-103, DTensor :420-470, CyKNGraph :880-1000,
CyTBGraph :560-700); only what the persistent-kernel path and the rms_norm/matmul
micro-graphs use is kept.
"""
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch


class dtype:
    """Element type handle (`yirage.bfloat16`, `yirage.int64`, ...)."""

    _SIZES = {"int8": 1, "int16": 2, "int32": 4, "int64": 8, "uint8": 1, "uint16": 2,
              "uint32": 4, "uint64": 8, "fp16": 2, "bf16": 2, "fp32": 4, "fp64": 8}
    # numeric codes used by the reference's task-graph JSON (include/yirage/type.h:84-119)
    _CODES = {"fp16": 940, "bf16": 941, "fp32": 942, "int32": 955, "int64": 965}

    def __init__(self, name: str):
        if name not in self._SIZES:
            raise ValueError(f"unknown dtype {name}")
        self.name = name

    @staticmethod
    def is_dtype(type_str):
        return type_str in dtype._SIZES

    @property
    def itemsize(self):
        return self._SIZES[self.name]

    @property
    def code(self):
        return self._CODES.get(self.name, 999)

    def __eq__(self, other):
        return isinstance(other, dtype) and other.name == self.name

    def __hash__(self):
        return hash(self.name)

    def __repr__(self):
        return f"yirage.{self.name}"


int8 = dtype("int8")
int16 = dtype("int16")
int32 = dtype("int32")
int64 = dtype("int64")
uint8 = dtype("uint8")
uint16 = dtype("uint16")
uint32 = dtype("uint32")
uint64 = dtype("uint64")
float16 = dtype("fp16")
bfloat16 = dtype("bf16")
float32 = dtype("fp32")
float64 = dtype("fp64")

_TORCH2DT = {
    torch.int8: int8, torch.int16: int16, torch.int32: int32, torch.int64: int64,
    torch.uint8: uint8, torch.float16: float16, torch.bfloat16: bfloat16,
    torch.float32: float32, torch.float64: float64,
}
_DT2TORCH = {v.name: k for k, v in _TORCH2DT.items()}


def convert_torch_type_to_dtype(t):
    if t not in _TORCH2DT:
        raise RuntimeError(f"Unsupported torch dtype: {t}")
    return _TORCH2DT[t]


def convert_dtype_to_torch_type(dt):
    return _DT2TORCH[dt.name]


@dataclass(eq=False)
class DTensor:
    """A device tensor of a kernel graph: shape, strides, type, and where its storage
    comes from (`kind`):
      input    - graph input supplied at call time (micro-graph surface)
      torch    - attached caller-owned torch tensor      (IODesc::TorchTensor)
      cuda     - allocated by the runtime                (IODesc::CUDAMallocTensor)
      nvshmem  - allocated by the runtime, peer-visible  (IODesc::NVSHMEMMallocTensor)
      shuffled - row interleave of attached tensors      (IODesc::ShuffledTorchTensor)
      op       - produced by a graph operator
    """
    dims: Tuple[int, ...]
    strides: Tuple[int, ...]
    dtype: dtype
    guid: int
    kind: str = "input"
    name: Optional[str] = None
    torch_tensor: Optional[torch.Tensor] = None
    sources: List["DTensor"] = field(default_factory=list)
    num_groups: int = 0
    producer: Optional[object] = None

    @property
    def num_dims(self):
        return len(self.dims)

    def dim(self, i):
        return self.dims[i]

    def stride(self, i):
        return self.strides[i]

    @property
    def nbytes(self):
        n = 1
        for d in self.dims:
            n *= d
        return n * self.dtype.itemsize

    def __repr__(self):
        return f"DTensor({self.name or self.guid}, {tuple(self.dims)}, {self.dtype.name}, {self.kind})"


def _row_major_strides(dims):
    strides, total = [], 1
    for d in reversed(dims):
        strides.append(total)
        total *= d
    return tuple(reversed(strides))


@dataclass
class KNOp:
    """One operator of the kernel graph."""
    kind: str                      # matmul | rms_norm | silu | mul | add | customized
    inputs: List[DTensor]
    outputs: List[DTensor]
    attrs: dict = field(default_factory=dict)


@dataclass
class TBInput:
    dtensor: Optional[DTensor]
    input_map: Tuple[int, int, int]
    forloop_dim: int
    store_in_dmem: bool


class CyTBGraph:
    """Thread-block graph of a customized operator.  On the persistent-kernel path it only
    carries the operands with their grid partition maps (python/yirage/persistent_kernel.py
    builds nothing else), plus the launch hints."""

    def __init__(self, grid_dim, block_dim, forloop_range, reduction_dimx):
        self.grid_dim = tuple(grid_dim)
        self.block_dim = tuple(block_dim)
        self.forloop_range = forloop_range
        self.reduction_dimx = reduction_dimx
        self.inputs: List[TBInput] = []

    def new_input(self, dtensor, input_map, forloop_dim, store_in_dmem=False):
        inp = TBInput(dtensor, tuple(input_map), forloop_dim, store_in_dmem)
        self.inputs.append(inp)
        return inp

    def tile_dims(self, inp: TBInput):
        """Per-task tile of an operand: dimension input_map[a] is divided by grid_dim[a]
        (src/threadblock/input_loader.cc:84-110)."""
        if inp.dtensor is None:
            return None
        dims = list(inp.dtensor.dims)
        for axis, d in enumerate(inp.input_map):
            if d >= 0:
                if dims[d] == 1:
                    continue        # a dimension of one entry is not cut (the reference's own
                                    # speculative-decoding demo maps its [tokens, 1] output so)
                if dims[d] % self.grid_dim[axis]:
                    raise ValueError(
                        f"dimension {d} ({dims[d]}) is not divisible by grid {self.grid_dim[axis]}")
                dims[d] //= self.grid_dim[axis]
        return tuple(dims)


class CyKNGraph:
    def __init__(self, disable_fingerprint=False):
        self.disable_fingerprint = disable_fingerprint
        self.tensors: List[DTensor] = []
        self.ops: List[KNOp] = []
        self.outputs: List[DTensor] = []
        self.tasks = []          # (tb_graph, task_name, params, operands)

    def _new(self, dims, strides, dt, kind, **kw):
        t = DTensor(tuple(int(d) for d in dims), tuple(int(s) for s in strides), dt,
                    guid=len(self.tensors), kind=kind, **kw)
        self.tensors.append(t)
        return t

    def new_input(self, dims, strides, dt):
        if strides is None:
            strides = _row_major_strides(dims)
        return self._new(dims, strides, dt, "input")

    def mark_output(self, t, strides=None):
        self.outputs.append(t)
        return t

    def _binary_shape(self, a, b):
        if a.dims != b.dims:
            raise ValueError(f"shape mismatch {a.dims} vs {b.dims}")
        return a.dims

    def matmul(self, a, b):
        if a.dims[-1] != b.dims[-2]:
            raise ValueError(f"matmul shape mismatch {a.dims} x {b.dims}")
        dims = tuple(a.dims[:-1]) + (b.dims[-1],)
        out = self._new(dims, _row_major_strides(dims), a.dtype, "op")
        op = KNOp("matmul", [a, b], [out])
        out.producer = op
        self.ops.append(op)
        return out

    def rms_norm(self, a, normalized_shape):
        if tuple(normalized_shape) != tuple(a.dims[-len(normalized_shape):]):
            raise ValueError("normalized_shape must match the trailing dimensions")
        out = self._new(a.dims, _row_major_strides(a.dims), a.dtype, "op")
        op = KNOp("rms_norm", [a], [out], {"normalized_shape": tuple(normalized_shape)})
        out.producer = op
        self.ops.append(op)
        return out

    def _unary(self, kind, a):
        out = self._new(a.dims, _row_major_strides(a.dims), a.dtype, "op")
        op = KNOp(kind, [a], [out])
        out.producer = op
        self.ops.append(op)
        return out

    def _binary(self, kind, a, b):
        dims = self._binary_shape(a, b)
        out = self._new(dims, _row_major_strides(dims), a.dtype, "op")
        op = KNOp(kind, [a, b], [out])
        out.producer = op
        self.ops.append(op)
        return out

    def silu(self, a):
        return self._unary("silu", a)

    def mul(self, a, b):
        return self._binary("mul", a, b)

    def add(self, a, b):
        return self._binary("add", a, b)

    def customized(self, inputs, tb_graph):
        op = KNOp("customized", [t for t in inputs if t is not None], [], {"tb_graph": tb_graph})
        self.ops.append(op)
        return []
