"""Execution of kernel graphs built with new_kernel_graph() (the micro-graphs of
benchmark/rmsnorm.py and benchmark/gated_mlp.py in the reference).

The reference turns such a graph into CUDA through its superoptimizer search and
transpiler (python/yirage/kernel.py:584-1247).  Here the graph is matched, operator by
operator, onto the task kernels of the persistent runtime and run as a one-pass task
graph:

    rms_norm -> matmul                       one LINEAR task set with the norm folded in
    matmul, matmul -> silu -> mul            one LINEAR task set with the SiLU*mul epilogue
    matmul                                   LINEAR
    rms_norm alone                           RMSNORM

The kernel-graph matmul takes its weight as [K, N] row-major (src/kernel/matmul.cc), the
streaming GEMV wants [N, K]; a weight is transposed once, the first time a tensor (same
storage, same version) is seen, and the transposed copy is reused on later calls.
Graphs that use operators without a task kernel (gelu, exp, div, reductions, ...) are
rejected: there is no generic fallback.
"""
from typing import Dict, List

import torch

from . import core
from .core import CyKNGraph, DTensor, KNOp
from .persistent_kernel import PersistentKernel


class MicroGraphExecutor:
    def __init__(self, graph: CyKNGraph):
        self.graph = graph
        if not graph.outputs:
            raise ValueError("the graph has no output (mark_output)")
        self.inputs = [t for t in graph.tensors if t.kind == "input" and t.producer is None]
        self.plan = self._match()
        self._built_for = None
        self._ypk = None
        self._outs: List[torch.Tensor] = []
        self._wt_cache: Dict[tuple, torch.Tensor] = {}

    # ------------------------------------------------------------------ matching
    def _match(self):
        ops = list(self.graph.ops)
        consumers: Dict[int, List[KNOp]] = {}
        for op in ops:
            for t in op.inputs:
                consumers.setdefault(t.guid, []).append(op)
        outputs = {t.guid for t in self.graph.outputs}

        def only_consumer(t, op):
            return consumers.get(t.guid, []) == [op] and t.guid not in outputs

        plan, done = [], set()
        for op in ops:
            if id(op) in done:
                continue
            if op.kind == "rms_norm":
                nxt = consumers.get(op.outputs[0].guid, [])
                if len(nxt) == 1 and nxt[0].kind == "matmul" and nxt[0].inputs[0] is op.outputs[0] \
                        and op.outputs[0].guid not in outputs:
                    continue  # folded into that matmul below
                plan.append(("rmsnorm", op.inputs[0], op.outputs[0]))
                done.add(id(op))
            elif op.kind == "matmul":
                a, w = op.inputs
                if a.num_dims != 2 or w.num_dims != 2:
                    raise NotImplementedError("only 2-D matmul is on the decode path")
                norm_src = None
                if a.producer is not None and a.producer.kind == "rms_norm" and only_consumer(a, op):
                    norm_src = a.producer.inputs[0]
                # gated pattern: this matmul -> silu -> mul <- another matmul of the same input
                y = op.outputs[0]
                cs = consumers.get(y.guid, [])
                fused = False
                if len(cs) == 1 and cs[0].kind == "silu" and only_consumer(y, cs[0]):
                    s_out = cs[0].outputs[0]
                    ms = consumers.get(s_out.guid, [])
                    if len(ms) == 1 and ms[0].kind == "mul" and only_consumer(s_out, ms[0]):
                        other = [t for t in ms[0].inputs if t is not s_out]
                        if other and other[0].producer is not None and other[0].producer.kind == "matmul" \
                                and other[0].producer.inputs[0] is a and only_consumer(other[0], ms[0]) \
                                and other[0].producer.inputs[1].dims == w.dims:
                            up = other[0].producer
                            plan.append(("gated", norm_src or a, norm_src is not None, w,
                                         up.inputs[1], ms[0].outputs[0]))
                            done.update(id(o) for o in (op, cs[0], ms[0], up))
                            fused = True
                if not fused:
                    plan.append(("linear", norm_src or a, norm_src is not None, w, y))
                    done.add(id(op))
            elif op.kind in ("silu", "mul"):
                raise NotImplementedError(
                    f"'{op.kind}' outside the matmul->silu->mul<-matmul pattern has no task kernel")
            else:
                raise NotImplementedError(f"kernel-graph operator '{op.kind}' has no task kernel")
        return plan

    # ------------------------------------------------------------------ building
    def _transposed(self, w: torch.Tensor) -> torch.Tensor:
        key = (w.data_ptr(), w._version, tuple(w.shape), w.dtype)
        if key not in self._wt_cache:
            self._wt_cache = {k: v for k, v in self._wt_cache.items() if k[0] != key[0]}
            # turned by the library's own kernel (torch only provides the memory)
            from . import _native as N
            import ctypes as C
            K, Nc = w.shape
            if not w.is_contiguous() or w.element_size() != 2:
                raise NotImplementedError("matmul weights must be contiguous 16-bit tensors")
            wt = torch.empty((Nc, K), dtype=w.dtype, device=w.device)
            N.check(None, N.load().ypk_transpose_16bit(
                C.c_void_p(w.data_ptr()), C.c_void_p(wt.data_ptr()), K, Nc,
                C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            self._wt_cache[key] = wt
        return self._wt_cache[key]

    def _build(self, feed: Dict[int, torch.Tensor]):
        batch = self.inputs[0].dims[0]
        ypk = PersistentKernel(
            mode="onepass", world_size=1, mpi_rank=0, num_workers=128, num_local_schedulers=0,
            num_remote_schedulers=0, max_seq_length=64, max_num_batched_requests=1,
            max_num_batched_tokens=batch, max_num_pages=1, page_size=64, eos_token_id=-1,
            meta_tensors={})
        ypk.rms_norm_eps = 0.0   # the kernel-graph rms_norm has no epsilon and no weight
        handle: Dict[int, DTensor] = {}

        def act(t: DTensor) -> DTensor:
            if t.guid not in handle:
                if t.guid in feed:
                    handle[t.guid] = ypk.attach_input(feed[t.guid], name=f"in{t.guid}")
                else:
                    handle[t.guid] = ypk.new_tensor(dims=t.dims, dtype=t.dtype, name=f"t{t.guid}")
            return handle[t.guid]

        def weight(t: DTensor) -> DTensor:
            if t.guid not in feed:
                raise NotImplementedError("matmul weights must be graph inputs")
            return ypk.attach_input(self._transposed(feed[t.guid]), name=f"w{t.guid}T")

        outs = {}
        for out_t in self.graph.outputs:
            outs[out_t.guid] = torch.empty(out_t.dims, dtype=core.convert_dtype_to_torch_type(out_t.dtype),
                                           device="cuda")
            handle[out_t.guid] = ypk.attach_input(outs[out_t.guid], name=f"out{out_t.guid}")
        g1 = (1, 1, 1)
        for step in self.plan:
            if step[0] == "rmsnorm":
                _, x, y = step
                ypk.rmsnorm_layer(act(x), None, act(y), (batch, 1, 1), (128, 1, 1), eps=0.0)
            elif step[0] == "linear":
                _, x, normed, w, y = step
                src = act(x)
                if normed:
                    tmp = ypk.new_tensor(dims=x.dims, dtype=x.dtype, name=f"normed{x.guid}_{y.guid}")
                    ypk.rmsnorm_layer(src, None, tmp, (batch, 1, 1), (128, 1, 1), eps=0.0)
                    src = tmp
                ypk.linear_layer(src, weight(w), act(y), g1, (128, 1, 1))
            else:
                _, x, normed, wg, wu, y = step
                src = act(x)
                if normed:
                    tmp = ypk.new_tensor(dims=x.dims, dtype=x.dtype, name=f"normed{x.guid}_{y.guid}")
                    ypk.rmsnorm_layer(src, None, tmp, (batch, 1, 1), (128, 1, 1), eps=0.0)
                    src = tmp
                gu = ypk.shuffle_tensors([weight(wg), weight(wu)], 0, 1, f"gu{y.guid}")
                mid = ypk.new_tensor(dims=(batch, 2 * wg.dims[1]), dtype=x.dtype, name=f"mid{y.guid}")
                ypk.linear_layer(src, gu, mid, g1, (128, 1, 1))
                ypk.silu_mul_layer(mid, act(y), g1, (128, 1, 1))
        ypk.compile()
        self._ypk, self._batch = ypk, batch
        self._outs = [outs[t.guid] for t in self.graph.outputs]

    # ------------------------------------------------------------------ running
    def run(self, inputs: List[torch.Tensor], stream=None):
        if len(inputs) != len(self.inputs):
            raise ValueError(f"the graph has {len(self.inputs)} inputs, got {len(inputs)}")
        if not torch.cuda.is_available():
            raise RuntimeError("kernel graphs run on a CUDA device only (sm_100a); "
                               "there is no CPU execution path")
        for t, x in zip(self.inputs, inputs):
            if tuple(x.shape) != tuple(t.dims) or core.convert_torch_type_to_dtype(x.dtype) != t.dtype:
                raise ValueError(f"input {t.guid}: expected {t.dims} {t.dtype}, got {tuple(x.shape)} {x.dtype}")
            if not x.is_cuda or not x.is_contiguous():
                raise ValueError("inputs must be contiguous CUDA tensors")
        key = tuple((x.data_ptr(), x._version) for x in inputs)
        if key != self._built_for:
            if self._ypk is not None:
                self._ypk.finalize()
            self._build({t.guid: x for t, x in zip(self.inputs, inputs)})
            self._built_for = key
        self._ypk(batch=self._batch, stream=stream)
        return self._outs
