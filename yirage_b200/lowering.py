"""Host-side task-graph generation for the persistent megakernel.

Takes the operators registered through the PersistentKernel layer builders and produces
what the C ABI's ypk_load_graph wants: a task table in dependency order, one event per
operator, and a per-worker queue.  This is the counterpart of the reference's
Graph::generate_task_graph (src/kernel/runtime.cc:53-600,1416-1449) and of the shape
derivation in src/kernel/task_register.cc, with three differences that come from the
B200 design:

  * operators are fused before tasks are cut: rmsnorm -> linear becomes one LINEAR task
    with the norm folded in, linear(gate|up) -> silu_mul becomes a LINEAR task with the
    SiLU*mul epilogue (so mlp_mid and rmsnorm_out are never written);
  * the reference cuts an operator into grid_dim tasks and lets scheduler warps deal them
    round-robin at run time; here grid_dim is a hint: every linear operator is cut into
    one contiguous row slab per worker CTA, sized so that the *cumulative* weight bytes
    per worker stay level across operators, and the queues are fixed ahead of time;
  * dependencies are whole-operator events (every task of operator i waits for all tasks
    of operator i-1), which is what the reference's chain of consecutive operators
    degenerates to for these graphs (runtime.cc:446-503);
  * with at most 8 tokens in flight, a tensor that a linear operator produces and only
    linear operators read (the residual stream, the MLP activation) is not handed over
    through an event at all: it travels as flagged 8-byte words {two values, tag} that the
    readers poll (`plan_handoff`).  Under tensor parallelism the row-split projections push
    their partial sums straight into every rank's exchange buffer in that form and the
    ALLREDUCE tasks only poll, add and pass the sum on.

Nothing here touches the GPU; it is plain Python and is unit-tested on CPU.
"""
import json
import os
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from . import _native as N
from .core import DTensor, bfloat16, float16, float32, int32, int64

MAX_TASK_ROWS = 256          # kMaxAccRows in device_common.cuh
KV_TILE = 64
HEAD_DIM = 128
MAX_NEW_TOKENS = 8           # kMaxNewTokens: new tokens one ATTENTION task takes
MAX_NEW_KEYS = 64            # kMaxNewKeys: new tokens of a request per iteration over query tiles
MAX_ATTN_ROWS = 32           # kMaxAttnRows
ATTN_ROW_FLOATS = HEAD_DIM + 4   # kAttnRowFloats in task_attention.cuh
MAX_SPLITS = 16
# A worker that ran an attention task of a graph of at most 8 tokens reaches the next LINEAR
# operator late (the task takes 6-8 us from the moment q/k/v are there, the other workers spend
# that time polling with their activations half staged): it is given this many weight bytes
# less of that operator, ~3.4 us of streaming (measured on Llama-3-8B decode: 2.99 -> 2.96 ms
# per token between 100 and 220 KB).
ATTN_LOAD_BYTES = 160 * 1024
ATTN_TILES_PER_SPLIT = 4     # kAttnTilesPerSplit in device_common.cuh
ALLREDUCE_TILE = 256          # columns per ALLREDUCE task
SILU_GRAN = 2                # kSiluGran: fused gate/up rows come as 2 gate + 2 up
# Widest tensor handed over as flagged words.  A reader polls 2x the bytes with four 16-byte
# loads in flight per thread and round, so a very wide tensor takes several trips to L2
# against the one of a plain copy: measured on Llama-3-8B, the 14336-wide MLP activation is
# still 0.7 % faster per token as flagged words than behind an event.
MAX_FLAGGED_COLS = int(os.environ.get("YPK_MAX_FLAGGED_COLS", "16384"))
# Above this width a tensor is taken as flagged words only by iterations of one or two tokens:
# with more tokens the reader has to poll tokens x width words chunk by chunk (measured on the
# 14336-wide MLP activation of Llama-3-8B at 8 tokens: the down projection takes 1.3x as long
# as behind an event), so the producer also publishes its event and the reader decides per
# iteration (YPK_F_LL_OPT).
WIDE_FLAGGED_COLS = 8192
ARGMAX_TAG_ID = 255           # tag id of the cross-rank arg-max exchange (operators use 0..253)


@dataclass
class RegisteredTask:
    """What a layer builder recorded: reference task name, operands in TB-graph order,
    launch hints and integer parameters."""
    name: str
    operands: List[Optional[DTensor]]
    grid_dim: Tuple[int, int, int]
    block_dim: Tuple[int, int, int]
    params: List[int] = field(default_factory=list)
    attrs: dict = field(default_factory=dict)


@dataclass
class FusedOp:
    kind: str                       # embed | linear | attention | argmax_partial | ...
    src: List[RegisteredTask]
    t: Dict[str, Optional[DTensor]]  # named operands
    flags: int = 0
    attrs: dict = field(default_factory=dict)


@dataclass
class TaskSpec:
    type: int
    flags: int = 0
    op_id: int = 0
    ptr: List[Optional[Tuple[DTensor, int]]] = field(default_factory=lambda: [None] * N.NPTR)
    ptr_aux: Optional[Tuple[DTensor, int]] = None           # ninth operand (F_NORM_OUT)
    iarg: List[int] = field(default_factory=lambda: [0] * N.NINT)
    farg: List[float] = field(default_factory=lambda: [0.0] * N.NFLT)
    dep_event: int = -1
    dep_count: int = 0
    trig_event: int = -1
    worker: int = 0
    weight_bytes: int = 0
    flagged_deps: List[int] = field(default_factory=list)   # tag ids this task polls for
    flagged_out: int = -1                                   # tag id it writes
    # tensors of the graph that the task reads / writes only in flagged-word form (their plain
    # copies are not touched); listed in the JSON so that the data flow stays readable
    logical_in: List[Tuple[DTensor, int]] = field(default_factory=list)
    logical_out: List[Tuple[DTensor, int]] = field(default_factory=list)


@dataclass
class LoweredGraph:
    ops: List[FusedOp]
    tasks: List[TaskSpec]
    num_events: int
    queue: List[int]
    queue_off: List[int]
    shuffles: List[dict]            # {dst, sources, rows, gran, row_bytes}
    internal: List[DTensor]         # scratch tensors the runtime has to allocate
    worker_bytes: List[int]         # weight bytes streamed per worker per iteration

    @property
    def num_tasks(self):
        return len(self.tasks)


_SUFFIXES = ("_sm100", "_sm90", "_hopper", "_swapAB", "_cutlass")


def canonical_name(name: str) -> str:
    """Strip the architecture suffixes the reference appends per compute capability
    (persistent_kernel.py:372,604-609,822-833,981-1011)."""
    changed = True
    while changed:
        changed = False
        for s in _SUFFIXES:
            if name.endswith(s):
                name = name[: -len(s)]
                changed = True
    return name


# ---------------------------------------------------------------------------- fusion
def _reads(rt: RegisteredTask) -> List[DTensor]:
    name = canonical_name(rt.name)
    ops = rt.operands
    n_out = {"argmax_partial": 2, "moe_topk_softmax": 3}.get(name, 1)
    return [t for t in ops[: len(ops) - n_out] if t is not None]


def _writes(rt: RegisteredTask) -> List[DTensor]:
    name = canonical_name(rt.name)
    ops = rt.operands
    n_out = {"argmax_partial": 2, "moe_topk_softmax": 3}.get(name, 1)
    return [t for t in ops[len(ops) - n_out:] if t is not None]


def _dead_after(regs: List[RegisteredTask], start: int, t: DTensor) -> bool:
    """True if nothing from regs[start:] reads `t` before it is written again."""
    for rt in regs[start:]:
        if any(x is t for x in _reads(rt)):
            return False
        if any(x is t for x in _writes(rt)):
            return True
    return True


def fuse(regs: List[RegisteredTask], default_eps: float, fuse_norm: bool = True) -> List[FusedOp]:
    """`fuse_norm` False keeps every RMSNorm an operator of its own (graphs of more than 8
    tokens: the tensor-core LINEAR path takes its tokens by TMA and cannot scale them on the
    way in; a norm over 16..128 rows as a separate operator costs a few microseconds)."""
    out: List[FusedOp] = []
    i = 0
    n = len(regs)
    while i < n:
        rt = regs[i]
        name = canonical_name(rt.name)
        if name == "embedding":
            ids, table, o = rt.operands
            out.append(FusedOp("embed", [rt], {"ids": ids, "table": table, "out": o}))
            i += 1
        elif name in ("rmsnorm", "linear", "linear_with_residual"):
            norm_rt = None
            j = i
            if name == "rmsnorm":
                x, nw, y = rt.operands
                nxt = regs[i + 1] if i + 1 < n else None
                if (fuse_norm and nxt is not None
                        and canonical_name(nxt.name) in ("linear", "linear_with_residual")
                        and nxt.operands[0] is y and _dead_after(regs, i + 2, y)):
                    norm_rt = rt
                    j = i + 1
                else:
                    out.append(FusedOp("rmsnorm", [rt], {"x": x, "w": nw, "out": y},
                                       attrs={"eps": rt.attrs.get("eps", default_eps)}))
                    i += 1
                    continue
            lin = regs[j]
            lname = canonical_name(lin.name)
            if lname == "linear":
                xin, w, y = lin.operands
                res = None
            else:
                xin, w, res, y = lin.operands
            flags = 0
            t = {"x": xin, "w": w, "out": y, "norm_w": None, "res": res}
            attrs = {"eps": default_eps}
            srcs = [lin]
            if norm_rt is not None:
                t["x"] = norm_rt.operands[0]
                t["norm_w"] = norm_rt.operands[1]
                flags |= N.F_NORM if norm_rt.operands[1] is not None else N.F_NORM_NOWEIGHT
                attrs["eps"] = norm_rt.attrs.get("eps", default_eps)
                srcs = [norm_rt, lin]
            if res is not None:
                flags |= N.F_RESIDUAL
            k = j + 1
            nxt = regs[k] if k < n else None
            if (res is None and nxt is not None and canonical_name(nxt.name) == "silu_mul"
                    and nxt.operands[0] is y and w.kind == "shuffled" and len(w.sources) == 2
                    and w.sources[0].dims == w.sources[1].dims
                    and w.sources[0].dims[0] % SILU_GRAN == 0 and _dead_after(regs, k + 1, y)):
                flags |= N.F_SILU_MUL
                t["out"] = nxt.operands[1]
                srcs.append(nxt)
                k += 1
            out.append(FusedOp("linear", srcs, t, flags, attrs))
            i = k
        elif name == "paged_attention":
            qkv, kc, vc, qn, kn, cos, sin, o = rt.operands
            flags = N.F_ROPE if (cos is not None and sin is not None) else 0
            attrs = {"num_q_heads": rt.params[0], "num_kv_heads": rt.params[1]}
            if qn is not None or kn is not None:
                # q/k RMSNorm of Qwen3 (demo/qwen3/demo.py:444-476): the two weight vectors are
                # packed into one [2, 128] tensor when the graph is compiled
                if qn is None or kn is None or rt.attrs.get("qk_norm_packed") is None:
                    raise ValueError("paged attention needs both q_norm and k_norm, or neither")
                flags |= N.F_QK_NORM
                attrs.update(q_norm=qn, k_norm=kn, qk_norm_packed=rt.attrs["qk_norm_packed"],
                             eps=rt.attrs.get("eps", default_eps))
            out.append(FusedOp("attention", [rt], {"qkv": qkv, "k_cache": kc, "v_cache": vc,
                                                    "cos": cos, "sin": sin, "out": o}, flags, attrs))
            i += 1
        elif name == "silu_mul":
            x, o = rt.operands
            out.append(FusedOp("silu_mul", [rt], {"in": x, "out": o},
                               attrs={"groups": rt.grid_dim[0]}))
            i += 1
        elif name == "argmax_partial":
            x, pv, pi = rt.operands
            out.append(FusedOp("argmax_partial", [rt], {"in": x, "val": pv, "idx": pi},
                               attrs={"nparts": rt.grid_dim[0],
                                      "valid_cols": rt.attrs.get("valid_cols")}))
            i += 1
        elif name == "argmax_reduce":
            pv, pi, o = rt.operands
            out.append(FusedOp("argmax_reduce", [rt], {"val": pv, "idx": pi, "out": o},
                               attrs={"vocab_offset": rt.attrs.get("vocab_offset", 0),
                                      "exchange": rt.attrs.get("exchange", False)}))
            i += 1
        elif name == "moe_topk_softmax":
            x, wts, routing, mask = rt.operands
            out.append(FusedOp("moe_topk", [rt], {"in": x, "weights": wts, "routing": routing, "mask": mask}))
            i += 1
        elif name in ("moe_w13_linear", "moe_w2_linear"):
            x, w, routing, mask, o = rt.operands
            out.append(FusedOp("moe_linear", [rt], {"x": x, "w": w, "routing": routing, "mask": mask, "out": o},
                               attrs={"which": "w13" if name == "moe_w13_linear" else "w2"}))
            i += 1
        elif name == "moe_silu_mul":
            x, o = rt.operands
            out.append(FusedOp("moe_silu_mul", [rt], {"in": x, "out": o}))
            i += 1
        elif name == "moe_mul_sum_add":
            x, wts, res, o = rt.operands
            out.append(FusedOp("moe_combine", [rt], {"in": x, "weights": wts, "res": res, "out": o}))
            i += 1
        elif name == "find_ngram_partial":
            toks, o = rt.operands
            out.append(FusedOp("ngram_partial", [rt], {"tokens": toks, "out": o},
                               attrs={"ngram_size": rt.params[0]}))
            i += 1
        elif name == "find_ngram_global":
            part, toks, o = rt.operands
            out.append(FusedOp("ngram_global", [rt], {"partial": part, "tokens": toks, "out": o},
                               attrs={"ngram_size": rt.params[0], "spec_length": rt.params[1]}))
            i += 1
        elif name == "target_verify_greedy":
            spec, target, o = rt.operands
            out.append(FusedOp("verify", [rt], {"spec": spec, "target": target, "out": o},
                               attrs={"spec_length": rt.attrs.get("spec_length")}))
            i += 1
        elif name == "allreduce":
            x, buf, o = rt.operands
            out.append(FusedOp("allreduce", [rt], {"in": x, "buf": buf, "out": o},
                               attrs={"world": rt.params[0], "rank": rt.params[1]}))
            i += 1
        else:
            raise NotImplementedError(f"task '{rt.name}' is outside the decode hot path")
    return out


# --------------------------------------------------------------------- flagged hand-off
_OUTPUT_KEYS = {"embed": ("out",), "linear": ("out", "norm_out", "ss_out"), "attention": ("out",), "rmsnorm": ("out",),
                "silu_mul": ("out",), "argmax_partial": ("val", "idx"), "argmax_reduce": ("out",),
                "allreduce": ("out",), "ngram_partial": ("out",), "ngram_global": ("out",),
                "verify": ("out",), "moe_topk": ("weights", "routing", "mask"), "moe_linear": ("out",),
                "moe_silu_mul": ("out",), "moe_combine": ("out",)}
# operands that are not activations produced inside the iteration
_STATIC_KEYS = {"w", "norm_w", "norm_out_w", "table", "k_cache", "v_cache", "cos", "sin", "buf", "tokens"}


def _op_outputs(op):
    return [op.t[k] for k in _OUTPUT_KEYS[op.kind] if op.t.get(k) is not None]


def _op_inputs(op):
    """(role, tensor) of the activations an operator reads."""
    outs = _OUTPUT_KEYS[op.kind]
    return [(k, t) for k, t in op.t.items()
            if t is not None and k not in outs and k not in _STATIC_KEYS]


def _readers(ops, i, T):
    """Operators that read what operator i wrote into T, as (index, role), and whether the
    value is also read across the iteration boundary (by an operator at or before i)."""
    found, wraps = [], False
    n = len(ops)
    for step in range(1, n + 1):
        j = (i + step) % n
        if j == i:
            break
        for role, t in _op_inputs(ops[j]):
            if t is T:
                found.append((j, role))
                wraps = wraps or j < i
        if any(t is T for t in _op_outputs(ops[j])):
            break
    return found, wraps


def plan_handoff(ops, world_size: int):
    """Which tensors leave their producer as flagged words.  Returns per operator index a
    dict with optional entries
        "out":  (key, tag id, push)   producer side (linear, or allreduce passing its sum on)
        "x" / "res" / "in": (key, tag id)   consumer side
    where `key` names the flagged-word buffer (one per tensor, shared by all layers).

    Tag ids in the plan are unique per producer; the device sees them modulo 254
    (`device_tag`).  Two producers whose ids agree modulo 254 must not write the same buffer
    in one iteration (a reader could take one for the other): checked here.

    The exchange buffers of pushed partial sums are single-buffered, which is safe only if
    consecutive all-reduces (cyclically, across the iteration boundary) use different
    buffers: a rank can then overwrite a peer's slot only after that peer has pushed the
    next all-reduce, i.e. has finished reading this one.  A graph where that does not hold
    (one all-reduce per iteration, or an odd number alternating between two tensors) keeps
    its all-reduces on the event path, whose buffer halves alternate on the device."""
    plan = {i: {} for i in range(len(ops))}
    next_id = 0
    if world_size > 1:
        ar_inputs = [id(op.t["in"]) for op in ops if op.kind == "allreduce"]
        push_safe = len(ar_inputs) >= 2 and all(
            ar_inputs[k] != ar_inputs[(k + 1) % len(ar_inputs)] for k in range(len(ar_inputs)))
    else:
        push_safe = False
    def reader_ok(j, role):
        return (ops[j].kind == "linear" and role in ("x", "res")) or \
               (ops[j].kind == "attention" and role == "qkv")

    for i, op in enumerate(ops):
        if op.kind not in ("linear", "attention"):
            continue
        T = op.t["out"]
        if T.dims[1] > MAX_FLAGGED_COLS:
            continue
        readers, wraps = _readers(ops, i, T)
        if not readers or wraps:
            continue
        ar = None
        if (op.kind == "linear" and len(readers) == 1 and ops[readers[0][0]].kind == "allreduce"
                and world_size > 1 and readers[0][0] == i + 1):
            if not push_safe:
                continue
            ar = readers[0][0]
            T2 = ops[ar].t["out"]
            readers2, wraps2 = _readers(ops, ar, T2)
            if not readers2 or wraps2 or T.dims[1] % ALLREDUCE_TILE:
                continue
            final = readers2
        else:
            final = readers
        if not all(reader_ok(j, role) for j, role in final):
            continue
        if any(role == "res" and (ops[j].flags & N.F_SILU_MUL) for j, role in final):
            continue
        wide = T.dims[1] > WIDE_FLAGGED_COLS
        if wide and not (ar is None and len(final) == 1 and final[0] == (i + 1, "x")
                         and ops[i + 1].kind == "linear"):
            continue        # the per-iteration choice is built for "next operator reads it as x"
        if ar is None:
            pid = next_id
            next_id += 1
            plan[i]["out"] = (("ll", id(T)), pid, False, T)
            for j, role in final:
                plan[j][role] = (("ll", id(T)), pid)
                if wide:
                    plan[j]["x_opt"] = True
        else:
            pid, aid = next_id, next_id + 1
            next_id += 2
            plan[i]["out"] = (("push", id(T)), pid, True, T)
            plan[ar]["in"] = (("push", id(T)), pid)
            plan[ar]["out"] = (("ll", id(T2)), aid, False, T2)
            for j, role in final:
                plan[j][role] = (("ll", id(T2)), aid)
    seen = set()
    for i in plan:
        if "out" in plan[i]:
            key, pid = plan[i]["out"][0], plan[i]["out"][1]
            if (key, device_tag(pid)) in seen:
                raise NotImplementedError(
                    "more than 254 flagged-word producers alias on one buffer; use handoff='event'")
            seen.add((key, device_tag(pid)))
    return plan


def query_tile_slots(max_requests: int, max_tokens: int, chunk: int) -> int:
    """Most query tiles one iteration can hold: every request contributes one tile per
    `chunk` new tokens, the last one possibly short.  With n requests sharing max_tokens
    tokens that is n + (max_tokens - n) // chunk, largest for the most requests."""
    n = min(max_requests, max_tokens)
    return n + (max_tokens - n) // chunk


def device_tag(pid: int) -> int:
    """Tag id as the device sees it (8 bits; 254 and 255 are reserved)."""
    return pid % 254


# ------------------------------------------------------------------------- balancing
def level_partition(n_units: int, unit_bytes: int, loads: List[float]) -> List[int]:
    """Split n_units equal units over the workers so that load[i] + count[i]*unit_bytes is
    as level as possible (water-filling).  Returns the count per worker."""
    W = len(loads)
    if n_units <= 0:
        return [0] * W
    lo, hi = min(loads), max(loads) + float(n_units) * unit_bytes
    for _ in range(60):
        mid = 0.5 * (lo + hi)
        got = sum(max(0.0, (mid - l) / unit_bytes) for l in loads)
        if got < n_units:
            lo = mid
        else:
            hi = mid
    ideal = [max(0.0, (hi - l) / unit_bytes) for l in loads]
    counts = [int(math.floor(x)) for x in ideal]
    rem = n_units - sum(counts)
    order = sorted(range(W), key=lambda i: (ideal[i] - counts[i]), reverse=True)
    k = 0
    while rem > 0:
        counts[order[k % W]] += 1
        rem -= 1
        k += 1
    while rem < 0:  # floor can only undershoot, but keep the invariant explicit
        idx = max(range(W), key=lambda i: counts[i])
        counts[idx] -= 1
        rem += 1
    assert sum(counts) == n_units and min(counts) >= 0
    return counts


def splitk_plan(nrows: int, K: int, gran: int, W: int):
    """Row blocks x K ranges for a linear operator of a graph with more than 8 tokens, or None
    to keep plain row slabs.  The tensor-core LINEAR path wants 100+ weight rows per task (an
    instruction then covers enough weight bytes to follow HBM); an operator with fewer rows
    per worker than that (o_proj, down_proj, qkv) is cut along K as well, so that it still
    makes about one task per worker.  Returns (rows per block, number of splits)."""
    if nrows >= 96 * W or K % 64:
        return None
    nkb = K // 64
    for S in range(2, 17):
        if nkb < 4 * S:
            break
        nb = max(1, W // S)
        unit = 8 if gran in (1, 2, 4, 8) else gran
        rows = -(-nrows // nb)
        rows = -(-rows // unit) * unit
        if rows > MAX_TASK_ROWS:
            continue
        if rows >= 100 or S == 16 or nkb < 4 * (S + 1):
            return rows, S
    return None


def carry_norms(ops: List[FusedOp]) -> List[FusedOp]:
    """Graphs of more than 8 tokens keep every RMSNorm an operator of its own (`fuse`), which
    costs two operators per layer.  Where the norm sits between two LINEAR operators,
    linear(+residual) -> rmsnorm -> linear, it is carried across them instead: the first
    writes, besides its rows, the rows times the norm weight and the sums of their squares
    per row block (F_NORM_OUT), the second reads that copy as its input and applies the RMS
    factor to its dot products (F_NORM_PRE), the order of operations of the fused norm of
    narrow graphs.  The RMSNORM operator disappears.  Tensor-core path only: set
    YPK_TENSOR_CORE=never to keep the operators apart."""
    import os
    if os.environ.get("YPK_TENSOR_CORE", "") == "never":
        return ops
    out: List[FusedOp] = []
    i, n = 0, len(ops)
    while i < n:
        a = ops[i]
        nm = ops[i + 1] if i + 1 < n else None
        b = ops[i + 2] if i + 2 < n else None
        ok = (a.kind == "linear" and nm is not None and b is not None and nm.kind == "rmsnorm"
              and b.kind == "linear" and not (a.flags & (N.F_SILU_MUL | N.F_NORM | N.F_NORM_NOWEIGHT | N.F_NORM_PRE))
              and not (b.flags & (N.F_NORM | N.F_NORM_NOWEIGHT)) and nm.t["w"] is not None
              and nm.t["x"] is a.t["out"] and b.t["x"] is nm.t["out"]
              and a.t["w"].dims[0] % 8 == 0 and a.t["w"].dims[1] % 64 == 0
              and a.t["out"].dims == nm.t["out"].dims and nm.t["w"].dims == (a.t["out"].dims[1],))
        if ok:
            # nobody else may read the normalised rows
            readers, _ = _readers(ops, i + 1, nm.t["out"])
            ok = readers == [(i + 2, "x")]
        if not ok:
            out.append(a)
            i += 1
            continue
        a.flags |= N.F_NORM_OUT
        a.t["norm_out"], a.t["norm_out_w"] = nm.t["out"], nm.t["w"]
        a.src = list(a.src) + list(nm.src)
        b.flags |= N.F_NORM_PRE
        b.attrs["eps"] = nm.attrs["eps"]
        b.attrs["norm_from"] = a
        out.append(a)
        i += 2          # the rmsnorm operator is dropped; b is looked at next (it may carry on)
    return out


def _carry_operands(op, op_tasks, splitk, flags, max_tokens, scratch, norm_bufs):
    """Operands of a carried norm (see carry_norms) on the tasks of a LINEAR operator.  The
    producer's row blocks are its tasks, or with a split along K the blocks its splits share;
    every block owns a row [max_tokens] of the sums-of-squares buffer."""
    if flags & N.F_NORM_OUT:
        for k, ts in enumerate(op_tasks):
            ts.iarg[12] = (ts.iarg[10] if splitk else k) | (max_tokens << 16)
        nblk = max(ts.iarg[12] & 0xffff for ts in op_tasks) + 1
        if nblk > 0xffff:
            raise NotImplementedError("a carried norm over more than 65535 row blocks")
        key = (op.t["out"].dims[1], nblk)
        if key not in norm_bufs:
            norm_bufs[key] = scratch((nblk * max_tokens,), float32, f"norm_ss_{key[0]}x{nblk}")
        op.t["ss_out"] = norm_bufs[key]
        op.attrs["ss_nblk"] = nblk
        for ts in op_tasks:
            ts.ptr[3] = (op.t["norm_out_w"], 0)
            ts.ptr[6] = (op.t["ss_out"], 0)
            ts.ptr_aux = (op.t["norm_out"], 0)
    if flags & N.F_NORM_PRE:
        prod = op.attrs["norm_from"]
        op.t["ss_in"] = prod.t["ss_out"]
        for ts in op_tasks:
            ts.ptr[3] = (op.t["ss_in"], 0)
            ts.iarg[12] = prod.attrs["ss_nblk"] | (max_tokens << 16)


# --------------------------------------------------------------------------- lowering
def _all_flagged(plan, ops, oi):
    """True if every activation operator `oi` reads arrives as flagged words."""
    ins = _op_inputs(ops[oi])
    return bool(ins) and all(role in plan[oi] for role, _ in ins)   # ("x_opt" is not a role)


def _link(tasks, first, ev, plan, ops, oi, prev_event, prev_count):
    """Events of the tasks of operator `oi` (tasks[first:]).  An operator waits for its
    predecessor's event unless all its activations come as flagged words, and triggers its
    own unless the next operator does not wait for it."""
    # an operator whose flagged input is optional (x_opt) also waits for the event of the
    # operator before it, which therefore publishes it; the device skips that wait in
    # iterations of one or two tokens
    waits = not _all_flagged(plan, ops, oi) or bool(plan[oi].get("x_opt"))
    last = oi == len(ops) - 1
    next_opt = not last and bool(plan[oi + 1].get("x_opt"))
    triggers = last or not _all_flagged(plan, ops, oi + 1) or next_opt
    # published for the sake of an optional reader only: not in iterations of one or two tokens
    wide_only = next_opt and not last and _all_flagged(plan, ops, oi + 1)
    for ts in tasks[first:]:
        if wide_only:
            ts.flags |= N.F_TRIG_WIDE
        ts.trig_event = ev if triggers else -1
        ts.dep_event = prev_event if waits else -1
        ts.dep_count = prev_count if waits else 0
        ts.flagged_deps = [plan[oi][r][1] for r in ("x", "res", "in", "qkv") if r in plan[oi]]
        ts.flagged_out = plan[oi]["out"][1] if "out" in plan[oi] else -1


def tensor_dependencies(ops, serving: bool):
    """Which operator each operator has to wait for, derived from the tensors they read and
    write (the reference derives its events the same way, src/kernel/runtime.cc:446-503),
    instead of chaining every operator to its predecessor.  Operator j must run after the
    last writer of everything it reads (read after write), after the readers of what it
    overwrites and after its previous writer.  A task carries one dependency event, so j
    waits for the latest of those operators, m, provided m's completion implies the others'
    (they are among the operators m itself, transitively, waited for).  Returns the list of
    operator indices (-1: none), or None when one event per task cannot express the graph,
    or when, in serving mode, completion of the last operator would not imply completion of
    all (the iteration boundary waits for the last operator only); the caller then keeps the
    chain."""
    n = len(ops)
    last_writer, readers_since = {}, {}
    dep, anc = [-1] * n, [None] * n
    for j, op in enumerate(ops):
        reads = [id(t) for _, t in _op_inputs(op)]
        writes = [id(t) for t in _op_outputs(op)]
        if op.kind == "attention":
            # appends to the caches it reads; all attention operators share the split scratch
            reads += [id(op.t["k_cache"]), id(op.t["v_cache"]), "attn_split_scratch"]
            writes += [id(op.t["k_cache"]), id(op.t["v_cache"]), "attn_split_scratch"]
        if op.kind == "allreduce":
            reads.append("allreduce_exchange")
            writes.append("allreduce_exchange")
        if op.attrs.get("splitk_key") is not None:
            # operators of one shape share the workspace of their split along K
            reads.append(("splitk", op.attrs["splitk_key"]))
            writes.append(("splitk", op.attrs["splitk_key"]))
        need = set()
        for t in reads:
            if t in last_writer:
                need.add(last_writer[t])
        for t in writes:
            if t in last_writer:
                need.add(last_writer[t])
            need |= readers_since.get(t, set())
        need.discard(j)
        if need:
            m = max(need)
            if need <= anc[m]:
                dep[j] = m
            elif need <= anc[j - 1]:
                dep[j] = j - 1
            else:
                return None
            anc[j] = {j} | anc[dep[j]]
        else:
            anc[j] = {j}
        for t in reads:
            readers_since.setdefault(t, set()).add(j)
        for t in writes:
            last_writer[t] = j
            readers_since[t] = set()
    if serving and anc[n - 1] != set(range(n)):
        return None
    return dep


def _is16(t: DTensor):
    return t.dtype in (bfloat16, float16)


def lower(regs: List[RegisteredTask], *, num_workers: int, max_tokens: int, max_requests: int,
          max_seq_length: int, page_size: int, world_size: int = 1, rank: int = 0,
          default_eps: float = 1e-6, new_tensor=None, handoff: str = "auto",
          serving: bool = True) -> LoweredGraph:
    """Fuse, cut into tasks, assign to workers.  `new_tensor(dims, dtype, name)` creates
    runtime-owned scratch tensors (attention split partials, flagged-word buffers).
    `handoff`: "event" = operators wait for events; "ll" = flagged words where possible (at
    most 8 tokens); "auto" = "ll" when max_tokens <= 8.  `serving`: the graph runs iteration
    after iteration with the batcher in between (offline mode) rather than once per launch.
    Where no tensor travels as flagged words the events follow the tensors
    (`tensor_dependencies`): independent operators do not wait for each other."""
    ops = fuse(regs, default_eps, fuse_norm=max_tokens <= 8)
    if max_tokens > 8 and world_size == 1:
        ops = carry_norms(ops)
    if handoff == "auto":
        handoff = "ll" if max_tokens <= 8 else "event"
    if handoff == "ll" and max_tokens > 8:
        raise ValueError("the flagged-word hand-off is built for at most 8 tokens in flight")
    plan = plan_handoff(ops, world_size) if handoff == "ll" else {i: {} for i in range(len(ops))}
    ll_bufs: Dict[tuple, DTensor] = {}

    def ll_buffer(key, T, push):
        if key not in ll_bufs:
            base = (T.name or f"tensor_{T.guid}")
            if push:
                ll_bufs[key] = scratch((world_size, max_tokens, T.dims[1]), int32,
                                       f"flagged_push_{base}", symmetric=True)
            else:
                ll_bufs[key] = scratch((max_tokens, T.dims[1]), int32, f"flagged_{base}")
        return ll_bufs[key]

    W = num_workers
    loads = [0.0] * W      # weight bytes per worker so far
    late = [0.0] * W       # allowance of the next LINEAR operator (graphs of at most 8 tokens)
    tasks: List[TaskSpec] = []
    shuffles: List[dict] = []
    internal: List[DTensor] = []
    shuffled_done: Dict[int, dict] = {}
    rr = 0  # rotating start for round-robin placed tasks

    def scratch(dims, dt, name, symmetric=False):
        if new_tensor is None:
            raise RuntimeError("lowering needs a tensor factory for scratch buffers")
        t = new_tensor(dims, dt, name, symmetric) if symmetric else new_tensor(dims, dt, name)
        internal.append(t)
        return t

    comm_buf = None
    num_signals = 0
    num_allreduce = 0
    allreduce_tasks: List[TaskSpec] = []

    attn_scratch = None
    attn_tag_ids = set()
    splitk_bufs: Dict[tuple, tuple] = {}
    norm_bufs: Dict[tuple, DTensor] = {}  # sums of squares of carried norms, by (width, blocks)
    moe_bufs: Dict[tuple, object] = {}    # scratch of the mixture-of-experts operators, by shape
    moe_state: Dict[str, object] = {}     # the routing the expert operators of a layer work under
    prev_event, prev_count = -1, 0

    for oi, op in enumerate(ops):
        first = len(tasks)
        ev = oi
        if op.kind == "embed":
            ids, table, o = op.t["ids"], op.t["table"], op.t["out"]
            hidden = table.dims[1]
            if hidden % 8:
                raise ValueError("embedding width must be a multiple of 8")
            # a few tasks at decode sizes; many tokens per iteration spread the copy wider
            ntask = max(1, min(8, hidden // 1024)) if max_tokens <= 8 else max(1, min(32, W, hidden // 128))
            cols = hidden // ntask // 8 * 8
            c = 0
            for k in range(ntask):
                nc = cols if k < ntask - 1 else hidden - c
                ts = TaskSpec(N.TASK_EMBED, op_id=oi)
                ts.ptr[0], ts.ptr[1], ts.ptr[2] = (ids, 0), (table, 0), (o, 0)
                ts.iarg[:6] = [hidden, c, nc, table.dims[1], o.dims[1], table.dims[0]]
                ts.worker = (rr + k) % W
                tasks.append(ts)
                c += nc
            rr += ntask
        elif op.kind == "linear":
            x, w, o = op.t["x"], op.t["w"], op.t["out"]
            nw, res = op.t["norm_w"], op.t["res"]
            if not (_is16(x) and x.dtype == w.dtype == o.dtype):
                raise ValueError("linear operands must share a 16-bit float type")
            K = w.dims[1]
            if x.dims[1] != K:
                raise ValueError(f"linear: input width {x.dims[1]} != weight K {K}")
            if K % 64:
                raise NotImplementedError(f"linear needs K % 64 == 0 (got {K})")
            Nrows = w.dims[0]
            silu = bool(op.flags & N.F_SILU_MUL)
            flags = op.flags | (N.F_F16 if x.dtype == float16 else 0)
            if (flags & N.F_RESIDUAL) and world_size > 1 and rank != 0:
                # partial sums are added across ranks afterwards: the residual goes in once
                flags &= ~N.F_RESIDUAL
            ll = plan[oi]
            if "x" in ll:
                flags |= N.F_LL_IN | (N.F_LL_OPT if ll.get("x_opt") else 0)
            if "res" in ll and (flags & N.F_RESIDUAL):
                flags |= N.F_LL_RES
            if "out" in ll:
                flags |= N.F_LL_OUT | (N.F_LL_PUSH if ll["out"][2] else 0)
            gran = 2 * SILU_GRAN if silu else (2 if (flags & (N.F_LL_OUT | N.F_LL_RES)) else 1)
            if flags & N.F_NORM_OUT:
                gran = 4          # the carried norm is written four rows at a time
            if w.kind == "shuffled" and id(w) not in shuffled_done:
                srcs = w.sources
                if silu:
                    g = [SILU_GRAN, SILU_GRAN]
                else:
                    if any(s.dims[0] % w.num_groups for s in srcs):
                        raise ValueError("shuffle_tensors: rows not divisible by num_groups")
                    g = [s.dims[0] // w.num_groups for s in srcs]
                sh = {"dst": w, "sources": list(srcs), "rows": [s.dims[0] for s in srcs],
                      "gran": g, "row_bytes": K * w.dtype.itemsize}
                shuffles.append(sh)
                shuffled_done[id(w)] = sh
            elif w.kind == "shuffled" and silu and shuffled_done[id(w)]["gran"] != [SILU_GRAN, SILU_GRAN]:
                raise ValueError("a shuffled weight is used both fused and unfused")
            expect_out = Nrows // 2 if silu else Nrows
            if o.dims[1] < expect_out:
                raise ValueError(f"linear: output width {o.dims[1]} < {expect_out}")
            units = Nrows // gran
            if Nrows % gran:
                raise ValueError(f"fused gate/up weight rows must be a multiple of {gran}")
            unit_bytes = gran * K * 2
            sk = splitk_plan(Nrows, K, gran, W) if max_tokens > 8 else None
            if sk is not None:
                # row blocks x K ranges: every task leaves fp32 partial sums in a workspace,
                # the last split of a block to arrive adds them and writes the rows
                rows_blk, S = sk
                key = (Nrows, S)
                if key not in splitk_bufs:
                    nb_max = -(-Nrows // rows_blk)
                    splitk_bufs[key] = (
                        scratch((S * max_tokens * Nrows,), float32, f"splitk_ws_{Nrows}x{S}"),
                        scratch((nb_max * S * max_tokens,), float32, f"splitk_ss_{Nrows}x{S}"),
                        scratch((nb_max * ((max_tokens + 15) // 16),), int32, f"splitk_cnt_{Nrows}x{S}"))
                ws, ws_ss, ws_cnt = splitk_bufs[key]
                op.attrs["splitk_key"] = key
                nkb = K // 64
                kb_edges = [nkb * s // S for s in range(S + 1)]
                order = sorted(range(W), key=lambda w_: loads[w_])
                ti_local = 0
                for blk, r in enumerate(range(0, Nrows, rows_blk)):
                    take = min(rows_blk, Nrows - r)
                    for s_ in range(S):
                        k0, k1 = kb_edges[s_] * 64, kb_edges[s_ + 1] * 64
                        ts = TaskSpec(N.TASK_LINEAR, flags=flags, op_id=oi)
                        ts.ptr[0], ts.ptr[1], ts.ptr[2] = (x, 0), (w, 0), (o, 0)
                        if nw is not None:
                            ts.ptr[3] = (nw, 0)
                        if flags & N.F_RESIDUAL:
                            ts.ptr[4] = (res, 0)
                        ts.ptr[5], ts.ptr[6], ts.ptr[7] = (ws, 0), (ws_ss, 0), (ws_cnt, 0)
                        ts.iarg[:9] = [K, r, take, x.dims[1], w.dims[1], o.dims[1],
                                       res.dims[1] if res is not None else 0, 0, Nrows]
                        ts.iarg[10] = blk
                        ts.iarg[13], ts.iarg[14] = k0, k1 - k0
                        ts.iarg[15] = s_ | (S << 8) | (max_tokens << 16)
                        ts.farg[0] = float(op.attrs.get("eps", default_eps))
                        ts.worker = order[ti_local % W]
                        ts.weight_bytes = take * (k1 - k0) * 2
                        loads[ts.worker] += ts.weight_bytes
                        tasks.append(ts)
                        ti_local += 1
                _carry_operands(op, tasks[first:], True, flags, max_tokens, scratch, norm_bufs)
                count = len(tasks) - first
                _link(tasks, first, ev, plan, ops, oi, prev_event, prev_count)
                prev_event, prev_count = ev, count
                continue
            if max_tokens <= 8:
                # Every operator of such a graph waits for all of its predecessor: what counts
                # is the largest slab of THIS operator, so the rows are levelled per operator
                # (against the allowance of workers that come late from an attention task);
                # the bytes a worker has streamed so far only decide who gets the larger of
                # two otherwise equal slabs.
                counts = level_partition(units, unit_bytes, late)
                groups: Dict[float, List[int]] = {}
                for wk in range(W):
                    groups.setdefault(late[wk], []).append(wk)
                for members in groups.values():
                    sizes = sorted((counts[wk] for wk in members), reverse=True)
                    for wk, c in zip(sorted(members, key=lambda w_: loads[w_]), sizes):
                        counts[wk] = c
                late = [0.0] * W
            else:
                counts = level_partition(units, unit_bytes, loads)
            r = 0
            for wk in range(W):
                nrows = counts[wk] * gran
                loads[wk] += counts[wk] * unit_bytes
                while nrows > 0:
                    take = min(nrows, MAX_TASK_ROWS)
                    ts = TaskSpec(N.TASK_LINEAR, flags=flags, op_id=oi)
                    ts.ptr[0], ts.ptr[1], ts.ptr[2] = (x, 0), (w, 0), (o, 0)
                    if nw is not None:
                        ts.ptr[3] = (nw, 0)
                    if flags & N.F_RESIDUAL:
                        ts.ptr[4] = (res, 0)
                    ts.iarg[:8] = [K, r, take, x.dims[1], w.dims[1], o.dims[1],
                                   res.dims[1] if res is not None else 0, 0]
                    if flags & N.F_LL_IN:
                        ts.ptr[5] = (ll_bufs[ll["x"][0]], 0)
                        ts.iarg[10] = device_tag(ll["x"][1])
                    if flags & N.F_LL_RES:
                        ts.ptr[6] = (ll_bufs[ll["res"][0]], 0)
                        ts.iarg[11] = device_tag(ll["res"][1])
                    if flags & N.F_LL_OUT:
                        key, pid, push, T = ll["out"]
                        ts.ptr[7] = (ll_buffer(key, T, push), 0)
                        ts.iarg[12] = device_tag(pid)
                    ts.farg[0] = float(op.attrs.get("eps", default_eps))
                    ts.worker = wk
                    ts.weight_bytes = take * K * 2
                    tasks.append(ts)
                    r += take
                    nrows -= take
            assert r == Nrows
            _carry_operands(op, tasks[first:], False, flags, max_tokens, scratch, norm_bufs)
        elif op.kind == "attention":
            qkv, kc, vc, o = op.t["qkv"], op.t["k_cache"], op.t["v_cache"], op.t["out"]
            hq, hkv = op.attrs["num_q_heads"], op.attrs["num_kv_heads"]
            if kc.dims[3] != HEAD_DIM:
                raise NotImplementedError("attention is built for head_dim 128")
            if hq % hkv or hq // hkv > 8:
                raise NotImplementedError("attention needs 1..8 q heads per kv head")
            if page_size % KV_TILE:
                raise NotImplementedError(f"attention needs page_size % {KV_TILE} == 0")
            G = hq // hkv
            if qkv.dims[1] != hkv * (G + 2) * HEAD_DIM:
                raise ValueError("packed qkv width does not match the head counts")
            max_tiles = (max_seq_length + KV_TILE - 1) // KV_TILE
            # Graphs of more than 8 tokens let a request bring more new tokens than one task
            # takes: the tasks are made per entry of the iteration's query-tile list (one
            # entry per `chunk` new tokens of a request) instead of per request slot.
            qtiles = max_tokens > MAX_NEW_TOKENS
            chunk = min(MAX_NEW_TOKENS, MAX_ATTN_ROWS // G)
            nslots = query_tile_slots(max_requests, max_tokens, chunk) if qtiles else max_requests
            # the device never activates more than ceil(tiles / ATTN_TILES_PER_SPLIT) splits
            nsplit = max(1, min(W // max(1, nslots * hkv), -(-max_tiles // ATTN_TILES_PER_SPLIT),
                                MAX_SPLITS))
            max_rows = min(G * MAX_NEW_TOKENS, MAX_ATTN_ROWS)
            if nsplit > 1:
                # partial rows travel as 8-byte flagged words {fp32 bits, tag}: two floats each
                need = 2 * nslots * hkv * nsplit * max_rows * ATTN_ROW_FLOATS
                if attn_scratch is None or attn_scratch.dims[0] < need:
                    attn_scratch = scratch((need,), float32, "attn_split_scratch")
                # all layers share the scratch: the tags of two attention operators must differ
                if oi % 254 in attn_tag_ids:
                    raise NotImplementedError("two attention operators 254 operators apart share "
                                              "a split-KV tag; reduce the graph or the splits")
                attn_tag_ids.add(oi % 254)
            qk_packed = None
            if op.flags & N.F_QK_NORM:
                qk_packed = op.attrs["qk_norm_packed"]
                if id(qk_packed) not in shuffled_done:
                    qn_t, kn_t = op.attrs["q_norm"], op.attrs["k_norm"]
                    if not (qn_t.dims == kn_t.dims == (HEAD_DIM,) and _is16(qn_t) and qn_t.dtype == kn_t.dtype
                            and qn_t.dtype == qkv.dtype):
                        raise ValueError("q_norm / k_norm must be 16-bit vectors of head_dim entries")
                    sh = {"dst": qk_packed, "sources": [qn_t, kn_t], "rows": [1, 1], "gran": [1, 1],
                          "row_bytes": HEAD_DIM * 2}
                    shuffles.append(sh)
                    shuffled_done[id(qk_packed)] = sh
            k = 0
            for r in range(nslots):
                for h in range(hkv):
                    for s in range(nsplit):
                        ts = TaskSpec(N.TASK_ATTENTION, flags=op.flags | (N.F_QTILES if qtiles else 0),
                                      op_id=oi)
                        ts.ptr[0], ts.ptr[1], ts.ptr[2], ts.ptr[3] = (qkv, 0), (kc, 0), (vc, 0), (o, 0)
                        if op.flags & N.F_ROPE:
                            ts.ptr[4], ts.ptr[5] = (op.t["cos"], 0), (op.t["sin"], 0)
                        if nsplit > 1:
                            ts.ptr[6] = (attn_scratch, 0)
                        if qk_packed is not None:
                            ts.ptr[7] = (qk_packed, 0)
                            ts.farg[0] = float(op.attrs["eps"])
                        ts.iarg[:9] = [r, h, s, nsplit, G, hkv, qkv.dims[1], o.dims[1], max_rows]
                        ts.iarg[13] = oi % 254     # tag id of the split-KV partials
                        if qtiles:
                            ts.iarg[14] = nslots
                        if "qkv" in plan[oi]:    # packed q/k/v arrive as flagged words
                            ts.flags |= N.F_LL_IN
                            ts.logical_in.append((qkv, 0))
                            ts.ptr[0] = (ll_bufs[plan[oi]["qkv"][0]], 0)
                            ts.iarg[11] = device_tag(plan[oi]["qkv"][1])
                        if "out" in plan[oi]:    # and the result leaves the same way
                            key, pid, _, Tout = plan[oi]["out"]
                            ts.flags |= N.F_LL_OUT
                            ts.logical_out.append((o, 0))
                            ts.ptr[3] = (ll_buffer(key, Tout, False), 0)
                            ts.iarg[12] = device_tag(pid)
                        # splits of one (request, head) go to different workers
                        ts.worker = (rr + k) % W
                        if max_tokens <= 8:
                            late[ts.worker] += ATTN_LOAD_BYTES
                        tasks.append(ts)
                        k += 1
            rr += k
        elif op.kind == "argmax_partial":
            x, pv, pi = op.t["in"], op.t["val"], op.t["idx"]
            nparts = op.attrs["nparts"]
            V = x.dims[1]
            if V % nparts:
                raise ValueError("argmax_partial: vocabulary not divisible by the task count")
            if pv.dims[1] < nparts or pi.dims[1] < nparts:
                raise ValueError("argmax_partial: partial buffers narrower than the task count")
            per = V // nparts
            for p in range(nparts):
                ts = TaskSpec(N.TASK_ARGMAX_PARTIAL, op_id=oi)
                ts.ptr[0], ts.ptr[1], ts.ptr[2] = (x, 0), (pv, 0), (pi, 0)
                ts.iarg[:6] = [p * per, per, x.dims[1], p, pv.dims[1],
                               int(op.attrs.get("valid_cols") or 0)]
                ts.worker = (rr + p) % W
                tasks.append(ts)
            rr += nparts
            op.attrs["ld_parts"] = pv.dims[1]
        elif op.kind == "argmax_reduce":
            pv, pi, o = op.t["val"], op.t["idx"], op.t["out"]
            # only the first `nparts` columns of the partial buffers were written
            nparts = None
            for prev in reversed(ops[:oi]):
                if prev.kind == "argmax_partial" and prev.t["val"] is pv:
                    nparts = prev.attrs["nparts"]
                    break
            if nparts is None:
                nparts = pv.dims[1]
            ts = TaskSpec(N.TASK_ARGMAX_REDUCE, op_id=oi)
            ts.ptr[0], ts.ptr[1], ts.ptr[2] = (pv, 0), (pi, 0), (o, 0)
            ts.iarg[0] = nparts
            ts.iarg[4] = pv.dims[1]      # row pitch: only the first nparts columns were written
            if op.attrs.get("exchange") and world_size > 1:
                xbuf = scratch((world_size, max_tokens, 2), int64, "argmax_exchange", symmetric=True)
                ts.flags |= N.F_LL_PUSH
                ts.ptr[3] = (xbuf, 0)
                ts.iarg[1:4] = [op.attrs["vocab_offset"], world_size, rank]
                ts.iarg[12] = ARGMAX_TAG_ID
            ts.worker = 0
            tasks.append(ts)
        elif op.kind == "moe_topk":
            x, wts, routing, mask = op.t["in"], op.t["weights"], op.t["routing"], op.t["mask"]
            E, topk = x.dims[1], wts.dims[1]
            if not (_is16(x) and wts.dtype == float32 and routing.dtype == int32 and mask.dtype == int32):
                raise ValueError("moe_topk_softmax: 16-bit logits, fp32 weights, int32 routing and mask")
            if routing.dims != (E, max_tokens) or mask.dims[0] != E + 1 or wts.dims[0] != max_tokens:
                raise ValueError("moe_topk_softmax: routing is [experts, max_tokens], mask [experts + 1], "
                                 "weights [max_tokens, experts per token]")
            # Expert work is laid out by active slot (the a-th expert, ascending, that some token
            # of the iteration selected); the buffers are shared by all layers.
            key = ("moe", E, topk)
            if key not in moe_bufs:
                moe_bufs[key] = {"slot": scratch((max_tokens, topk), int32, "moe_token_slot"),
                                 "slots": min(E, max_tokens * topk), "E": E, "topk": topk}
            moe_state.update(moe_bufs[key], mask=mask, weights=wts)
            ts = TaskSpec(N.TASK_MOE_TOPK, op_id=oi)
            ts.ptr[0], ts.ptr[1], ts.ptr[2], ts.ptr[3] = (x, 0), (wts, 0), (routing, 0), (mask, 0)
            ts.ptr[4] = (moe_state["slot"], 0)
            ts.iarg[:3] = [E, topk, x.dims[1]]
            ts.worker = rr % W
            tasks.append(ts)
            rr += 1
        elif op.kind == "moe_linear":
            x, w, o = op.t["x"], op.t["w"], op.t["out"]
            if not moe_state or op.t["mask"] is not moe_state["mask"]:
                raise ValueError("an expert projection needs the routing of the moe_topk_softmax before it")
            if len(w.dims) != 3 or not _is16(w) or w.dims[0] != moe_state["E"]:
                raise ValueError("expert weights are [experts, rows, K], 16-bit")
            E, Nrows, K = w.dims
            S, MT = moe_state["slots"], max_tokens
            if K % 64:
                raise NotImplementedError(f"linear needs K % 64 == 0 (got {K})")
            which = op.attrs["which"]
            # per slot an [max_tokens, width] block in and out, whatever the caller's tensors
            # look like (the reference's are [tokens, experts per token, width])
            bkey = (which, S, MT, Nrows)
            if bkey not in moe_bufs:
                moe_bufs[bkey] = scratch((S * MT, Nrows), w.dtype, f"moe_{which}_out")
            out_buf = moe_bufs[bkey]
            moe_state[which + "_out"] = out_buf
            if which == "w13":
                if x.dims[1] != K:
                    raise ValueError("moe_w13: input width != K")
                xin = lambda a: (x, 0)
                ldx = x.dims[1]
            else:
                act = moe_state.get("act")
                if act is None or act.dims[1] != K:
                    raise ValueError("moe_w2 needs the moe_silu_mul before it")
                xin = lambda a: (act, a * MT * K * 2)
                ldx = K
            # Enough slabs per slot that one token's experts fill the machine; the slots only
            # a second and later token can reach get fewer, larger slabs (a task whose slot is
            # unused still costs its fetch).
            topk = moe_state["topk"]
            nslab = max(1, min(W // topk, (Nrows + 15) // 16))     # one token's pairs: at most one per worker
            nslab_far = max((Nrows + MAX_TASK_ROWS - 1) // MAX_TASK_ROWS, nslab // 4, 1)
            k = 0
            for a in range(S):
                ns = nslab if a < topk else nslab_far
                per = ((Nrows + ns - 1) // ns + 15) // 16 * 16
                for r0 in range(0, Nrows, per):
                    ts = TaskSpec(N.TASK_LINEAR, flags=N.F_MOE, op_id=oi)
                    ts.ptr[0], ts.ptr[1], ts.ptr[2] = xin(a), (w, 0), (out_buf, a * MT * Nrows * 2)
                    ts.ptr[5] = (moe_state["mask"], 0)
                    ts.iarg[:8] = [K, r0, min(per, Nrows - r0), ldx, K, Nrows, 0, 0]
                    ts.iarg[8] = 1 if which == "w2" else 0    # (only tells the two apart in the JSON)
                    ts.iarg[9] = -1
                    ts.iarg[10], ts.iarg[11], ts.iarg[12] = a, E, Nrows
                    ts.worker = (rr + k) % W
                    ts.weight_bytes = 0      # data dependent: not part of the static balance
                    tasks.append(ts)
                    k += 1
            rr += k
        elif op.kind == "moe_silu_mul":
            src = moe_state.get("w13_out")
            if src is None:
                raise ValueError("moe_silu_mul needs the moe_w13_linear before it")
            S, MT, I = moe_state["slots"], max_tokens, src.dims[1] // 2
            bkey = ("act", S, MT, I)
            if bkey not in moe_bufs:
                moe_bufs[bkey] = scratch((S * MT, I), src.dtype, "moe_silu_mul_out")
            moe_state["act"] = moe_bufs[bkey]
            ntask = min(W, S)
            per = (S + ntask - 1) // ntask
            for k in range(ntask):
                ts = TaskSpec(N.TASK_MOE_SILU_MUL, op_id=oi)
                ts.ptr[0], ts.ptr[1], ts.ptr[2] = (src, 0), (moe_state["act"], 0), (moe_state["mask"], 0)
                ts.iarg[:4] = [I, moe_state["E"], k * per, min(per, S - k * per)]
                ts.worker = (rr + k) % W
                if ts.iarg[3] > 0:
                    tasks.append(ts)
            rr += ntask
        elif op.kind == "moe_combine":
            src = moe_state.get("w2_out")
            res, o = op.t["res"], op.t["out"]
            if src is None or op.t["weights"] is not moe_state["weights"]:
                raise ValueError("moe_mul_sum_add needs the moe_w2_linear and the routing weights before it")
            H = src.dims[1]
            if res.dims[1] != H or o.dims[1] != H:
                raise ValueError("moe_mul_sum_add: residual and output are [tokens, hidden]")
            ntask = max(1, min(W, H // 64))
            cols = (H // ntask + 7) // 8 * 8
            k = 0
            for c in range(0, H, cols):
                ts = TaskSpec(N.TASK_MOE_COMBINE, op_id=oi)
                ts.ptr[0], ts.ptr[1], ts.ptr[2] = (src, 0), (moe_state["weights"], 0), (moe_state["slot"], 0)
                ts.ptr[3], ts.ptr[4] = (res, 0), (o, 0)
                ts.iarg[:6] = [H, moe_state["topk"], c, min(cols, H - c), res.dims[1], o.dims[1]]
                ts.worker = (rr + k) % W
                tasks.append(ts)
                k += 1
            rr += k
        elif op.kind == "ngram_partial":
            part = op.t["out"]
            if part.dtype != int32 and part.dtype != int64:
                raise ValueError("find_ngram_partial: the partial results are integers")
            # the reference sizes this buffer [requests, 96] int64; here it is read as int32
            # [max_requests][nparts] with as many parts as fit, one task each
            words = part.nbytes // 4
            nparts = max(1, min(W, words // max(1, max_requests)))
            op.attrs["nparts"] = nparts
            for p in range(nparts):
                ts = TaskSpec(N.TASK_NGRAM_PARTIAL, op_id=oi)
                ts.ptr[0] = (part, 0)
                ts.iarg[:3] = [p, nparts, int(op.attrs["ngram_size"])]
                ts.worker = (rr + p) % W
                tasks.append(ts)
            rr += nparts
        elif op.kind == "ngram_global":
            part, ids = op.t["partial"], op.t["out"]
            nparts = None
            for prev in reversed(ops[:oi]):
                if prev.kind == "ngram_partial" and prev.t["out"] is part:
                    nparts = prev.attrs["nparts"]
                    break
            if nparts is None:
                raise ValueError("find_ngram_global without the find_ngram_partial that feeds it")
            if ids.dtype != int64 or ids.nbytes < max_tokens * 8:
                raise ValueError("find_ngram_global: the draft ids are int64, one per token slot")
            ts = TaskSpec(N.TASK_NGRAM_GLOBAL, op_id=oi)
            ts.ptr[0], ts.ptr[1] = (part, 0), (ids, 0)
            ts.iarg[:2] = [nparts, int(op.attrs["ngram_size"])]
            ts.worker = rr % W
            tasks.append(ts)
            rr += 1
            op.attrs["ids"] = ids
        elif op.kind == "verify":
            spec_len = op.attrs.get("spec_length")
            if spec_len is None:
                for prev in reversed(ops[:oi]):
                    if prev.kind == "ngram_global" and prev.t["out"] is op.t["spec"]:
                        spec_len = prev.attrs["spec_length"]
                        break
            if not spec_len:
                raise ValueError("target_verify_greedy: the draft length is unknown")
            ts = TaskSpec(N.TASK_VERIFY, op_id=oi)
            ts.ptr[0], ts.ptr[1] = (op.t["spec"], 0), (op.t["target"], 0)
            ts.iarg[0] = int(spec_len)
            ts.worker = 0
            tasks.append(ts)
        elif op.kind == "rmsnorm":
            x, nw, o = op.t["x"], op.t["w"], op.t["out"]
            ntask = min(max_tokens, W)
            per = (max_tokens + ntask - 1) // ntask
            for k in range(ntask):
                ts = TaskSpec(N.TASK_RMSNORM, op_id=oi,
                              flags=N.F_F16 if x.dtype == float16 else 0)
                ts.ptr[0], ts.ptr[2] = (x, 0), (o, 0)
                if nw is not None:
                    ts.ptr[1] = (nw, 0)
                ts.iarg[:5] = [x.dims[1], k * per, per, x.dims[1], o.dims[1]]
                ts.farg[0] = float(op.attrs.get("eps", default_eps))
                ts.worker = (rr + k) % W
                tasks.append(ts)
            rr += ntask
        elif op.kind == "silu_mul":
            x, o = op.t["in"], op.t["out"]
            inter = o.dims[1]
            groups = max(1, op.attrs.get("groups", 1))
            if x.dims[1] != 2 * inter or inter % groups:
                raise ValueError("silu_mul: input must be twice as wide as the output")
            gs = inter // groups
            ntask = min(W, groups)
            per_groups = (groups + ntask - 1) // ntask
            k = 0
            g0 = 0
            while g0 < groups:
                ng = min(per_groups, groups - g0)
                ts = TaskSpec(N.TASK_SILU_MUL, op_id=oi)
                ts.ptr[0], ts.ptr[1] = (x, 0), (o, 0)
                ts.iarg[:5] = [g0 * gs, ng * gs, gs, x.dims[1], o.dims[1]]
                ts.worker = (rr + k) % W
                tasks.append(ts)
                g0 += ng
                k += 1
            rr += k
        elif op.kind == "allreduce":
            x, o = op.t["in"], op.t["out"]
            world_a, rank_a = op.attrs["world"], op.attrs["rank"]
            if world_a != world_size or rank_a != rank:
                raise ValueError("allreduce_layer was built for another rank / world size")
            if world_size < 2:
                raise ValueError("allreduce_layer needs world_size > 1")
            hidden = x.dims[1]
            if hidden % ALLREDUCE_TILE or o.dims[1] != hidden:
                raise NotImplementedError(f"all-reduce width must be a multiple of {ALLREDUCE_TILE}")
            ntile = hidden // ALLREDUCE_TILE
            if "in" in plan[oi]:
                # flagged-word form: the producing LINEAR tasks have pushed their partial sums
                # into every rank's exchange buffer; these tasks poll, add and pass the sum on
                key_o, aid, _, T2 = plan[oi]["out"]
                for k in range(ntile):
                    ts = TaskSpec(N.TASK_ALLREDUCE, op_id=oi, flags=N.F_LL_IN | N.F_LL_OUT)
                    ts.ptr[0], ts.ptr[1], ts.ptr[2] = (x, 0), (ll_bufs[plan[oi]["in"][0]], 0), (o, 0)
                    ts.ptr[7] = (ll_buffer(key_o, T2, False), 0)
                    ts.iarg[:10] = [k * ALLREDUCE_TILE, ALLREDUCE_TILE, x.dims[1], o.dims[1], hidden,
                                    max_tokens, 0, 0, world_size, rank]
                    ts.iarg[10], ts.iarg[12] = device_tag(plan[oi]["in"][1]), device_tag(aid)
                    ts.worker = (rr + k) % W
                    tasks.append(ts)
                rr += ntile
                count = len(tasks) - first
                _link(tasks, first, ev, plan, ops, oi, prev_event, prev_count)
                prev_event, prev_count = ev, count
                continue
            # The caller's buffer tensor ([world, tokens, hidden]) is not used: the runtime keeps
            # one double-buffered exchange area and one counter per all-reduce tile in the
            # symmetric arena (identical offsets on every rank).
            if comm_buf is None or comm_buf.dims[-1] != hidden:
                comm_buf = scratch((2, world_size, max_tokens, hidden), bfloat16, "allreduce_exchange",
                                   symmetric=True)
            sig0 = num_signals
            num_signals += ntile
            for k in range(ntile):
                ts = TaskSpec(N.TASK_ALLREDUCE, op_id=oi)
                ts.ptr[0], ts.ptr[1], ts.ptr[2] = (x, 0), (comm_buf, 0), (o, 0)
                # iarg[6] = index among the iteration's all-reduces, iarg[10] (filled in below)
                # their number: the device derives the buffer half from the running count
                ts.iarg[:10] = [k * ALLREDUCE_TILE, ALLREDUCE_TILE, x.dims[1], o.dims[1], hidden,
                                max_tokens, num_allreduce, sig0 + k, world_size, rank]
                ts.worker = (rr + k) % W
                tasks.append(ts)
                allreduce_tasks.append(ts)
            rr += ntile
            num_allreduce += 1
        else:
            raise NotImplementedError(op.kind)
        count = len(tasks) - first
        _link(tasks, first, ev, plan, ops, oi, prev_event, prev_count)
        prev_event, prev_count = ev, count

    if all(not p for p in plan.values()):
        dep = tensor_dependencies(ops, serving)
        if dep is not None:
            by_op: Dict[int, List[TaskSpec]] = {}
            for ts in tasks:
                by_op.setdefault(ts.op_id, []).append(ts)
            awaited = {d for d in dep if d >= 0}
            for j in range(len(ops)):
                for ts in by_op[j]:
                    ts.dep_event = dep[j]
                    ts.dep_count = len(by_op[dep[j]]) if dep[j] >= 0 else 0
                    ts.trig_event = j if (j in awaited or j == len(ops) - 1) else -1

    if allreduce_tasks:
        signals = scratch((num_signals,), int64, "allreduce_signals", symmetric=True)
        for ts in allreduce_tasks:
            ts.ptr[3] = (signals, 0)
            ts.iarg[10] = num_allreduce

    # queues: tasks of a worker in task (= operator) order
    per_worker: List[List[int]] = [[] for _ in range(W)]
    for ti, ts in enumerate(tasks):
        per_worker[ts.worker].append(ti)
    queue, queue_off = [], [0]
    for wk in range(W):
        queue.extend(per_worker[wk])
        queue_off.append(len(queue))
    worker_bytes = [0] * W
    for ts in tasks:
        worker_bytes[ts.worker] += ts.weight_bytes
    return LoweredGraph(ops, tasks, len(ops), queue, queue_off, shuffles, internal, worker_bytes)


# ------------------------------------------------------------------------- simulation
def simulate(g: LoweredGraph, iterations: int = 2):
    """Host model of the device protocol (the reference's sanity_check, runtime.cc:540-600):
    workers run their queues in order, a task may start once its dependency counter has
    reached dep_count * iteration.  Returns the number of executions per task; raises if
    the graph deadlocks."""
    ntask = len(g.tasks)
    counters = [0] * g.num_events
    executed = [0] * ntask
    # flagged words: a reader needs every task that writes the tag to have run this iteration
    writers: Dict[int, int] = {}
    for ts in g.tasks:
        if ts.flagged_out >= 0:
            writers[ts.flagged_out] = writers.get(ts.flagged_out, 0) + 1
    for it in range(1, iterations + 1):
        heads = [g.queue_off[w] for w in range(len(g.queue_off) - 1)]
        remaining = ntask
        written: Dict[int, int] = {}
        while remaining:
            progressed = False
            for w in range(len(heads)):
                while heads[w] < g.queue_off[w + 1]:
                    ts = g.tasks[g.queue[heads[w]]]
                    if ts.dep_event >= 0 and counters[ts.dep_event] < ts.dep_count * it:
                        break
                    if any(written.get(d, 0) < writers.get(d, 1) for d in ts.flagged_deps):
                        break
                    if ts.trig_event >= 0:
                        counters[ts.trig_event] += 1
                    if ts.flagged_out >= 0:
                        written[ts.flagged_out] = written.get(ts.flagged_out, 0) + 1
                    executed[g.queue[heads[w]]] += 1
                    heads[w] += 1
                    remaining -= 1
                    progressed = True
            if not progressed:
                raise RuntimeError(f"task graph deadlocks in iteration {it}")
    return executed


# ------------------------------------------------------------------------------- JSON
_REF_TASK_TYPE = {  # TaskType numbers of the reference (runtime_header.h:62-124)
    N.TASK_EMBED: 101, N.TASK_LINEAR: 253, N.TASK_ATTENTION: 257, N.TASK_ARGMAX_PARTIAL: 259,
    N.TASK_ARGMAX_REDUCE: 258, N.TASK_RMSNORM: 154, N.TASK_SILU_MUL: 118, N.TASK_ALLREDUCE: 107,
    N.TASK_NGRAM_PARTIAL: 112, N.TASK_NGRAM_GLOBAL: 113, N.TASK_VERIFY: 114,
    N.TASK_MOE_TOPK: 260, N.TASK_MOE_SILU_MUL: 118, N.TASK_MOE_COMBINE: 261,
}
REF_TASK_NAMES = {101: "TASK_EMBEDDING", 253: "TASK_LINEAR_SM100", 252: "TASK_LINEAR_WITH_RESIDUAL_SM100",
                  257: "TASK_ATTN_SM100", 259: "TASK_ARGMAX_PARTIAL_SM100",
                  258: "TASK_ARGMAX_REDUCE_SM100", 154: "TASK_RMS_NORM_HOPPER", 118: "TASK_SILU_MUL",
                  107: "TASK_REDUCE", 112: "TASK_FIND_NGRAM_PARTIAL", 113: "TASK_FIND_NGRAM_GLOBAL",
                  114: "TASK_TARGET_VERIFY_GREEDY", 254: "TASK_MOE_W13_LINEAR_SM100",
                  255: "TASK_MOE_W2_LINEAR_SM100", 260: "TASK_MOE_TOPK_SOFTMAX_SM100",
                  261: "TASK_MOE_MUL_SUM_ADD_SM100"}
EVENT_INVALID_ID = 0x7ffffffffffffffe     # runtime_header.h:55: "no event"
EVENT_LAUNCH_DEPENDENT_TASKS = 903        # runtime_header.h:126-134
EVENT_END_OF_TASK_GRAPH = 910
_JSON_DTYPES = (940, 941, 965)            # fp16, bf16, int64: what the reference's tools accept
# pointer slots of ypk_task that a task writes, by task type (the rest are inputs)
_OUTPUT_SLOTS = {N.TASK_EMBED: (2,), N.TASK_LINEAR: (2,), N.TASK_ATTENTION: (3,),
                 N.TASK_ARGMAX_PARTIAL: (1, 2), N.TASK_ARGMAX_REDUCE: (2,), N.TASK_RMSNORM: (2,),
                 N.TASK_SILU_MUL: (1,), N.TASK_ALLREDUCE: (2,), N.TASK_NGRAM_PARTIAL: (0,),
                 N.TASK_NGRAM_GLOBAL: (1,), N.TASK_VERIFY: (), N.TASK_MOE_TOPK: (1, 2, 3, 4),
                 N.TASK_MOE_SILU_MUL: (1,), N.TASK_MOE_COMBINE: (4,)}


# pointer slots that hold runtime-internal buffers (flagged-word copies, exchange areas, scratch)
_INTERNAL_SLOTS = {N.TASK_LINEAR: (5, 6, 7), N.TASK_ALLREDUCE: (1, 3, 7), N.TASK_ATTENTION: (6,),
                   N.TASK_ARGMAX_REDUCE: (3,)}


def ref_task_type(ts: TaskSpec) -> int:
    """TaskType number of the reference task this task stands for (runtime_header.h:62-124)."""
    if ts.type == N.TASK_LINEAR and (ts.flags & N.F_RESIDUAL):
        return 252
    if ts.type == N.TASK_LINEAR and (ts.flags & N.F_MOE):
        return 255 if ts.iarg[8] else 254      # w2 / w13 expert projections
    return _REF_TASK_TYPE.get(ts.type, ts.type)


def to_json(g: LoweredGraph) -> str:
    """Task graph in the layout of the reference's task_graph.json (src/kernel/runtime.cc:
    847-1318), so that its tools (scripts/display_task_graph.py) read it: all_tasks with
    task_type / variant_id / inputs / outputs / trigger_event / dependent_event / request_id /
    expert_offset, operands as {base_ptr = the name given at attach_input / new_tensor, offset
    in bytes, data_type, dims, strides}, all_events with event_type / num_triggers /
    first_task_id / last_task_id, and first_tasks.  "No event" is EVENT_INVALID_ID as there.
    What the reference has no field for sits under each task's "ypk" key (and the worker
    queues under the top-level "ypk_queues"): worker, operator, the task's integer
    arguments, flagged-word tags, and the runtime-internal operands (flagged-word buffers,
    split scratch), whose element types the reference's tools do not know."""
    def operand(ref):
        t, off = ref
        return {"base_ptr": t.name or f"tensor_{t.guid}", "offset": off, "dims": list(t.dims),
                "strides": list(t.strides), "data_type": t.dtype.code}

    def event_id(e):
        return e if e >= 0 else EVENT_INVALID_ID

    tasks = []
    for ti, ts in enumerate(g.tasks):
        outs = _OUTPUT_SLOTS.get(ts.type, ())
        inputs, outputs, internal = [], [], []
        for slot, p in enumerate(ts.ptr):
            if p is None:
                continue
            o = operand(p)
            if o["data_type"] not in _JSON_DTYPES or slot in _INTERNAL_SLOTS.get(ts.type, ()):
                o["slot"] = slot
                internal.append(o)
            elif slot in outs:
                outputs.append(o)
            else:
                inputs.append(o)
        inputs += [operand(p) for p in ts.logical_in]
        outputs += [operand(p) for p in ts.logical_out]
        if ts.ptr_aux is not None:     # the rows times the weight of the norm that follows
            outputs.append(operand(ts.ptr_aux))
        tasks.append({
            "task_type": ref_task_type(ts),
            "variant_id": 0,
            "inputs": inputs,
            "outputs": outputs,
            "trigger_event": event_id(ts.trig_event),
            "dependent_event": event_id(ts.dep_event),
            "request_id": ts.iarg[0] if ts.type == N.TASK_ATTENTION else -1,
            "expert_offset": -1,
            "ypk": {"task_type": N.TASK_NAMES[ts.type], "flags": ts.flags, "worker": ts.worker,
                    "op_id": ts.op_id, "dependent_count": ts.dep_count, "iarg": list(ts.iarg),
                    "farg": list(ts.farg), "flagged_inputs": list(ts.flagged_deps),
                    "flagged_output": ts.flagged_out, "internal_operands": internal},
        })
    events = []
    last_event = max((ts.trig_event for ts in g.tasks), default=-1)
    for e in range(g.num_events):
        ids = [i for i, ts in enumerate(g.tasks) if ts.dep_event == e]
        events.append({"event_type": EVENT_END_OF_TASK_GRAPH if (e == last_event and not ids)
                       else EVENT_LAUNCH_DEPENDENT_TASKS,
                       "num_triggers": sum(1 for ts in g.tasks if ts.trig_event == e),
                       "first_task_id": ids[0] if ids else 0,
                       "last_task_id": ids[-1] + 1 if ids else 0})
    first = [i for i, ts in enumerate(g.tasks) if ts.dep_event < 0]
    return json.dumps({"all_tasks": tasks, "all_events": events, "first_tasks": first,
                       "ypk_queues": {"queue": g.queue, "queue_off": g.queue_off}})
