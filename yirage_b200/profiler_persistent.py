"""Timeline export for the persistent kernel.

The reference records begin/end words per CTA (persistent_kernel/profiler.h:33-158) and
converts them to a Perfetto trace with tg4perfetto (python/yirage/profiler_persistent.py:
89-136).  This build records, for every task of the last iteration a launch ran, eight
words per (worker, queue position): {iteration << 32 | task index, t_fetch,
t_dependency_met, t_done, t_inputs_staged, t_last_stage_consumed, 0, 0} in globaltimer
nanoseconds (the fifth and sixth only for LINEAR tasks), and exports Chrome trace JSON, which
Perfetto opens and which needs no extra package.
"""
import json

import torch


def decode_records(profiler_tensor: torch.Tensor, num_workers: int, stride: int):
    """-> list of dicts {worker, slot, iteration, task, fetch, ready, done}."""
    words = profiler_tensor.detach().cpu().view(torch.int64).view(-1)
    words = words[: num_workers * stride * 8].view(num_workers, stride, 8)
    out = []
    for w in range(num_workers):
        for s in range(stride):
            tag, t0, t1, t2, t3, t4, t5, t6 = (int(v) & ((1 << 64) - 1) for v in words[w, s].tolist()[:8])
            if t2 == 0:
                continue
            out.append({"worker": w, "slot": s, "iteration": tag >> 32, "task": tag & 0xffffffff,
                        "fetch": t0, "ready": t1, "done": t2, "staged": t3, "last_stage": t4,
                        "arrived": t5, "probe": t6})
    return out


def summarize(records, tasks, ops):
    """Per operator of the last recorded iteration: when its first task became ready, when
    its last task finished, and the mean time its tasks spent waiting / executing (us)."""
    if not records:
        return []
    last = max(r["iteration"] for r in records)
    recs = [r for r in records if r["iteration"] == last]
    t0 = min(r["fetch"] for r in recs)
    rows = {}
    for r in recs:
        op = tasks[r["task"]].op_id
        e = rows.setdefault(op, {"op": op, "kind": ops[op].kind, "n": 0, "first_ready": 1 << 62,
                                 "last_done": 0, "wait": 0.0, "exec": 0.0, "max_exec": 0.0})
        e["n"] += 1
        e["first_ready"] = min(e["first_ready"], r["ready"] - t0)
        e["last_done"] = max(e["last_done"], r["done"] - t0)
        e["wait"] += (r["ready"] - r["fetch"]) / 1e3
        if r["staged"]:
            e["stage_in"] = e.get("stage_in", 0.0) + (r["staged"] - r["ready"]) / 1e3
            e["stream"] = e.get("stream", 0.0) + (r["last_stage"] - r["staged"]) / 1e3
            e["finish"] = e.get("finish", 0.0) + (r["done"] - r["last_stage"]) / 1e3
        ex = (r["done"] - r["ready"]) / 1e3
        e["exec"] += ex
        e["max_exec"] = max(e["max_exec"], ex)
    out = []
    for op in sorted(rows):
        e = rows[op]
        e["wait"] /= e["n"]
        e["exec"] /= e["n"]
        for k in ("stage_in", "stream", "finish"):
            if k in e:
                e[k] /= e["n"]
        e["first_ready"] /= 1e3
        e["last_done"] /= 1e3
        out.append(e)
    return out


def export_trace(profiler_tensor: torch.Tensor, file_name: str, num_workers: int = None,
                 stride: int = None, tasks=None):
    if num_workers is None or stride is None:
        raise ValueError("export_trace needs the worker count and the records per worker")
    events = []
    for r in decode_records(profiler_tensor, num_workers, stride):
        if tasks is None:
            name = f"task {r['task']}"
        else:
            # event names as the reference's trace has them (python/yirage/profiler_persistent.py:
            # 12-78: "<task type name>_<number>")
            from .lowering import REF_TASK_NAMES, ref_task_type
            ts = tasks[r["task"]]
            name = f"{REF_TASK_NAMES.get(ref_task_type(ts), 'TASK')}_{ts.op_id}"
        events.append({"name": "wait", "ph": "X", "ts": r["fetch"] / 1e3,
                       "dur": (r["ready"] - r["fetch"]) / 1e3, "pid": 0, "tid": r["worker"]})
        events.append({"name": name, "ph": "X", "ts": r["ready"] / 1e3,
                       "dur": (r["done"] - r["ready"]) / 1e3, "pid": 0, "tid": r["worker"]})
    path = file_name if file_name.endswith(".json") else file_name + ".trace.json"
    with open(path, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ns"}, f)
    return path


export_to_perfetto_trace = export_trace
