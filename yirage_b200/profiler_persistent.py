"""Trace export for the persistent kernel (python/yirage/profiler_persistent.py:89-136 in
the reference writes a Perfetto trace through tg4perfetto).  This build exports Chrome
trace JSON, which needs no extra package and loads in Perfetto as well.

Record format (one uint64 per record, as the reference's profiler.h:33-44): tag in the
high 32 bits (event_no << 19 | block_group << 11 | event_type << 2 | begin/end), low 32
bits of %globaltimer in the low half.  The device side of this build does not write
records yet; a buffer of zeros exports as an empty trace.
"""
import json

import torch


def decode_records(profiler_tensor: torch.Tensor):
    vals = profiler_tensor.detach().cpu().view(torch.int64).tolist()
    out = []
    for v in vals:
        v &= (1 << 64) - 1
        if v == 0:
            continue
        tag, ts = v >> 32, v & 0xffffffff
        out.append({"event_no": tag >> 19, "block_group": (tag >> 11) & 0xff,
                    "event_type": (tag >> 2) & 0x1ff, "phase": "B" if (tag & 3) == 0 else "E",
                    "ts_ns": ts})
    return out


def export_trace(profiler_tensor: torch.Tensor, file_name: str):
    events = [{"name": f"task_{r['event_type']}", "ph": r["phase"], "ts": r["ts_ns"] / 1000.0,
               "pid": 0, "tid": r["block_group"]} for r in decode_records(profiler_tensor)]
    path = file_name if file_name.endswith(".json") else file_name + ".trace.json"
    with open(path, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ns"}, f)
    return path


# name used by the reference
export_to_perfetto_trace = export_trace
