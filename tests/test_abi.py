"""The C-ABI library loads, exports every symbol include/ypk.h declares, and validates
graphs on a host-only handle (no GPU, no compute)."""
import ctypes as C
import os
import re

import pytest

from yirage_b200 import _native as N

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "ypk.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(ypk_[a-z_0-9]+)\s*\(", src)))


def test_every_declared_symbol_is_exported(native_lib):
    names = declared_functions()
    assert "ypk_create" in names and "ypk_launch" in names
    for name in names:
        assert hasattr(native_lib, name), f"{name} declared in ypk.h but not exported"
    assert sorted(N.SYMBOLS) == names, "ctypes prototypes and header disagree"


def test_struct_sizes_match_header(native_lib):
    assert C.sizeof(N.Task) == 176
    assert native_lib.ypk_abi_version() == N.YPK_ABI_VERSION


def host_handle(**kw):
    cfg = N.Config()
    cfg.device = -1
    cfg.world_size, cfg.rank, cfg.mode = 1, 0, 0
    cfg.max_num_batched_tokens = kw.get("max_tokens", 8)
    cfg.max_num_batched_requests = 1
    cfg.page_size = 64
    cfg.max_num_pages = 4
    return N.Handle(cfg)


def linear_task(x=0, w=1, out=2, K=512, row0=0, nrows=32, flags=0, dep=-1, depc=0, trig=0):
    t = N.Task()
    t.type, t.flags = N.TASK_LINEAR, flags
    t.dep_event, t.dep_count, t.trig_event = dep, depc, trig
    t.ptr[0], t.ptr[1], t.ptr[2] = N.ref(x), N.ref(w), N.ref(out)
    for i, v in enumerate([K, row0, nrows, K, K, 64, 0, 0]):
        t.iarg[i] = v
    return t


def test_host_only_handle_validates_and_refuses_to_launch(native_lib):
    h = host_handle()
    h.alloc(0, "x", 8 * 512 * 2)
    h.alloc(1, "w", 64 * 512 * 2)
    h.alloc(2, "out", 8 * 64 * 2)
    h.load_graph([linear_task(nrows=32), linear_task(row0=32, nrows=32)], 1, [0, 1], [0, 1, 2])
    with pytest.raises(N.YpkError) as e:
        h.launch(batch=1)
    assert e.value.code == N.ERR_STATE
    h.close()


def test_bad_graphs_are_rejected_with_a_message(native_lib):
    h = host_handle()
    h.alloc(0, "x", 8 * 512 * 2)
    h.alloc(1, "w", 64 * 512 * 2)
    h.alloc(2, "out", 8 * 64 * 2)
    cases = {
        "K % 64": [linear_task(K=520)],
        "reaches byte": [linear_task(row0=48, nrows=32)],           # rows past the weight
        "unbound tensor slot": [linear_task(w=7)],
        "operand 3 is required": [linear_task(flags=N.F_NORM)],      # norm weight missing
        "4-row granules": [linear_task(nrows=30, flags=N.F_SILU_MUL)],
        "waits for 2 triggers": [linear_task(trig=0), linear_task(dep=0, depc=2, trig=1)],
    }
    for needle, tasks in cases.items():
        with pytest.raises(N.YpkError) as e:
            h.load_graph(tasks, 2, list(range(len(tasks))), [0, len(tasks)])
        assert needle in str(e.value), (needle, str(e.value))
    # queue that runs tasks out of dependency order
    with pytest.raises(N.YpkError) as e:
        h.load_graph([linear_task(trig=0), linear_task(dep=0, depc=1, trig=1)], 2, [1, 0], [0, 2])
    assert "not in task order" in str(e.value)
    h.close()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(N, "_lib", None)
    monkeypatch.setattr(N, "LIB_PATH", str(tmp_path / "libypk.so"))
    with pytest.raises(ImportError):
        N.load()
