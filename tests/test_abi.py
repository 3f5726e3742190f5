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


def test_carried_norm_operands_are_validated(native_lib):
    """YPK_F_NORM_OUT / YPK_F_NORM_PRE: the ninth operand, the sums-of-squares buffer and the
    graph size are checked when the graph is loaded."""
    h = host_handle(max_tokens=64)
    h.alloc(0, "x", 64 * 256 * 2)
    h.alloc(1, "w", 64 * 256 * 2)
    h.alloc(2, "out", 64 * 64 * 2)
    h.alloc(3, "g", 64 * 2)
    h.alloc(4, "ss", 64 * 4)
    h.alloc(5, "xg", 64 * 64 * 2)

    def task(flags, g=True, ssbuf=True, aux=True, ss=0 | (64 << 16)):
        t = linear_task(K=256, nrows=64, flags=flags)
        t.iarg[12] = ss
        if g:
            t.ptr[3] = N.ref(3)
        if ssbuf:
            t.ptr[6] = N.ref(4)
        if aux:
            t.ptr_aux = N.ref(5)
        return t

    h.load_graph([task(N.F_NORM_OUT)], 1, [0], [0, 1])
    for bad, msg in ((task(N.F_NORM_OUT, aux=False), "operand 8 is required"),
                     (task(N.F_NORM_OUT, ss=0 | (8 << 16)), "sums of squares for 8 tokens"),
                     (task(N.F_NORM_OUT, ss=1 | (64 << 16)), "reaches byte"),   # block 1 of a one-row buffer
                     (task(0, g=False, ssbuf=False), "takes no ninth operand"),
                     (task(N.F_NORM_OUT | N.F_NORM_PRE), "NORM_PRE and NORM_OUT"),
                     (task(N.F_NORM_OUT | N.F_NORM), "plain 16-bit rows")):
        with pytest.raises(N.YpkError) as e:
            h.load_graph([bad], 1, [0], [0, 1])
        assert msg in str(e.value), str(e.value)
    # graphs of at most 8 tokens have no such form
    h8 = host_handle(max_tokens=8)
    for slot, n in ((0, 8 * 256 * 2), (1, 64 * 256 * 2), (2, 8 * 64 * 2), (3, 128), (4, 32), (5, 8 * 64 * 2)):
        h8.alloc(slot, f"t{slot}", n)
    with pytest.raises(N.YpkError) as e:
        h8.load_graph([task(N.F_NORM_OUT, ss=0 | (8 << 16))], 1, [0], [0, 1])
    assert "more than 8 tokens" in str(e.value)
