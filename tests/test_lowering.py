"""Host logic of the task-graph generator: fusion, balanced row partition, events,
queues, the protocol simulator, JSON export, and validation of a whole Llama graph by the
native library on a host-only handle (no GPU)."""
import json

import pytest
import torch

import yirage_b200 as yr
from yirage_b200 import _native as N
from yirage_b200 import llama, lowering


def small_graph(world_size=1, rank=0, layers=2, handoff="event"):
    shape = llama.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=layers,
                             num_attention_heads=8, num_key_value_heads=2, vocab_size=2048)
    w = llama.init_weights(shape, "cpu", 0)
    tokens = torch.zeros(2, 128, dtype=torch.int64)
    pl = torch.tensor([5, 7], dtype=torch.int32)
    return shape, llama.build_decode_kernel(
        shape, w, tokens=tokens, prompt_lengths=pl, max_num_batched_requests=2,
        max_num_batched_tokens=8, max_num_pages=8, page_size=64, compile=False,
        handoff=handoff)[0]


def test_demo_layer_sequence_fuses_to_five_operators_per_layer():
    _, ypk = small_graph()
    g = ypk.lower(148)
    kinds = [o.kind for o in g.ops]
    assert kinds == ["embed"] + ["linear", "attention", "linear", "linear", "linear"] * 2 + \
        ["linear", "argmax_partial", "argmax_reduce"]
    qkv, o_proj, gate_up, down = g.ops[1], g.ops[3], g.ops[4], g.ops[5]
    assert qkv.flags & N.F_NORM and not qkv.flags & N.F_RESIDUAL
    assert o_proj.flags & N.F_RESIDUAL and not o_proj.flags & N.F_NORM
    assert gate_up.flags & N.F_NORM and gate_up.flags & N.F_SILU_MUL
    assert gate_up.t["out"].name == "silu_mul_out", "mlp_mid must not be materialised"
    assert down.flags & N.F_RESIDUAL
    # fused gate/up weights are interleaved in 2-row granules, qkv per kv head
    gran = {sh["dst"].name: sh["gran"] for sh in g.shuffles}
    assert gran["layer_0_gatedup_proj"] == [2, 2]
    assert gran["layer_0_qkv_proj"] == [4 * 128, 128, 128]


def test_every_task_runs_once_per_iteration_and_graph_cannot_deadlock():
    _, ypk = small_graph()
    g = ypk.lower(148)
    assert set(lowering.simulate(g, iterations=3)) == {3}
    # whole-operator events: the dependency count equals the producer's task count
    per_op = {}
    for ts in g.tasks:
        per_op[ts.op_id] = per_op.get(ts.op_id, 0) + 1
    for ts in g.tasks:
        if ts.op_id == 0:
            assert ts.dep_event == -1
        else:
            assert ts.dep_event == ts.op_id - 1 and ts.dep_count == per_op[ts.op_id - 1]
    # queues are in task order
    for a, b in zip(g.queue_off[:-1], g.queue_off[1:]):
        assert g.queue[a:b] == sorted(g.queue[a:b])


def test_flagged_word_handoff_plan():
    """At most 8 tokens: the residual stream and the MLP activation travel as flagged words.
    Their readers wait for no event, their producers trigger none; everything else keeps the
    whole-operator events."""
    _, ypk = small_graph(handoff="ll")
    g = ypk.lower(148)
    assert set(lowering.simulate(g, iterations=3)) == {3}
    kinds = [o.kind for o in g.ops]
    by_op = {}
    for ts in g.tasks:
        by_op.setdefault(ts.op_id, []).append(ts)
    LL = N.F_LL_IN | N.F_LL_RES | N.F_LL_OUT | N.F_LL_PUSH
    # layer 0: qkv (x from the embedding: event), attention, o_proj (residual from the
    # embedding: event), gate/up, down; layer 1: everything flagged
    qkv0, att0, o0, gu0, dn0, qkv1, att1, o1 = (by_op[i][0] for i in range(1, 9))
    assert qkv0.flags & LL == N.F_LL_OUT and qkv0.dep_event == 0 and qkv0.trig_event == -1
    assert att0.flags & LL == N.F_LL_IN | N.F_LL_OUT and att0.dep_event == -1 and att0.trig_event == 2
    assert o0.flags & LL == N.F_LL_IN | N.F_LL_OUT and o0.dep_event == 2 and o0.trig_event == -1
    assert gu0.flags & LL == N.F_LL_IN | N.F_LL_OUT and gu0.dep_event == -1 and gu0.trig_event == -1
    assert dn0.flags & LL == N.F_LL_IN | N.F_LL_RES | N.F_LL_OUT and dn0.dep_event == -1
    assert qkv1.flags & LL == N.F_LL_IN | N.F_LL_OUT and qkv1.dep_event == -1 and qkv1.trig_event == -1
    assert att1.dep_event == -1 and att1.trig_event == -1
    assert o1.flags & LL == N.F_LL_IN | N.F_LL_RES | N.F_LL_OUT and o1.dep_event == -1
    # tags: a reader polls for the tag its producer writes
    assert att0.flagged_deps == [qkv0.flagged_out] and o0.flagged_deps == [att0.flagged_out]
    assert gu0.flagged_deps == [o0.flagged_out] and dn0.flagged_deps == [gu0.flagged_out, o0.flagged_out]
    assert qkv1.flagged_deps == [dn0.flagged_out]
    assert o1.flagged_deps == [att1.flagged_out, dn0.flagged_out]
    # a tensor wider than MAX_FLAGGED_COLS keeps its event
    wide = lowering.MAX_FLAGGED_COLS
    lowering.MAX_FLAGGED_COLS = 512
    try:
        _, ypk2 = small_graph(handoff="ll")
        g2 = ypk2.lower(148)
        dn = [ts for ts in g2.tasks if ts.op_id == 5][0]
        gu = [ts for ts in g2.tasks if ts.op_id == 4][0]
        assert not dn.flags & N.F_LL_IN and dn.dep_event == 4 and gu.trig_event == 4
        assert set(lowering.simulate(g2, iterations=2)) == {2}
    finally:
        lowering.MAX_FLAGGED_COLS = wide
    # flagged results come in pairs of columns: rows of every such slab are even
    for ts in g.tasks:
        if ts.type == N.TASK_LINEAR and ts.flags & (N.F_LL_OUT | N.F_LL_RES):
            assert ts.iarg[1] % 2 == 0 and ts.iarg[2] % 2 == 0
    # the lm_head reads flagged words and hands its logits to the arg-max through an event
    lm = by_op[kinds.index("argmax_partial") - 1][0]
    assert lm.flags & LL == N.F_LL_IN and lm.trig_event >= 0
    # dropping a producer is caught
    victim = next(i for i, ts in enumerate(g.tasks) if ts.flagged_out == gu0.flagged_out)
    g.tasks[victim].flagged_out = -1
    g.tasks[victim].flagged_deps = [255]
    with pytest.raises(RuntimeError, match="deadlock"):
        lowering.simulate(g, iterations=1)


def test_a_broken_dependency_is_caught_by_the_simulator():
    _, ypk = small_graph()
    g = ypk.lower(148)
    g.tasks[-1].dep_count += 1          # waits for a trigger nobody sends
    with pytest.raises(RuntimeError, match="deadlock"):
        lowering.simulate(g, iterations=1)


def test_weight_rows_are_covered_exactly_once_and_bytes_are_level(monkeypatch):
    shape, ypk = small_graph()
    g = ypk.lower(148)
    # workers that run an attention task get less of the operator after it
    att = next(oi for oi, op in enumerate(g.ops) if op.kind == "attention")
    att_workers = {ts.worker for ts in g.tasks if ts.op_id == att}
    rows_after = {ts.worker: ts.iarg[2] for ts in g.tasks if ts.op_id == att + 1}
    assert max(rows_after.get(w, 0) for w in att_workers) <= min(
        rows_after.get(w, 0) for w in range(148) if w not in att_workers)
    # without that allowance the cumulative bytes are level
    monkeypatch.setattr(lowering, "ATTN_LOAD_BYTES", 0)
    shape, ypk = small_graph()
    g = ypk.lower(148)
    for oi, op in enumerate(g.ops):
        if op.kind != "linear":
            continue
        rows = sorted((ts.iarg[1], ts.iarg[2]) for ts in g.tasks if ts.op_id == oi)
        pos = 0
        for r0, n in rows:
            assert r0 == pos and 0 < n <= lowering.MAX_TASK_ROWS
            pos += n
        assert pos == op.t["w"].dims[0]
    total = shape.decode_weight_bytes(1, llama.padded_vocab(shape.vocab_size))
    assert sum(g.worker_bytes) == total
    assert max(g.worker_bytes) - min(g.worker_bytes) <= 2 * 16 * 1024 * 2  # two granules of the widest K


def test_level_partition_water_fills():
    counts = lowering.level_partition(10, 100, [0.0, 300.0, 0.0, 0.0])
    assert sum(counts) == 10 and counts[1] <= 2 and max(counts) - min(c for i, c in enumerate(counts) if i != 1) <= 1
    assert lowering.level_partition(0, 10, [0.0, 0.0]) == [0, 0]
    assert sum(lowering.level_partition(7, 5, [1e9, 0.0, 0.0])) == 7


def test_unfusable_patterns_stay_separate():
    ypk = yr.PersistentKernel(mode="onepass", world_size=1, mpi_rank=0, num_workers=128,
                              num_local_schedulers=0, num_remote_schedulers=0, max_seq_length=64,
                              max_num_batched_requests=1, max_num_batched_tokens=8, max_num_pages=1,
                              page_size=64, eos_token_id=-1, meta_tensors={})
    x = ypk.attach_input(torch.zeros(8, 512, dtype=torch.bfloat16), "x")
    nw = ypk.attach_input(torch.zeros(512, dtype=torch.bfloat16), "nw")
    w1 = ypk.attach_input(torch.zeros(256, 512, dtype=torch.bfloat16), "w1")
    w2 = ypk.attach_input(torch.zeros(256, 512, dtype=torch.bfloat16), "w2")
    normed = ypk.new_tensor(dims=(8, 512), name="normed")
    o1, o2 = ypk.new_tensor(dims=(8, 256), name="o1"), ypk.new_tensor(dims=(8, 256), name="o2")
    ypk.rmsnorm_layer(x, nw, normed, (8, 1, 1), (128, 1, 1))
    ypk.linear_layer(normed, w1, o1, (4, 1, 1), (128, 1, 1))
    ypk.linear_layer(normed, w2, o2, (4, 1, 1), (128, 1, 1))   # second reader of `normed`
    assert [o.kind for o in ypk.lower(148).ops] == ["rmsnorm", "linear", "linear"]


def test_out_of_scope_builders_say_so():
    _, ypk = small_graph()
    with pytest.raises(NotImplementedError):
        ypk.attention_layer()            # contiguous-KV attention of the reference's older demos
    with pytest.raises(NotImplementedError):
        ypk.identity_layer()


def test_online_mode_is_the_one_request_case_of_the_batcher():
    """MODE_ONLINE of the reference (persistent_kernel.cuh:325-352) serves one request."""
    i32 = dict(dtype=torch.int32)
    def meta(requests):
        return {"tokens": torch.zeros(requests, 64, dtype=torch.int64),
                "qo_indptr_buffer": torch.zeros(2, **i32), "paged_kv_indptr_buffer": torch.zeros(2, **i32),
                "paged_kv_indices_buffer": torch.zeros(1, **i32),
                "paged_kv_last_page_len_buffer": torch.zeros(1, **i32)}
    kw = dict(mode="online", world_size=1, mpi_rank=0, num_workers=1, num_local_schedulers=0,
              num_remote_schedulers=0, max_seq_length=64, max_num_batched_requests=1,
              max_num_batched_tokens=8, max_num_pages=1, page_size=64, eos_token_id=0)
    ypk = yr.PersistentKernel(meta_tensors=meta(1), **kw)
    assert ypk.online and ypk.mode == "offline" and ypk.total_num_requests == 1
    with pytest.raises(ValueError):
        yr.PersistentKernel(meta_tensors=meta(2), **kw)


# TaskType / EventType numbers of the reference (persistent_kernel/runtime_header.h:62-134) and
# the element types its tools accept (scripts/display_task_graph.py:34-38)
REF_TASK_TYPES = {101, 107, 118, 154, 252, 253, 257, 258, 259}
REF_EVENT_TYPES = {900, 901, 902, 903, 910, 911, 999}
EVENT_INVALID_ID = 0x7ffffffffffffffe


@pytest.mark.parametrize("handoff", ["event", "ll"])
def test_task_graph_json_follows_the_reference_layout(handoff):
    """Every key scripts/display_task_graph.py and the reference's JSON loader
    (runtime.cc:650-745) read is there with the reference's types and conventions."""
    _, ypk = small_graph(handoff=handoff)
    res = ypk.kn_graph.generate_task_graph(num_gpus=1, my_gpu_id=0)
    assert set(res) == {"json_file", "cuda_code"}
    j = json.loads(res["json_file"])
    assert {"all_tasks", "all_events", "first_tasks"} <= set(j)
    for t in j["all_tasks"]:
        assert {"task_type", "variant_id", "inputs", "outputs", "trigger_event", "dependent_event",
                "request_id", "expert_offset"} <= set(t)
        assert t["task_type"] in REF_TASK_TYPES and isinstance(t["variant_id"], int)
        for ev in (t["trigger_event"], t["dependent_event"]):
            assert ev == EVENT_INVALID_ID or 0 <= ev < len(j["all_events"])
        for o in t["inputs"] + t["outputs"]:
            assert set(o) == {"base_ptr", "offset", "dims", "strides", "data_type"}
            assert isinstance(o["base_ptr"], str) and o["base_ptr"]
            assert o["data_type"] in (940, 941, 965) and o["offset"] >= 0
            assert len(o["dims"]) == len(o["strides"])
        assert t["outputs"], "every task names what it writes"
    for e in j["all_events"]:
        assert set(e) == {"event_type", "num_triggers", "first_task_id", "last_task_id"}
        assert e["event_type"] in REF_EVENT_TYPES
    triggering = [t for t in j["all_tasks"] if t["trigger_event"] != EVENT_INVALID_ID]
    assert sum(e["num_triggers"] for e in j["all_events"]) == len(triggering)
    assert all(j["all_tasks"][i]["dependent_event"] == EVENT_INVALID_ID for i in j["first_tasks"])


def test_reference_display_script_reads_the_emitted_task_graph(tmp_path, monkeypatch):
    """scripts/display_task_graph.py of the reference, run unchanged on a task_graph.json this
    build emitted.  graphviz and matplotlib are not installed here, so the two names the
    script takes from them are stood in for by recorders; everything else (the enum parsing
    from the reference headers, the walk over tasks, events and operands) is its own code."""
    import os, sys, types, importlib.util
    ref = os.environ.get("YIRAGE_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
    script = os.path.join(ref, "scripts", "display_task_graph.py")
    if not os.path.exists(script):
        pytest.skip("reference tree not mounted")
    nodes, edges = [], []

    class Digraph:
        def attr(self, *a, **k): pass
        def node(self, name, label=None): nodes.append(name)
        def edge(self, a, b): edges.append((a, b))
        def save(self, path): open(path, "w").write("digraph {}")

    gv = types.ModuleType("graphviz"); gv.Digraph = Digraph
    mpl = types.ModuleType("matplotlib"); colors = types.ModuleType("matplotlib.colors")
    colors.CSS4_COLORS = {f"colour{i}": "#000000" for i in range(400)}
    mpl.colors = colors
    for name, mod in (("graphviz", gv), ("matplotlib", mpl), ("matplotlib.colors", colors)):
        monkeypatch.setitem(sys.modules, name, mod)
    monkeypatch.setenv("YIRAGE_HOME", ref)
    _, ypk = small_graph()
    path = tmp_path / "task_graph.json"
    path.write_text(ypk.kn_graph.generate_task_graph(num_gpus=1, my_gpu_id=0)["json_file"])
    spec = importlib.util.spec_from_file_location("ref_display_task_graph", script)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.display_task_graph(str(path), False)
    g = ypk.lower()
    assert sum(n.startswith("task_") for n in nodes) == g.num_tasks
    assert sum(n.startswith("event_") for n in nodes) == g.num_events + 1   # + the base event
    assert len(edges) == 2 * g.num_tasks
    assert (tmp_path / "task_graph.dot").exists()


def test_events_follow_tensors_so_independent_chains_do_not_wait_for_each_other():
    """Two chains that share only a graph input: x -> A1 -> A2 and x -> B1 -> B2.  An
    operator waits for the producer of what it reads (src/kernel/runtime.cc:446-503), not for
    whatever was registered before it."""
    ypk = yr.PersistentKernel(
        mode="onepass", world_size=1, mpi_rank=0, num_workers=128, num_local_schedulers=0,
        num_remote_schedulers=0, max_seq_length=64, max_num_batched_requests=1,
        max_num_batched_tokens=8, max_num_pages=1, page_size=64, eos_token_id=-1, meta_tensors={})
    ypk.handoff = "event"
    x = ypk.attach_input(torch.zeros(16, 512, dtype=torch.bfloat16), "x")
    def chain(tag):
        w1 = ypk.attach_input(torch.zeros(512, 512, dtype=torch.bfloat16), f"{tag}w1")
        w2 = ypk.attach_input(torch.zeros(512, 512, dtype=torch.bfloat16), f"{tag}w2")
        h = ypk.new_tensor(dims=(16, 512), name=f"{tag}h")
        y = ypk.new_tensor(dims=(16, 512), name=f"{tag}y")
        ypk.linear_layer(x, w1, h, (8, 1, 1), (128, 1, 1))
        ypk.linear_layer(h, w2, y, (8, 1, 1), (128, 1, 1))
    chain("a")
    chain("b")
    g = ypk.lower(148)
    assert [o.kind for o in g.ops] == ["linear"] * 4
    assert lowering.tensor_dependencies(g.ops, serving=False) == [-1, 0, -1, 2]
    dep = {ts.op_id: ts.dep_event for ts in g.tasks}
    assert dep == {0: -1, 1: 0, 2: -1, 3: 2}
    trig = {ts.op_id: ts.trig_event for ts in g.tasks}
    assert trig == {0: 0, 1: -1, 2: 2, 3: 3}, "only awaited operators (and the last) publish an event"
    assert set(lowering.simulate(g, 1)) == {1}
    ypk.compile(dry_run=True)       # the native validation accepts it
    ypk.finalize()
    # a buffer reused by the second chain orders it after the first chain's reader
    ypk2 = yr.PersistentKernel(
        mode="onepass", world_size=1, mpi_rank=0, num_workers=128, num_local_schedulers=0,
        num_remote_schedulers=0, max_seq_length=64, max_num_batched_requests=1,
        max_num_batched_tokens=8, max_num_pages=1, page_size=64, eos_token_id=-1, meta_tensors={})
    ypk2.handoff = "event"
    x = ypk2.attach_input(torch.zeros(16, 512, dtype=torch.bfloat16), "x")
    h = ypk2.new_tensor(dims=(16, 512), name="h")
    ws = [ypk2.attach_input(torch.zeros(512, 512, dtype=torch.bfloat16), f"w{i}") for i in range(4)]
    ys = [ypk2.new_tensor(dims=(16, 512), name=f"y{i}") for i in range(2)]
    ypk2.linear_layer(x, ws[0], h, (8, 1, 1), (128, 1, 1))
    ypk2.linear_layer(h, ws[1], ys[0], (8, 1, 1), (128, 1, 1))
    ypk2.linear_layer(x, ws[2], h, (8, 1, 1), (128, 1, 1))      # overwrites h: after its reader
    ypk2.linear_layer(h, ws[3], ys[1], (8, 1, 1), (128, 1, 1))
    assert lowering.tensor_dependencies(ypk2.lower(148).ops, serving=False) == [-1, 0, 1, 2]
    # serving graphs end every iteration on the last operator: the chain is kept when the last
    # operator's completion would not imply everybody's
    assert lowering.tensor_dependencies(g.ops, serving=True) is None


def test_embedding_and_argmax_tasks_carry_the_real_table_and_vocabulary_sizes():
    shape, ypk = small_graph()
    g = ypk.lower(148)
    emb = [t for t in g.tasks if t.type == N.TASK_EMBED]
    assert emb and all(t.iarg[5] == shape.vocab_size for t in emb)
    part = [t for t in g.tasks if t.type == N.TASK_ARGMAX_PARTIAL]
    assert part and all(t.iarg[5] == shape.vocab_size for t in part)


def test_embed_task_without_a_row_count_is_refused(native_lib):
    from tests.test_abi import host_handle
    h = host_handle()
    h.alloc(0, "ids", 8 * 8)
    h.alloc(1, "table", 100 * 512 * 2)
    h.alloc(2, "out", 8 * 512 * 2)
    t = N.Task()
    t.type, t.dep_event, t.trig_event = N.TASK_EMBED, -1, 0
    t.ptr[0], t.ptr[1], t.ptr[2] = N.ref(0), N.ref(1), N.ref(2)
    for i, v in enumerate([512, 0, 512, 512, 512, 0]):
        t.iarg[i] = v
    with pytest.raises(N.YpkError, match="row count"):
        h.load_graph([t], 1, [0], [0, 1])
    t.iarg[5] = 101                                  # one row more than the table holds
    with pytest.raises(N.YpkError, match="reaches byte"):
        h.load_graph([t], 1, [0], [0, 1])
    t.iarg[5] = 100
    h.load_graph([t], 1, [0], [0, 1])
    h.close()


def _tp_graph(n_allreduce_layers, handoff, world=2):
    """A tensor-parallel graph with `n` all-reduces per iteration: x -> (linear -> allreduce) x n."""
    ypk = yr.PersistentKernel(
        mode="onepass", world_size=world, mpi_rank=0, num_workers=128, num_local_schedulers=0,
        num_remote_schedulers=0, max_seq_length=64, max_num_batched_requests=1,
        max_num_batched_tokens=8, max_num_pages=1, page_size=64, eos_token_id=-1, meta_tensors={})
    ypk.handoff = handoff
    x = ypk.attach_input(torch.zeros(8, 512, dtype=torch.bfloat16), "x")
    buf = ypk.new_tensor(dims=(world, 8, 512), name="buf", io_category="nvshmem_tensor")
    for i in range(n_allreduce_layers):
        w = ypk.attach_input(torch.zeros(512, 512, dtype=torch.bfloat16), f"w{i}")
        part = ypk.new_tensor(dims=(8, 512), name=f"part{i % 2}_{i}", io_category="nvshmem_tensor")
        out = ypk.new_tensor(dims=(8, 512), name=f"sum{i}", io_category="nvshmem_tensor")
        ypk.linear_layer(x, w, part, (8, 1, 1), (128, 1, 1))
        ypk.allreduce_layer(part, buf, out, (8, 1, 1), (128, 1, 1))
        x = out
    wl = ypk.attach_input(torch.zeros(512, 512, dtype=torch.bfloat16), "w_last")
    y = ypk.new_tensor(dims=(8, 512), name="y")
    ypk.linear_layer(x, wl, y, (8, 1, 1), (128, 1, 1))
    return ypk


@pytest.mark.parametrize("n", [1, 2, 3])
def test_allreduce_buffer_halves_alternate_for_any_count_per_iteration(n):
    """Event form: the half is the parity of the running all-reduce number, so with an odd
    count per iteration the last all-reduce of one iteration and the first of the next still
    differ (the task carries index and count, the device adds iterations * count)."""
    g = _tp_graph(n, "event").lower(148)
    ar = [t for t in g.tasks if t.type == N.TASK_ALLREDUCE]
    assert {t.iarg[6] for t in ar} == set(range(n)) and {t.iarg[10] for t in ar} == {n}
    halves = [((it * n + k) & 1) for it in range(4) for k in range(n)]
    assert all(a != b for a, b in zip(halves, halves[1:]))


def test_single_buffered_pushes_are_used_only_where_consecutive_allreduces_differ():
    """Flagged-word form: a peer's slot may be overwritten once that peer has pushed the next
    all-reduce.  With one all-reduce per iteration the next one is the same buffer: such
    a graph keeps the event form."""
    one = _tp_graph(1, "ll").lower(148)
    assert not any(t.flags & N.F_LL_PUSH for t in one.tasks)
    assert all(not (t.flags & N.F_LL_IN) for t in one.tasks if t.type == N.TASK_ALLREDUCE)
    two = _tp_graph(2, "ll").lower(148)
    assert any(t.flags & N.F_LL_PUSH for t in two.tasks)
    for g in (one, two):
        assert set(lowering.simulate(g, 2)) == {2}


def test_more_flagged_producers_than_tag_ids_do_not_confuse_the_simulator():
    """40 layers under 2-way tensor parallelism have 284 flagged producers for 254 tag ids:
    the ids repeat on the device (never twice on one buffer within an iteration), the plan
    and the simulator tell the producers apart."""
    shape = llama.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=40,
                             num_attention_heads=8, num_key_value_heads=2, vocab_size=2048)
    w = llama.init_weights(shape, "cpu", 0, world_size=2, rank=0)
    tokens = torch.zeros(1, 64, dtype=torch.int64)
    ypk, _ = llama.build_decode_kernel(shape, w, tokens=tokens, prompt_lengths=torch.tensor([5], dtype=torch.int32),
                                       max_num_batched_requests=1, max_num_batched_tokens=8, max_num_pages=1,
                                       page_size=64, world_size=2, rank=0, compile=False, handoff="ll")
    g = ypk.lower(148)
    outs = {t.flagged_out for t in g.tasks if t.flagged_out >= 0}
    assert len(outs) > 254
    assert set(lowering.simulate(g, 2)) == {2}


def test_qk_norm_attention_lowers_with_packed_weights(native_lib):
    """Dense Qwen3 form: q/k RMSNorm inside the attention task (demo/qwen3/demo.py:444-476)."""
    shape = llama.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                             num_attention_heads=8, num_key_value_heads=2, vocab_size=2048,
                             rms_norm_eps=1e-6, qk_norm=True)
    w = llama.init_weights(shape, "cpu", 0)
    tokens = torch.zeros(1, 64, dtype=torch.int64)
    ypk, _ = llama.build_decode_kernel(shape, w, tokens=tokens, prompt_lengths=torch.tensor([5], dtype=torch.int32),
                                       max_num_batched_requests=1, max_num_batched_tokens=8, max_num_pages=1,
                                       page_size=64, compile=False)
    g = ypk.lower(148)
    att = [t for t in g.tasks if t.type == N.TASK_ATTENTION]
    assert att and all(t.flags & N.F_QK_NORM and t.ptr[7] is not None for t in att)
    assert all(abs(t.farg[0] - 1e-6) < 1e-12 for t in att)
    packed = [sh for sh in g.shuffles if sh["rows"] == [1, 1]]
    assert len(packed) == 2 and packed[0]["row_bytes"] == 256
    assert [s.name for s in packed[0]["sources"]] == ["layer_0_q_norm", "layer_0_k_norm"]
    ypk.compile(dry_run=True)
    ypk.finalize()


def test_native_library_accepts_the_lowered_llama_graph(native_lib):
    _, ypk = small_graph()
    ypk.compile(dry_run=True)          # host-only handle: bind, shuffle, validate, resolve
    with pytest.raises(RuntimeError):
        ypk()                          # no device, no launch - and no silent fallback
    ypk.finalize()


def test_compile_without_a_gpu_fails_loudly():
    if torch.cuda.is_available():
        pytest.skip("needs a machine without a GPU")
    _, ypk = small_graph()
    with pytest.raises(RuntimeError, match="no CPU execution path"):
        ypk.compile()


def test_kernel_graph_matching():
    from yirage_b200.micrograph import MicroGraphExecutor
    g = yr.new_kernel_graph()
    X = g.new_input(dims=(8, 4096), dtype=yr.float16)
    W = g.new_input(dims=(4096, 4096), dtype=yr.float16)
    g.mark_output(g.matmul(g.rms_norm(X, normalized_shape=(4096,)), W))
    plan = MicroGraphExecutor(g.cygraph).plan
    assert [p[0] for p in plan] == ["linear"] and plan[0][2] is True      # norm folded in
    g2 = yr.new_kernel_graph()
    X = g2.new_input(dims=(8, 4096), dtype=yr.bfloat16)
    W1 = g2.new_input(dims=(4096, 4096), dtype=yr.bfloat16)
    W2 = g2.new_input(dims=(4096, 4096), dtype=yr.bfloat16)
    g2.mark_output(g2.mul(g2.silu(g2.matmul(X, W1)), g2.matmul(X, W2)))
    assert [p[0] for p in MicroGraphExecutor(g2.cygraph).plan] == ["gated"]
    g3 = yr.new_kernel_graph()
    A = g3.new_input(dims=(8, 64), dtype=yr.bfloat16)
    g3.mark_output(g3.silu(A))
    with pytest.raises(NotImplementedError):
        MicroGraphExecutor(g3.cygraph)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU execution path"):
            g.superoptimize()(inputs=[torch.zeros(8, 4096, dtype=torch.float16),
                                      torch.zeros(4096, 4096, dtype=torch.float16)])


def test_70b_shape_lowers_and_validates_under_tp8():
    """BASELINE's 70B shape (hidden 8192, 64 q / 8 kv heads, FFN 28672) sharded 8 ways, one
    layer and a small vocabulary: grid hints divide the sharded dimensions, the residual
    stream (8192 wide) still travels as flagged words, one kv head per rank, and the native
    library accepts the graph on a host-only handle."""
    shape = llama.LlamaShape(hidden_size=8192, intermediate_size=28672, num_hidden_layers=1,
                             num_attention_heads=64, num_key_value_heads=8, vocab_size=16384)
    w = llama.init_weights(shape, "cpu", 0, world_size=8, rank=3)
    tokens = torch.zeros(1, 128, dtype=torch.int64)
    pl = torch.tensor([40], dtype=torch.int32)
    ypk, _ = llama.build_decode_kernel(shape, w, tokens=tokens, prompt_lengths=pl,
                                       max_num_batched_requests=1, max_num_batched_tokens=8,
                                       max_num_pages=2, page_size=64, world_size=8, rank=3,
                                       compile=False)
    g = ypk.lower(148)
    assert set(lowering.simulate(g, 2)) == {2}
    kinds = [o.kind for o in g.ops]
    assert kinds.count("allreduce") == 2 and kinds.count("attention") == 1
    att = [t for t in g.tasks if t.type == N.TASK_ATTENTION]
    assert {t.iarg[4] for t in att} == {8} and {t.iarg[5] for t in att} == {1}
    gate_up = [t for t in g.tasks if t.op_id == kinds.index("allreduce") + 1][0]
    assert gate_up.flags & N.F_LL_IN and gate_up.iarg[0] == 8192
    red = [t for t in g.tasks if t.type == N.TASK_ARGMAX_REDUCE][0]
    assert red.flags & N.F_LL_PUSH and red.iarg[1] == 3 * (llama.padded_vocab(16384) // 8)
    ypk.compile(dry_run=True, defer_connect=True)
    ypk.finalize()


def test_wide_graphs_split_narrow_operators_along_k(native_lib):
    """More than 8 tokens: an operator with few rows per worker becomes row blocks x K ranges
    (about one task per worker, 100+ rows each) whose partial sums meet in a workspace; wide
    operators keep plain row slabs.  The native validation accepts the graph."""
    assert lowering.splitk_plan(4096, 4096, 1, 148) == (112, 4)        # o_proj of Llama-3-8B
    assert lowering.splitk_plan(6144, 4096, 1, 148) == (128, 3)        # qkv
    assert lowering.splitk_plan(28672, 4096, 4, 148) is None           # gate/up: 194 rows per worker
    shape = llama.LlamaShape(hidden_size=1024, intermediate_size=2048, num_hidden_layers=1,
                             num_attention_heads=8, num_key_value_heads=2, vocab_size=2048)
    w = llama.init_weights(shape, "cpu", 0)
    tokens = torch.zeros(4, 64, dtype=torch.int64)
    ypk, _ = llama.build_decode_kernel(shape, w, tokens=tokens, prompt_lengths=torch.full((4,), 9, dtype=torch.int32),
                                       max_num_batched_requests=4, max_num_batched_tokens=32, max_num_pages=4,
                                       page_size=64, compile=False)
    g = ypk.lower(148)
    lin = [t for t in g.tasks if t.type == N.TASK_LINEAR]
    split = [t for t in lin if (t.iarg[15] >> 8) & 0xff > 1]
    assert split
    by_block = {}
    for t in split:
        by_block.setdefault((t.op_id, t.iarg[10]), []).append(t)
    for (op, blk), ts in by_block.items():
        S = (ts[0].iarg[15] >> 8) & 0xff
        assert sorted(t.iarg[15] & 0xff for t in ts) == list(range(S)), "every split of a block once"
        assert len({(t.iarg[1], t.iarg[2]) for t in ts}) == 1, "the splits of a block share its rows"
        assert sum(t.iarg[14] for t in ts) == ts[0].iarg[0], "the K ranges tile K"
        assert all(t.iarg[13] % 64 == 0 and t.iarg[14] % 64 == 0 for t in ts)
        assert len({t.worker for t in ts}) == S, "on different workers"
    # rows of every operator are covered exactly once per split
    for op in {t.op_id for t in split}:
        rows = sorted((t.iarg[1], t.iarg[2]) for t in split if t.op_id == op and (t.iarg[15] & 0xff) == 0)
        assert rows[0][0] == 0 and all(a[0] + a[1] == b[0] for a, b in zip(rows, rows[1:]))
    assert set(lowering.simulate(g, 2)) == {2}
    ypk.compile(dry_run=True)
    ypk.finalize()


def test_prompt_lookup_graph_lowers_and_validates(native_lib):
    """Speculative decoding by prompt lookup (demo/qwen3/demo.py:377-384,457-470,625-632): the
    draft operators sit in front of the embedding, which reads the draft ids; the verification
    is the last operator; the reference's task types are in the JSON."""
    from yirage_b200 import speculative
    shape = llama.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                             num_attention_heads=8, num_key_value_heads=2, vocab_size=2048)
    w = llama.init_weights(shape, "cpu", 0)
    tokens = torch.zeros(2, 128, dtype=torch.int64)
    cfg = speculative.spec_decode_class("promptlookup", ngram_size=3, spec_length=5)
    ypk, _ = llama.build_decode_kernel(
        shape, w, tokens=tokens, prompt_lengths=torch.tensor([5, 7], dtype=torch.int32),
        max_num_batched_requests=2, max_num_batched_tokens=8, max_num_pages=8, page_size=64,
        compile=False, spec_decode_config=cfg)
    g = ypk.lower(148)
    kinds = [o.kind for o in g.ops]
    assert kinds[:3] == ["ngram_partial", "ngram_global", "embed"] and kinds[-1] == "verify"
    glob = [t for t in g.tasks if t.type == N.TASK_NGRAM_GLOBAL]
    emb = [t for t in g.tasks if t.type == N.TASK_EMBED]
    assert len(glob) == 1 and all(e.ptr[0][0] is glob[0].ptr[1][0] for e in emb), \
        "the embedding reads the ids the draft operator writes"
    parts = [t for t in g.tasks if t.type == N.TASK_NGRAM_PARTIAL]
    assert [t.iarg[0] for t in parts] == list(range(parts[0].iarg[1])) and parts[0].iarg[2] == 3
    ver = [t for t in g.tasks if t.type == N.TASK_VERIFY]
    assert len(ver) == 1 and ver[0].iarg[0] == 5 and ver[0] is g.tasks[-1]
    counts = lowering.simulate(g, iterations=3)
    assert set(counts) == {3}
    doc = json.loads(lowering.to_json(g))
    assert {112, 113, 114} <= {t["task_type"] for t in doc["all_tasks"]}
    ypk.compile(dry_run=True)          # the native library checks the new task kinds
    ypk.finalize()


def test_mixture_of_experts_graph_lowers_and_validates(native_lib):
    """Qwen3-MoE layer (demo/qwen3/demo_30B_A3B.py:564-645): router, top-k routing, expert
    projections as LINEAR tasks per (active slot, row slab) whose weights are picked at run time,
    activation, weighted sum.  One token's experts must be able to fill the machine."""
    shape = llama.LlamaShape(hidden_size=256, intermediate_size=128, num_hidden_layers=2,
                             num_attention_heads=2, num_key_value_heads=1, vocab_size=512,
                             num_experts=16, experts_per_token=4)
    w = llama.init_weights(shape, "cpu", 0)
    assert w["layers"][0]["w13"].shape == (16, 256, 256) and w["layers"][0]["w2"].shape == (16, 256, 128)
    tokens = torch.zeros(2, 64, dtype=torch.int64)
    ypk, _ = llama.build_decode_kernel(
        shape, w, tokens=tokens, prompt_lengths=torch.tensor([5, 7], dtype=torch.int32),
        max_num_batched_requests=2, max_num_batched_tokens=8, max_num_pages=2, page_size=64,
        compile=False)
    g = ypk.lower(148)
    kinds = [o.kind for o in g.ops]
    i = kinds.index("moe_topk")
    assert kinds[i - 2:i + 5] == ["rmsnorm", "linear", "moe_topk", "moe_linear", "moe_silu_mul",
                                  "moe_linear", "moe_combine"]
    w13 = [t for t in g.tasks if t.type == N.TASK_LINEAR and t.flags & N.F_MOE and t.op_id == i + 1]
    slots = sorted({t.iarg[10] for t in w13})
    assert slots == list(range(16)), "min(experts, max_tokens * experts per token) active slots"
    first = [t for t in w13 if t.iarg[10] < 4]          # the slots one token uses
    assert len({t.worker for t in first}) == len(first) >= 32
    rows = sorted((t.iarg[1], t.iarg[2]) for t in w13 if t.iarg[10] == 0)
    assert rows[0][0] == 0 and sum(n for _, n in rows) == 256 and all(t.iarg[12] == 256 for t in w13)
    assert all(t.ptr[2][1] == t.iarg[10] * 8 * 256 * 2 for t in w13), "one [max_tokens, rows] block per slot"
    assert set(lowering.simulate(g, iterations=2)) == {2}
    doc = json.loads(lowering.to_json(g))
    assert {254, 255, 260, 261} <= {t["task_type"] for t in doc["all_tasks"]}
    ypk.compile(dry_run=True)
    ypk.finalize()


def test_norm_between_two_linears_is_carried_in_wide_graphs(monkeypatch):
    """Graphs of more than 8 tokens: linear(+residual) -> rmsnorm -> linear loses the RMSNORM
    operator; the producer writes the scaled rows and the sums of squares per row block, the
    consumer applies the RMS factor (reference: a separate norm task per layer half,
    demo/llama3/demo.py:402-470)."""
    def wide(layers=2):
        shape = llama.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=layers,
                                 num_attention_heads=8, num_key_value_heads=2, vocab_size=2048)
        w = llama.init_weights(shape, "cpu", 0)
        return llama.build_decode_kernel(
            shape, w, tokens=torch.zeros(2, 128, dtype=torch.int64),
            prompt_lengths=torch.tensor([5, 7], dtype=torch.int32), max_num_batched_requests=2,
            max_num_batched_tokens=64, max_num_pages=8, page_size=64, compile=False)[0]

    monkeypatch.delenv("YPK_TENSOR_CORE", raising=False)
    ypk = wide()
    g = ypk.lower(148)
    kinds = [o.kind for o in g.ops]
    assert kinds.count("rmsnorm") == 1            # only the one behind the embedding is left
    prods = [i for i, o in enumerate(g.ops) if o.flags & N.F_NORM_OUT]
    cons = [i for i, o in enumerate(g.ops) if o.flags & N.F_NORM_PRE]
    assert len(prods) == len(cons) == 4 and all(c == p + 1 for p, c in zip(prods, cons))
    for p, c in zip(prods, cons):
        po, co = g.ops[p], g.ops[c]
        assert po.flags & N.F_RESIDUAL and co.t["x"] is po.t["norm_out"] and co.t["ss_in"] is po.t["ss_out"]
        pt = [ts for ts in g.tasks if ts.op_id == p]
        ct = [ts for ts in g.tasks if ts.op_id == c]
        nblk = po.attrs["ss_nblk"]
        assert {ts.iarg[12] & 0xffff for ts in pt} == set(range(nblk))
        assert all(ts.iarg[12] >> 16 == 64 and ts.ptr_aux[0] is po.t["norm_out"] and
                   ts.ptr[3][0] is po.t["norm_out_w"] and ts.ptr[6][0] is po.t["ss_out"] for ts in pt)
        assert all(ts.iarg[12] == (nblk | (64 << 16)) and ts.ptr[3][0] is po.t["ss_out"] for ts in ct)
        # the consumer waits for the producer
        assert all(ts.dep_event == pt[0].trig_event and ts.dep_count == len(pt) for ts in ct)
    assert set(lowering.simulate(g, 2)) == {2}
    ypk.compile(dry_run=True)                      # the native validation accepts the operands

    # the GEMV passes have no such form: with the tensor cores switched off the norm stays
    monkeypatch.setenv("YPK_TENSOR_CORE", "never")
    g2 = wide().lower(148)
    assert [o.kind for o in g2.ops].count("rmsnorm") == 5
    assert not any(o.flags & (N.F_NORM_OUT | N.F_NORM_PRE) for o in g2.ops)



def _meta_llama3_8b_weights(shape):
    """Weights of the right shapes on the meta device: lowering looks at shapes only."""
    h, f, d = shape.hidden_size, shape.intermediate_size, shape.head_dim
    hq, hkv = shape.num_attention_heads, shape.num_key_value_heads
    e = lambda r, c: torch.empty(r, c, dtype=torch.bfloat16, device="meta")
    v = lambda n: torch.empty(n, dtype=torch.bfloat16, device="meta")
    w = {"embed": e(shape.vocab_size, h), "layers": [], "final_norm": v(h), "lm_head": e(shape.vocab_size, h)}
    for _ in range(shape.num_hidden_layers):
        w["layers"].append({"input_norm": v(h), "q": e(hq * d, h), "k": e(hkv * d, h), "v": e(hkv * d, h),
                            "o": e(h, hq * d), "post_norm": v(h), "gate": e(f, h), "up": e(f, h),
                            "down": e(h, f)})
    return w


def test_llama3_8b_rows_are_levelled_per_operator_and_attention_workers_get_less():
    """Every operator of a graph of at most 8 tokens waits for all tasks of its predecessor, so
    what counts is the largest slab of each operator: slabs differ by one granule at most,
    except behind attention, where the workers that ran an attention task get fewer rows.  No
    task is made for a split of the KV sequence that the context bound rules out."""
    shape = llama.LlamaShape.llama3_8b()
    shape.num_hidden_layers = 2
    ypk, _ = llama.build_decode_kernel(
        shape, _meta_llama3_8b_weights(shape), tokens=torch.zeros(1, 564, dtype=torch.int64, device="meta"),
        prompt_lengths=torch.zeros(1, dtype=torch.int32, device="meta"), max_num_batched_requests=1,
        max_num_batched_tokens=8, max_num_pages=9, page_size=64, compile=False)
    g = ypk.lower(148)
    kinds = [o.kind for o in g.ops]
    att = kinds.index("attention")
    att_tasks = [ts for ts in g.tasks if ts.op_id == att]
    # 564 tokens = 9 tiles of 64: at most ceil(9 / 4) = 3 splits are ever active
    assert len(att_tasks) == shape.num_key_value_heads * 3 and {ts.iarg[3] for ts in att_tasks} == {3}
    for oi, op in enumerate(g.ops):
        if op.kind != "linear":
            continue
        rows = [0] * 148
        for ts in g.tasks:
            if ts.op_id == oi:
                rows[ts.worker] += ts.iarg[2]
        gran = 4 if op.flags & N.F_SILU_MUL else 2
        if kinds[oi - 1] == "attention":
            att_workers = {ts.worker for ts in g.tasks if ts.op_id == oi - 1}
            others = [r for w_, r in enumerate(rows) if w_ not in att_workers]
            late = [rows[w_] for w_ in att_workers]
            assert max(others) - min(others) <= gran and max(late) < min(others)
        else:
            assert max(rows) - min(rows) <= gran, (oi, min(rows), max(rows))
    assert set(lowering.simulate(g, 2)) == {2}


def test_norm_with_two_readers_or_under_tensor_parallelism_is_not_carried():
    """The carried form needs the normalised rows to have exactly one reader, a LINEAR: the
    mixture-of-experts layer reads them twice (router and experts), and under tensor
    parallelism an all-reduce sits between the producing LINEAR and the norm."""
    moe = llama.LlamaShape(hidden_size=256, intermediate_size=128, num_hidden_layers=2,
                           num_attention_heads=2, num_key_value_heads=1, vocab_size=512,
                           qk_norm=True, num_experts=16, experts_per_token=4)
    w = llama.init_weights(moe, "cpu", 0)
    ypk = llama.build_decode_kernel(
        moe, w, tokens=torch.zeros(2, 64, dtype=torch.int64), prompt_lengths=torch.tensor([5, 7], dtype=torch.int32),
        max_num_batched_requests=2, max_num_batched_tokens=16, max_num_pages=4, page_size=64, compile=False)[0]
    g = ypk.lower(148)
    for i, op in enumerate(g.ops):
        if op.flags & N.F_NORM_OUT:
            nxt = g.ops[i + 1]
            assert nxt.kind == "linear" and nxt.flags & N.F_NORM_PRE and nxt.t["x"] is op.t["norm_out"]
            readers = [j for j, o in enumerate(g.ops)
                       if any(t is op.t["norm_out"] for _, t in lowering._op_inputs(o))]
            assert readers == [i + 1]
    # the post-attention norm of a mixture-of-experts layer feeds the router and the experts
    assert [o.kind for o in g.ops].count("rmsnorm") >= moe.num_hidden_layers
    assert set(lowering.simulate(g, 2)) == {2}

    shape = llama.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                             num_attention_heads=8, num_key_value_heads=2, vocab_size=2048)
    tp = llama.build_decode_kernel(
        shape, llama.init_weights(shape, "cpu", 0, world_size=2, rank=0),
        tokens=torch.zeros(2, 64, dtype=torch.int64), prompt_lengths=torch.tensor([5, 7], dtype=torch.int32),
        max_num_batched_requests=2, max_num_batched_tokens=64, max_num_pages=4, page_size=64,
        world_size=2, rank=0, compile=False)[0]
    g2 = tp.lower(148)
    assert "allreduce" in [o.kind for o in g2.ops]
    assert not any(o.flags & (N.F_NORM_OUT | N.F_NORM_PRE) for o in g2.ops)
