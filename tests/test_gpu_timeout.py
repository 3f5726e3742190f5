"""A device-side wait that runs out ends the launch with YPK_ERR_TIMEOUT and a record of who
gave up; the handle can be reset and used again.  Nothing faults or hangs: the wait is a
bounded poll of a flagged word that no task writes, with a budget of 50 ms."""
import ctypes as C

import pytest
import torch

from yirage_b200 import _native as N

pytestmark = pytest.mark.gpu

K, ROWS, MT = 512, 64, 8


def _linear(flags=0, ll_slot=None, tag=0):
    t = N.Task()
    t.type, t.flags = N.TASK_LINEAR, flags
    t.dep_event, t.dep_count, t.trig_event = -1, 0, 0
    t.ptr[0], t.ptr[1], t.ptr[2] = N.ref(0), N.ref(1), N.ref(2)
    if ll_slot is not None:
        t.ptr[5] = N.ref(ll_slot)
        t.iarg[10] = tag
    for i, v in enumerate([K, 0, ROWS, K, K, ROWS, 0, 0]):
        t.iarg[i] = v
    return t


def test_wait_that_runs_out_reports_and_the_handle_recovers(native_lib):
    torch.cuda.set_device(0)
    cfg = N.Config()
    cfg.device, cfg.world_size, cfg.rank, cfg.mode = 0, 1, 0, 0
    cfg.max_num_batched_tokens, cfg.max_num_batched_requests = MT, 1
    cfg.page_size, cfg.max_num_pages = 64, 1
    cfg.wait_budget_ns = 50_000_000
    h = N.Handle(cfg)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(MT, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(ROWS, K, generator=g) * 0.02).to(torch.bfloat16).cuda()
    out = torch.zeros(MT, ROWS, dtype=torch.bfloat16, device="cuda")
    h.bind(0, "x", x.data_ptr(), x.numel() * 2)
    h.bind(1, "w", w.data_ptr(), w.numel() * 2)
    h.bind(2, "out", out.data_ptr(), out.numel() * 2)
    h.alloc(3, "flagged_x", MT * K * 4)           # zero-filled: no word carries a current tag
    # the task takes x as flagged words under tag id 7, which no task of the graph writes
    h.load_graph([_linear(N.F_LL_IN, ll_slot=3, tag=7)], 1, [0], [0, 1])
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    with pytest.raises(N.YpkError) as e:
        h.launch(torch.cuda.current_stream().cuda_stream, 0, 4)
    ev1.record()
    torch.cuda.synchronize()
    assert e.value.code == N.ERR_TIMEOUT
    st = h.status()
    assert st.error == N.ERR_TIMEOUT and st.fail_task == 0 and st.fail_event == -6
    assert 0 <= st.fail_worker < 148
    assert 40.0 <= ev0.elapsed_time(ev1) < 1500.0, "the wait should give up after its 50 ms budget"
    assert torch.all(out == 0), "a task whose input never came must not write"
    # a failed handle refuses to launch until it is reset
    with pytest.raises(N.YpkError) as e2:
        h.launch(torch.cuda.current_stream().cuda_stream, 0, 4)
    assert e2.value.code == N.ERR_STATE
    h.reset()
    assert h.status().error == 0
    # the same handle, a graph that can run: correct result
    h.load_graph([_linear()], 1, [0], [0, 1])
    h.launch(torch.cuda.current_stream().cuda_stream, 0, 4)
    torch.cuda.synchronize()
    want = (x[:4].float() @ w.float().t()).cpu()
    got = out[:4].float().cpu()
    assert torch.allclose(got, want, atol=2e-2, rtol=1e-2)
    assert torch.all(out[4:] == 0)
    h.close()
