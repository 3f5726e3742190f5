"""Host side of tensor parallelism on CPU: two gloo ranks lower the sharded graph, validate
it on host-only handles, exchange arena handles and import each other's."""
import os
import socket

import pytest
import torch


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, port, ret, handoff):
    import torch.distributed as dist
    from yirage_b200 import _native as N
    from yirage_b200 import llama, lowering
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    shape = llama.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                             num_attention_heads=8, num_key_value_heads=2, vocab_size=2048)
    w = llama.init_weights(shape, "cpu", 0, world_size=2, rank=rank)
    tokens = torch.zeros(2, 64, dtype=torch.int64)
    plen = torch.tensor([5, 7], dtype=torch.int32)
    ypk, _ = llama.build_decode_kernel(shape, w, tokens=tokens, prompt_lengths=plen,
                                       max_num_batched_requests=2, max_num_batched_tokens=8,
                                       max_num_pages=4, page_size=64, world_size=2, rank=rank,
                                       compile=False, handoff=handoff)
    g = ypk.lower(148)
    kinds = [o.kind for o in g.ops]
    assert kinds.count("allreduce") == 2 * shape.num_hidden_layers
    assert set(lowering.simulate(g, 2)) == {2}
    ar = [t for t in g.tasks if t.type == N.TASK_ALLREDUCE]
    o_proj = [t for t in g.tasks if t.op_id == 3][0]
    if handoff == "event":
        # the buffer half is the parity of the running all-reduce number, derived on the device
        # from (index in the iteration, all-reduces per iteration)
        nar = 2 * shape.num_hidden_layers
        assert {t.iarg[6] for t in ar} == set(range(nar)) and {t.iarg[10] for t in ar} == {nar}
        assert sorted(t.iarg[7] for t in ar) == list(range(len(ar))), "one counter per tile"
    else:
        # flagged words: the row-split projections push their partial sums to every rank, the
        # all-reduce tasks poll them (no event in or out) and pass the sum on the same way
        assert o_proj.flags & N.F_LL_PUSH and o_proj.flags & N.F_LL_OUT and o_proj.trig_event == -1
        assert all(t.flags & N.F_LL_IN and t.flags & N.F_LL_OUT for t in ar)
        assert all(t.dep_event == -1 and t.trig_event == -1 for t in ar)
        assert all(t.flagged_deps == [o.flagged_out] for t, o in [(ar[0], o_proj)])
        gate_up = [t for t in g.tasks if t.op_id == 5][0]
        assert gate_up.flags & N.F_LL_IN and gate_up.flagged_deps == [ar[0].flagged_out]
    assert all(t.iarg[8] == 2 and t.iarg[9] == rank for t in ar)
    # the residual goes in on rank 0 only
    assert bool(o_proj.flags & N.F_RESIDUAL) == (rank == 0)
    # host-only handles: symmetric allocation, validation, handle exchange over gloo
    ypk.compile(dry_run=True)
    with pytest.raises(N.YpkError):
        ypk._handle.comm_import(1 - rank, b"\0" * 64)     # already imported by compile()
    offs = {t.name: ypk._handle.tensor_ptr(t.guid)[0] - ypk._handle.tensor_ptr(g.internal[-1].guid)[0]
            for t in g.internal if t.kind == "nvshmem"}
    gathered = [None, None]
    dist.all_gather_object(gathered, offs)
    assert gathered[0] == gathered[1], "symmetric tensors must sit at the same arena offsets"
    ret[rank] = True
    ypk.finalize()
    dist.destroy_process_group()


@pytest.mark.parametrize("handoff", ["event", "ll"])
def test_two_cpu_ranks_build_validate_and_connect(native_lib, handoff):
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(_free_port(), ret, handoff), nprocs=2, join=True)
    assert ret.get(0) and ret.get(1)


def test_allreduce_needs_a_process_group():
    from yirage_b200 import tensor_parallel
    with pytest.raises(RuntimeError, match="torch.distributed"):
        tensor_parallel.exchange_handles(b"x", 2, 0)
