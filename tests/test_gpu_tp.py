"""Tensor-parallel decode on 2 GPUs: one process per GPU, NCCL only for the bootstrap, the
all-reduce after each row-split projection done inside the persistent kernel over peer
memory.  Needs two devices; on a single-GPU box the test is skipped."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

WORLD = 2


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, port, prompt_lens, max_seq, ret, handoff):
    import torch.distributed as dist
    from tests.util import oracle_weights, replay_against_oracle
    from yirage_b200 import llama
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=torch.device("cuda", rank))
    shape = llama.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                             num_attention_heads=8, num_key_value_heads=2, vocab_size=3000)
    dev = torch.device("cuda", rank)
    w = llama.init_weights(shape, dev, 3, world_size=WORLD, rank=rank)
    g = torch.Generator().manual_seed(3)
    R = len(prompt_lens)
    tokens = torch.zeros(R, max_seq, dtype=torch.int64)
    for r, n in enumerate(prompt_lens):
        tokens[r, :n] = torch.randint(0, shape.vocab_size, (n,), generator=g)
    tokens = tokens.to(dev)
    plen = torch.tensor(prompt_lens, dtype=torch.int32, device=dev)
    ypk, st = llama.build_decode_kernel(
        shape, w, tokens=tokens, prompt_lengths=plen, max_num_batched_requests=2,
        max_num_batched_tokens=8, max_num_pages=4, page_size=64, world_size=WORLD, rank=rank,
        handoff=handoff)
    dist.barrier()
    ypk()
    torch.cuda.synchronize()
    status = ypk.status()
    assert status.error == 0 and status.finished == 1
    # every rank must have sampled the same tokens, bit for bit
    mine = tokens.clone()
    both = [torch.empty_like(mine) for _ in range(WORLD)]
    dist.all_gather(both, mine)
    assert torch.equal(both[0], both[1]), "ranks disagree on the generated tokens"
    if rank == 0:
        full = llama.init_weights(shape, dev, 3)       # the unsharded model
        iters, bs, last_logits, exact, total = replay_against_oracle(
            shape, oracle_weights(shape, full), tokens.cpu(), prompt_lens, max_seq=max_seq,
            max_requests=2, max_tokens=8, max_pages=4, page_size=64)
        assert status.iterations == iters
        assert st["meta"]["step"].cpu().tolist() == bs.step
        assert exact >= 0.75 * total
        ret["ok"] = (iters, exact, total)
    dist.barrier()
    ypk.finalize()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < WORLD, reason="needs 2 GPUs")
@pytest.mark.parametrize("handoff", ["ll", "event"])
def test_tp2_decode_matches_oracle_and_ranks_agree(handoff):
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(_free_port(), [9, 14, 5], 30, ret, handoff), nprocs=WORLD, join=True)
    assert "ok" in ret, "rank 0 did not finish its checks"


def _rank_main_pair(rank, port, prompt_lens, max_seq, ret):
    """Prompts on a 64-token graph, decoding on an 8-token graph, both tensor parallel."""
    import torch.distributed as dist
    from tests.util import oracle_weights, replay_against_oracle
    from yirage_b200 import llama
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=torch.device("cuda", rank))
    shape = llama.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                             num_attention_heads=8, num_key_value_heads=2, vocab_size=3000)
    dev = torch.device("cuda", rank)
    w = llama.init_weights(shape, dev, 3, world_size=WORLD, rank=rank)
    g = torch.Generator().manual_seed(3)
    tokens = torch.zeros(len(prompt_lens), max_seq, dtype=torch.int64)
    for r, n in enumerate(prompt_lens):
        tokens[r, :n] = torch.randint(0, shape.vocab_size, (n,), generator=g)
    tokens = tokens.to(dev)
    plen = torch.tensor(prompt_lens, dtype=torch.int32, device=dev)
    pair = llama.build_prefill_decode_pair(
        shape, w, tokens=tokens, prompt_lengths=plen, max_num_batched_requests=2, max_num_pages=6,
        page_size=64, prefill_tokens=64, decode_tokens=8, world_size=WORLD, rank=rank)
    dist.barrier()
    it_p, it_d = pair.run()
    torch.cuda.synchronize()
    sd = pair.decode.status()
    assert sd.error == 0 and sd.finished == 1 and pair.prefill.status().error == 0
    both = [torch.empty_like(tokens) for _ in range(WORLD)]
    dist.all_gather(both, tokens.clone())
    assert torch.equal(both[0], both[1]), "ranks disagree on the generated tokens"
    if rank == 0:
        full = llama.init_weights(shape, dev, 3)
        iters, bs, _, exact, total = replay_against_oracle(
            shape, oracle_weights(shape, full), tokens.cpu(), prompt_lens, max_seq=max_seq,
            max_requests=2, max_tokens=64, max_pages=6, page_size=64, decode_tokens=8)
        assert it_p + it_d == iters and pair.state["meta"]["step"].cpu().tolist() == bs.step
        assert exact >= 0.75 * total
        ret["ok"] = (it_p, it_d, exact, total)
    dist.barrier()
    pair.finalize()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < WORLD, reason="needs 2 GPUs")
def test_tp2_prefill_graph_hands_over_to_decode_graph():
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main_pair, args=(_free_port(), [130, 20, 77], 150, ret), nprocs=WORLD, join=True)
    assert "ok" in ret, "rank 0 did not finish its checks"
    assert 0 < ret["ok"][0] < 10
