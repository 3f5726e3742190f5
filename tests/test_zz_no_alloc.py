"""ypk_argmax_noalloc - the sampling entry point for hosts that cannot let a library
allocate device memory - against the existing graph path (ARGMAX_PARTIAL + ARGMAX_REDUCE
tasks with runtime-allocated chunk buffers), through the C ABI, on two calls in a row.

Collected last on purpose: if it fails, a run that stops at the first failure has already
run every other test.  It does not depend on them: the first call on a device sets the
entry point up by itself."""
import ctypes as C

import pytest
import torch

from tests.util import onepass_kernel, randn
from yirage_b200 import _native as N

pytestmark = pytest.mark.gpu


def graph_argmax(logits, batch, parts=128):
    MT, V = logits.shape
    ypk = onepass_kernel(MT)
    pv = ypk.new_tensor(dims=(MT, parts), name="part_val")
    import yirage_b200 as yr
    pi = ypk.new_tensor(dims=(MT, parts), dtype=yr.int64, name="part_idx")
    out = torch.full((MT, 1), -1, dtype=torch.int64, device="cuda")
    ypk.argmax_partial_layer(ypk.attach_input(logits, "logits"), (pv, pi), (parts, 1, 1), (128, 1, 1))
    ypk.argmax_reduce_layer((pv, pi), ypk.attach_input(out, "out"), (1, 1, 1), (128, 1, 1))
    ypk.compile()
    ypk(batch=batch)
    torch.cuda.synchronize()
    ypk.finalize()
    return out[:batch, 0].clone()


def noalloc_argmax(logits, batch, vocab):
    lib = N.load()
    out = torch.full((logits.shape[0],), -1, dtype=torch.int64, device="cuda")
    rc = lib.ypk_argmax_noalloc(C.c_void_p(logits.data_ptr()), batch, vocab, logits.stride(0),
                                C.c_void_p(out.data_ptr()),
                                C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.ypk_last_error(None)
    torch.cuda.synchronize()
    return out[:batch].clone()


def test_noalloc_argmax_matches_graph_path_twice_in_a_row():
    MT, V = 16, 128 * 1008          # the padded Llama-3 vocabulary: 128 chunks of 1008
    for call, seed in enumerate((101, 202)):
        logits = randn((MT, V), seed)
        logits[1, V - 1] = 90.0                    # last column
        logits[2, 5] = logits[2, 70000] = 80.0     # tie across chunks -> lowest index
        batch = 16 if call == 0 else 5             # the second call reuses the scratch as is
        want = graph_argmax(logits, batch)
        got = noalloc_argmax(logits, batch, V)
        assert torch.equal(got, want), f"call {call}: {got.tolist()} vs {want.tolist()}"
        assert got[1].item() == V - 1 and got[2].item() == 5


def test_noalloc_argmax_ragged_vocabulary_and_limits():
    lib = N.load()
    logits = randn((4, 3000), 7)                   # 3000 is not a multiple of 128 chunks
    got = noalloc_argmax(logits, 4, 3000)
    assert got.tolist() == logits.float().argmax(dim=-1).tolist()
    # beyond the built-in scratch: refused with a message, nothing launched
    big = torch.zeros(65, 256, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(65, dtype=torch.int64, device="cuda")
    rc = lib.ypk_argmax_noalloc(C.c_void_p(big.data_ptr()), 65, 256, 256, C.c_void_p(out.data_ptr()), None)
    assert rc == N.ERR_UNSUPPORTED
    assert b"outside 1..64" in lib.ypk_last_error(None)
