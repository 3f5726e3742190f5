"""Paged GQA attention task against the CPU oracle: decode (one new token) and chunked
prefill (several new tokens), ragged sequence lengths around page and tile boundaries,
split-KV on and off, RoPE fused, new K/V written to the right page slots."""
import pytest
import torch

import yirage_b200 as yr
from oracle import decode_oracle as O
from tests.util import assert_close, onepass_kernel, randn

pytestmark = pytest.mark.gpu

D = 128


def run_attention(seq_lens, new_tokens, *, hq=8, hkv=2, page_size=64, max_seq=None, seed=0,
                  theta=500000.0):
    R = len(seq_lens)
    G = hq // hkv
    MT = max(8, sum(new_tokens))
    pages_per = [(s + page_size - 1) // page_size for s in seq_lens]
    max_pages = sum(pages_per) + 3
    max_seq = max_seq or max(seq_lens) + 1
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(max_pages, generator=g).tolist()      # seeded random page order
    qo, kvp, idx, last = [0], [0], [], []
    for r in range(R):
        qo.append(qo[-1] + new_tokens[r])
        idx += perm[kvp[-1]:kvp[-1] + pages_per[r]]
        kvp.append(kvp[-1] + pages_per[r])
        last.append((seq_lens[r] - 1) % page_size + 1)
    i32 = dict(dtype=torch.int32, device="cuda")
    meta = {
        "qo_indptr_buffer": torch.tensor(qo, **i32),
        "paged_kv_indptr_buffer": torch.tensor(kvp, **i32),
        "paged_kv_indices_buffer": torch.tensor(idx + [0] * (max_pages - len(idx)), **i32),
        "paged_kv_last_page_len_buffer": torch.tensor(last, **i32),
    }
    qkv = randn((MT, hkv * (G + 2) * D), seed + 1)
    kc = randn((max_pages, page_size, hkv, D), seed + 2)
    vc = randn((max_pages, page_size, hkv, D), seed + 3)
    cos, sin = O.rope_tables(D, theta, max(max_seq, 64))
    cos, sin = cos.cuda(), sin.cuda()
    out = torch.zeros(MT, hq * D, dtype=torch.bfloat16, device="cuda")
    kc0, vc0 = kc.clone().cpu(), vc.clone().cpu()

    ypk = onepass_kernel(MT, meta, max_requests=R, max_pages=max_pages, page_size=page_size,
                         max_seq_length=max_seq)
    ypk.paged_attention_layer(
        ypk.attach_input(qkv, "qkv"), ypk.attach_input(kc, "kc"), ypk.attach_input(vc, "vc"),
        None, None, ypk.attach_input(cos, "cos"), ypk.attach_input(sin, "sin"),
        ypk.attach_input(out, "out"), (R, hkv, 1), (128, 1, 1))
    ypk.compile()
    ypk(batch=qo[-1])
    torch.cuda.synchronize()
    nsplit = ypk.lower().tasks[0].iarg[3]

    # oracle on CPU copies
    qkv_c = qkv.cpu().float().view(MT, hkv, G + 2, D)
    kref, vref = kc0.clone(), vc0.clone()
    for r in range(R):
        a, b = qo[r], qo[r + 1]
        if a == b:
            continue
        q = qkv_c[a:b, :, :G].reshape(b - a, hq, D)
        k = qkv_c[a:b, :, G]
        v = qkv_c[a:b, :, G + 1]
        want = O.paged_attention_step(q, k, v, kref, vref, idx[kvp[r]:kvp[r + 1]], seq_lens[r],
                                      page_size, hq, hkv, cos.cpu(), sin.cpu(), rounding="bf16")
        assert_close(out[a:b].view(b - a, hq, D), want, f"request {r} (len {seq_lens[r]})")
    # new V rows land bit-exactly in their slots, new K within tolerance, nothing else moves
    assert torch.equal(vc.cpu(), vref), "V cache: paged indexing of the append is wrong"
    changed = (kc.cpu() != kc0)
    should = (kref != kc0)
    assert not (changed & ~should).any(), "K cache written outside the new-token slots"
    assert_close(kc.cpu(), kref, "K cache after append")
    ypk.finalize()
    return nsplit


def test_decode_one_token_ragged_lengths():
    # lengths straddle tile (64) and half-tile (32) boundaries; last page exactly full
    run_attention([1, 33, 64, 65, 128, 191], [1, 1, 1, 1, 1, 1], hq=8, hkv=2)


def test_decode_split_kv_combine():
    # one request, long context: the splits of a head land on different CTAs
    nsplit = run_attention([1000], [1], hq=8, hkv=2, max_seq=1024)
    assert nsplit > 1


def test_chunked_prefill_causal_window():
    run_attention([8, 70, 5], [8, 6, 5], hq=8, hkv=2, seed=4)


def test_gqa_group_of_eight_heads():
    run_attention([200, 90], [1, 3], hq=16, hkv=2, seed=6)


def test_page_size_larger_than_tile():
    run_attention([300, 129], [1, 1], hq=4, hkv=1, page_size=256, seed=8)


def test_config3_shape_reduced_context():
    # BASELINE config 3 layout (batch 8, 32 q / 8 kv heads, 64-token pages, theta 5e5) at a
    # context the CPU oracle finishes quickly
    run_attention([513] * 8, [1] * 8, hq=32, hkv=8, seed=2)
