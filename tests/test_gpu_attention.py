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
                  theta=500000.0, qk_norm=False, eps=1e-6):
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
    qn = kn = qn_t = kn_t = None
    if qk_norm:
        qn, kn = randn((D,), seed + 4, 0.2, mean=1.0), randn((D,), seed + 5, 0.2, mean=1.0)
        qn_t, kn_t = ypk.attach_input(qn, "q_norm"), ypk.attach_input(kn, "k_norm")
        ypk.rms_norm_eps = eps
    ypk.paged_attention_layer(
        ypk.attach_input(qkv, "qkv"), ypk.attach_input(kc, "kc"), ypk.attach_input(vc, "vc"),
        qn_t, kn_t, ypk.attach_input(cos, "cos"), ypk.attach_input(sin, "sin"),
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
        norm = dict(q_norm_w=qn.cpu(), k_norm_w=kn.cpu(), qk_eps=eps) if qk_norm else {}
        want = O.paged_attention_step(q, k, v, kref, vref, idx[kvp[r]:kvp[r + 1]], seq_lens[r],
                                      page_size, hq, hkv, cos.cpu(), sin.cpu(), rounding="bf16", **norm)
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


def test_prefill_over_query_tiles():
    """More new tokens per request than one task takes: the request is spread over tasks of 8
    new tokens (4 with 8 q heads per kv head), each staging the earlier new tokens' k / v
    itself.  From an empty cache, on top of a cached context that ends inside a tile, with a
    short last tile, and next to a request that only decodes."""
    run_attention([50, 14], [50, 14], hq=8, hkv=2, seed=11)
    run_attention([300, 65], [63, 1], hq=8, hkv=2, seed=12, max_seq=320)
    run_attention([40], [40], hq=16, hkv=2, seed=13)          # tiles of 4 tokens
    run_attention([64, 200], [27, 37], hq=8, hkv=2, seed=14, qk_norm=True)


def test_gqa_group_of_eight_heads():
    run_attention([200, 90], [1, 3], hq=16, hkv=2, seed=6)


def test_page_size_larger_than_tile():
    run_attention([300, 129], [1, 1], hq=4, hkv=1, page_size=256, seed=8)


def test_config3_shape_reduced_context():
    # BASELINE config 3 layout (batch 8, 32 q / 8 kv heads, 64-token pages, theta 5e5) at a
    # context the CPU oracle finishes quickly
    run_attention([513] * 8, [1] * 8, hq=32, hkv=8, seed=2)


def test_config3_full_context_4096():
    """BASELINE config 3 as stated: batch 8, 32 q / 8 kv heads, KV length 4096 in 64-token pages
    in a seeded random page order, RoPE theta 5e5 on the new token at position 4096."""
    nsplit = run_attention([4097] * 8, [1] * 8, hq=32, hkv=8, seed=2, max_seq=4098)
    assert nsplit >= 2


def test_qk_norm_decode_and_prefill_chunks():
    """q/k RMSNorm inside attention (Qwen3): decode rows and multi-token chunks, page
    boundaries, split-KV."""
    run_attention([1, 64, 65, 200], [1, 1, 1, 1], hq=8, hkv=2, seed=10, qk_norm=True)
    run_attention([9, 70, 133], [8, 6, 5], hq=8, hkv=2, seed=11, qk_norm=True, eps=1e-5)
    run_attention([900], [1], hq=16, hkv=2, seed=12, qk_norm=True, max_seq=1024)


# ---- against outputs of the reference's own torch functions (tests/golden, written by
# ---- tests/golden/make_golden.py from tests/runtime_python/test_*paged_attention.py)
def _golden(name):
    import os
    return torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name))


def _run_fixture_case(qkv_rows, k_rows, v_rows, pages, seq_len, T, cos_tab, sin_tab, qw, kw, eps,
                      page_size=64, num_pages=16):
    """One request of the fixture layout (4 q heads, 1 kv head) through the attention task.
    Returns (out [T, 4, 128], K cache after the call [pages, page, 1, 128])."""
    MT = 8
    kc = torch.zeros(num_pages, page_size, 1, D, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    for p in range(seq_len):
        kc[int(pages[p // page_size]), p % page_size, 0] = k_rows[p]
        vc[int(pages[p // page_size]), p % page_size, 0] = v_rows[p]
    kc, vc = kc.cuda(), vc.cuda()
    npages = (seq_len + page_size - 1) // page_size
    i32 = dict(dtype=torch.int32, device="cuda")
    meta = {"qo_indptr_buffer": torch.tensor([0, T], **i32),
            "paged_kv_indptr_buffer": torch.tensor([0, npages], **i32),
            "paged_kv_indices_buffer": torch.tensor([int(p) for p in pages[:npages]] + [0] * (num_pages - npages), **i32),
            "paged_kv_last_page_len_buffer": torch.tensor([(seq_len - 1) % page_size + 1], **i32)}
    qkv = torch.zeros(MT, 6 * D, dtype=torch.bfloat16)
    qkv[:T] = qkv_rows.reshape(T, 6 * D)
    qkv = qkv.cuda()
    out = torch.zeros(MT, 4 * D, dtype=torch.bfloat16, device="cuda")
    ypk = onepass_kernel(MT, meta, max_requests=1, max_pages=num_pages, page_size=page_size,
                         max_seq_length=max(seq_len + 1, 64))
    qn_t = kn_t = None
    if qw is not None:
        qn_t = ypk.attach_input(qw.reshape(-1).cuda(), "q_norm")
        kn_t = ypk.attach_input(kw.reshape(-1).cuda(), "k_norm")
        ypk.rms_norm_eps = eps
    ypk.paged_attention_layer(
        ypk.attach_input(qkv, "qkv"), ypk.attach_input(kc, "kc"), ypk.attach_input(vc, "vc"),
        qn_t, kn_t, ypk.attach_input(cos_tab.cuda(), "cos"), ypk.attach_input(sin_tab.cuda(), "sin"),
        ypk.attach_input(out, "out"), (1, 1, 1), (128, 1, 1))
    ypk.compile()
    ypk(batch=T)
    torch.cuda.synchronize()
    res = out[:T].view(T, 4, D).cpu(), kc.cpu()
    ypk.finalize()
    return res


def _same_k(got, want, normed, what):
    """The K written to the page against the reference function's.  Rotation alone is three
    fp32 operations with the same rounding points on both sides: bit for bit.  With the
    RMSNorm in front the reciprocal square root and the order of the 128-term sum differ in
    the last fp32 bit, which can move a value across a bf16 rounding boundary: one bf16 step."""
    if not normed:
        assert torch.equal(got, want), f"{what}: appended K differs from the reference's"
        return
    g, w = got.float(), want.float()
    step = torch.maximum(w.abs(), torch.tensor(1e-30)).log2().floor().exp2() * 2.0 ** -7
    assert bool(((g - w).abs() <= step).all()), f"{what}: appended K more than one bf16 step off"
    assert float((g != w).float().mean()) < 0.05, f"{what}: too many K values differ"


def test_decode_matches_reference_torch_paged_attention():
    """torch_paged_attention (test_paged_attention.py:48-94) on the committed inputs: the
    appended K bit for bit, the output within tolerance; lengths 63/64/65, a full last page,
    a permuted page list, with and without q/k RMSNorm."""
    g = _golden("paged_attention_decode.pt")
    pages = g["pages"].tolist()
    for c in g["cases"]:
        L = c["seq_len"]
        cos = torch.zeros(max(L, 64), D, dtype=torch.bfloat16)
        sin = torch.zeros_like(cos)
        cos[L - 1], sin[L - 1] = c["cos_row"], c["sin_row"]
        qw, kw = (c["q_norm_w"], c["k_norm_w"]) if c["qk_norm"] else (None, None)
        out, kc = _run_fixture_case(c["qkv"][None], c["k_rows"], c["v_rows"], pages, L, 1, cos, sin,
                                    qw, kw, c["eps"])
        slot = kc[pages[(L - 1) // 64], (L - 1) % 64, 0]
        _same_k(slot, c["k_new_after"], c["qk_norm"], f"seq_len {L}")
        assert_close(out[0], c["out"][0], f"seq_len {L} qk_norm {c['qk_norm']}")


def test_chunks_match_reference_torch_multitoken_paged_attention():
    """torch_multitoken_paged_attention (test_multitoken_paged_attention.py:51-122): several new
    tokens, K updated in place in the page, causal among the new tokens."""
    g = _golden("paged_attention_multitoken.pt")
    for c in g["cases"]:
        T, L = c["num_tokens"], c["num_tokens"] + c["cached"]
        pages = c["pages"].tolist() + [0] * 16
        cos = torch.zeros(max(L + 1, 64), D, dtype=torch.bfloat16)
        sin = torch.zeros_like(cos)
        cos[:L + 1], sin[:L + 1] = c["cos"], c["sin"]
        qw, kw = (c["q_norm_w"], c["k_norm_w"]) if c["qk_norm"] else (None, None)
        out, kc = _run_fixture_case(c["qkv"], c["k_rows"], c["v_rows"], pages, L, T, cos, sin, qw, kw,
                                    c["eps"])
        got_rows = torch.stack([kc[pages[p // 64], p % 64, 0] for p in range(L)])
        assert torch.equal(got_rows[:c["cached"]], c["k_rows_after"][:c["cached"]]), "cached K rows moved"
        _same_k(got_rows[c["cached"]:], c["k_rows_after"][c["cached"]:], c["qk_norm"],
                f"cached {c['cached']} + {T}")
        assert_close(out, c["out"], f"cached {c['cached']} + {T} tokens qk_norm {c['qk_norm']}")
