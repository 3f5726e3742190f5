"""The CPU oracle against outputs of the reference's own PyTorch model code
(tests/golden/*.pt, written by tests/golden/make_golden.py from the reference tree)."""
import os

import pytest
import torch

from oracle import decode_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return torch.load(os.path.join(GOLD, name))


def bf16_ulps(a, b):
    """Largest difference in units of the bf16 spacing at the reference value."""
    a, b = a.float(), b.float()
    spacing = torch.maximum(b.abs(), torch.tensor(1e-30)).log2().floor().exp2() * 2.0 ** -7
    return float(((a - b).abs() / spacing).max())


@pytest.mark.parametrize("tag", ["eps1e-6", "eps1e-5"])
def test_rmsnorm_matches_reference_module(tag):
    g = load(f"rmsnorm_{tag}.pt")
    # the reference module works in bf16 throughout; the fp32 oracle rounded once must sit
    # within a couple of bf16 steps of it and inside the stated tolerance
    got = O.rmsnorm(g["x"], g["w"], g["eps"], rounding="bf16")
    assert bf16_ulps(got, g["y"]) <= 3.0
    assert O.within_tolerance(O.rmsnorm(g["x"], g["w"], g["eps"]), g["y"].float())[0]


def test_gated_mlp_matches_reference_module():
    g = load("gated_mlp.pt")
    got = O.gated_mlp(g["x"], g["gate"], g["up"], g["down"], rounding="bf16")
    assert O.within_tolerance(got, g["y"].float())[0]
    assert bf16_ulps(got, g["y"]) <= 4.0
    assert O.within_tolerance(O.gated_mlp(g["x"], g["gate"], g["up"], g["down"]), g["y"].float())[0]


def test_rope_tables_match_reference_rotary_embedding():
    g = load("rope_tables.pt")
    cos, sin = O.rope_tables(g["head_dim"], g["theta"], 4160)
    assert torch.equal(cos[g["positions"]], g["cos"])   # bit-exact bf16 tables
    assert torch.equal(sin[g["positions"]], g["sin"])


def test_decode_attention_matches_reference_sdpa():
    g = load("decode_attention.pt")
    q, k, v = g["q"][0].float(), g["k"].float(), g["v"].float()   # q [32,128]; k,v [ctx,8,128]
    out = torch.cat([O.attention_rows(q[h * 4:(h + 1) * 4], k[:, h], v[:, h]) for h in range(8)], 0)
    assert O.within_tolerance(out, g["out"][0].float())[0]


def test_prefill_attention_causal_window_matches_reference_sdpa():
    g = load("prefill_attention.pt")
    q, k, v = g["q"].float(), g["k"].float(), g["v"].float()      # q [5,32,128]
    T = q.shape[0]
    for h in range(8):
        qh = q[:, h * 4:(h + 1) * 4].reshape(T * 4, 128)
        vis = [t + 1 for t in range(T) for _ in range(4)]
        out = O.attention_rows(qh, k[:, h], v[:, h], vis).reshape(T, 4, 128)
        assert O.within_tolerance(out, g["out"][:, h * 4:(h + 1) * 4].float())[0]


def test_rope_application_matches_reference_test_function():
    """apply_rotary_pos_emb of the reference's kernel tests (test_paged_attention.py:18-34)
    on random cos/sin rows whose halves differ: same values after the one bf16 rounding."""
    g = load("rope_apply.pt")
    c, s = g["cos"][:, None, :], g["sin"][:, None, :]
    assert torch.equal(O.apply_rope(g["q"], c, s, "bf16").to(torch.bfloat16), g["q_out"])
    assert torch.equal(O.apply_rope(g["k"], c, s, "bf16").to(torch.bfloat16), g["k_out"])


def _scatter(rows, pages, page_size, num_pages):
    """Position-ordered rows [seq, d] -> a paged cache [pages, page_size, 1, d]."""
    cache = torch.zeros(num_pages, page_size, 1, rows.shape[-1], dtype=rows.dtype)
    for p in range(rows.shape[0]):
        cache[int(pages[p // page_size]), p % page_size, 0] = rows[p]
    return cache


def test_paged_attention_matches_reference_test_function():
    """torch_paged_attention (test_paged_attention.py:48-94): one new token against a cache
    in a permuted page order, lengths on either side of a page boundary and a last page that
    is exactly full; with the q/k RMSNorm of Qwen3 in three of the cases.  The rotated
    (normed) K that lands in the page is compared bit for bit, the output within tolerance
    (the reference function multiplies and normalises in bf16)."""
    g = load("paged_attention_decode.pt")
    PS, pages = g["page_size"], g["pages"].tolist()
    assert {c["seq_len"] for c in g["cases"]} >= {63, 64, 65, 128}
    for c in g["cases"]:
        L = c["seq_len"]
        kc = _scatter(c["k_rows"], pages, PS, 16)
        vc = _scatter(c["v_rows"], pages, PS, 16)
        qkv = c["qkv"].float()
        cos = torch.zeros(L, 128, dtype=torch.bfloat16)
        sin = torch.zeros(L, 128, dtype=torch.bfloat16)
        cos[L - 1], sin[L - 1] = c["cos_row"], c["sin_row"]
        norm = dict(q_norm_w=c["q_norm_w"], k_norm_w=c["k_norm_w"], qk_eps=c["eps"]) if c["qk_norm"] else {}
        out = O.paged_attention_step(qkv[None, :4], qkv[None, 4:5], qkv[None, 5:6], kc, vc,
                                     pages[:(L + PS - 1) // PS], L, PS, 4, 1, cos, sin, "bf16", **norm)
        slot = kc[pages[(L - 1) // PS], (L - 1) % PS, 0]
        assert torch.equal(slot, c["k_new_after"]), f"seq_len {L}: appended K differs"
        ok, max_abs, _ = O.within_tolerance(out[0], c["out"].float())
        assert ok, f"seq_len {L} qk_norm {c['qk_norm']}: max abs err {max_abs}"


def test_multitoken_paged_attention_matches_reference_test_function():
    """torch_multitoken_paged_attention (test_multitoken_paged_attention.py:51-122): several
    new tokens of one request, K updated in place in the page, causal among the new tokens."""
    g = load("paged_attention_multitoken.pt")
    PS = g["page_size"]
    for c in g["cases"]:
        T, cached = c["num_tokens"], c["cached"]
        L = T + cached
        pages = c["pages"].tolist()
        kc = _scatter(c["k_rows"], pages, PS, 16)
        vc = _scatter(c["v_rows"], pages, PS, 16)
        qkv = c["qkv"].float().view(T, 6, 128)
        norm = dict(q_norm_w=c["q_norm_w"], k_norm_w=c["k_norm_w"], qk_eps=c["eps"]) if c["qk_norm"] else {}
        out = O.paged_attention_step(qkv[:, :4], qkv[:, 4:5], qkv[:, 5:6], kc, vc, pages, L, PS, 4, 1,
                                     c["cos"], c["sin"], "bf16", **norm)
        want_k = _scatter(c["k_rows_after"], pages, PS, 16)
        assert torch.equal(kc, want_k), f"cached {cached} + {T}: K cache after the update differs"
        ok, max_abs, _ = O.within_tolerance(out, c["out"].float())
        assert ok, f"cached {cached} + {T} qk_norm {c['qk_norm']}: max abs err {max_abs}"


def test_decode_attention_with_qk_norm_matches_reference_test_function():
    """attention_decode (test_decoding_w_norm.py:55-72): RMSNorm of q and of the new k over the
    head dimension, then the rotation, contiguous cache."""
    g = load("decode_attention_qknorm.pt")
    for c in g["cases"]:
        L = c["valid_len"]
        kc, vc = c["k_cache"][None, :, None, :].clone(), c["v_cache"][None, :, None, :].clone()
        PS = kc.shape[1]
        cos = torch.zeros(L, 128, dtype=torch.bfloat16)
        sin = torch.zeros(L, 128, dtype=torch.bfloat16)
        cos[L - 1], sin[L - 1] = c["cos"], c["sin"]
        out = O.paged_attention_step(c["q"].float()[None], kc[0, L - 1:L, :, :].float(),
                                     vc[0, L - 1:L, :, :].float(), kc, vc, [0], L, PS, 4, 1, cos, sin,
                                     "bf16", q_norm_w=c["q_norm_w"], k_norm_w=c["k_norm_w"], qk_eps=c["eps"])
        assert torch.equal(kc[0, L - 1, 0], c["k_new_after"])
        assert O.within_tolerance(out[0], c["out"].float())[0]


def test_paged_attention_step_equals_contiguous_attention():
    """Paged indexing + in-place append against the contiguous formulation on the same data."""
    gen = torch.Generator().manual_seed(7)
    hq, hkv, d, page, L, T = 8, 2, 128, 64, 150, 3
    pages = [5, 1, 3]
    kc = torch.zeros(8, page, hkv, d, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kflat = torch.randn(L, hkv, d, generator=gen).to(torch.bfloat16)
    vflat = torch.randn(L, hkv, d, generator=gen).to(torch.bfloat16)
    for p in range(L - T):
        kc[pages[p // page], p % page] = kflat[p]
        vc[pages[p // page], p % page] = vflat[p]
    q = torch.randn(T, hq, d, generator=gen).to(torch.bfloat16).float()
    out = O.paged_attention_step(q, kflat[L - T:].float(), vflat[L - T:].float(), kc, vc, pages, L,
                                 page, hq, hkv, None, None, rounding=None)
    for h in range(hkv):
        vis = [L - T + t + 1 for t in range(T) for _ in range(4)]
        want = O.attention_rows(q[:, h * 4:(h + 1) * 4].reshape(T * 4, d), kflat[:, h], vflat[:, h], vis)
        assert torch.allclose(out[:, h * 4:(h + 1) * 4].reshape(T * 4, d), want, atol=1e-5)
    assert torch.equal(kc[pages[2], (L - 1) % page], kflat[L - 1])


def test_argmax_lowest_index_and_shuffle_rows():
    x = torch.tensor([[1.0, 3.0, 3.0, 2.0], [0.0, 0.0, 0.0, 0.0]])
    assert O.argmax_lowest(x).tolist() == [1, 0]
    a = torch.arange(8).view(4, 2)
    b = torch.arange(100, 104).view(2, 2)
    sh = O.shuffle_rows([a, b], 2)
    assert sh[:, 0].tolist() == [0, 2, 100, 4, 6, 102]


def test_batcher_model_chunks_prefill_and_recycles_pages():
    tokens = torch.zeros(3, 40, dtype=torch.int64)
    bs = O.BatchState(total_requests=3, max_requests=2, max_tokens=8, max_pages=2, page_size=64,
                      max_seq_length=12, eos=-1, tokens=tokens, prompt_len=[10, 3, 2])
    seen = []
    out = None
    while True:
        n = bs.prepare_next_batch(out)
        if n == 0:
            break
        seen.append((n, list(bs.request_ids), list(bs.kv_last_len[:2])))
        out = [7] * n
        assert len(seen) < 100
    # request 0 takes the whole first batch (8 of its 10 prompt tokens)
    assert seen[0][0] == 8 and seen[0][1] == [0, -1]
    # every request retires at max_seq_length - 1 tokens processed
    assert bs.step == [11, 11, 11]
    assert bs.tail - bs.head == 2, "all pages returned to the free queue"


def test_prompt_lookup_drafts_follow_the_reference_kernel():
    """find_ngram_partial / find_ngram_global (tasks/speculative_decoding/prompt_lookup.cuh:
    22-132) by hand: the history's last n-gram is searched in the history before it (earliest
    match), the drafts are the tokens after the match, -1 past the history's end or without
    a match; a history no longer than the n-gram gives no drafts."""
    #           0  1  2  3  4  5  6  7  8  9 10 11
    history = [5, 6, 7, 8, 5, 6, 7, 9, 1, 5, 6, 7]
    assert O.prompt_lookup(history, 11, 3, 4) == [8, 5, 6, 7]          # match at 0, not at 4
    assert O.prompt_lookup(history, 11, 3, 12)[:9] == [8, 5, 6, 7, 9, 1, 5, 6, 7]
    assert O.prompt_lookup(history, 11, 3, 12)[9:] == [-1, -1, -1]     # index > step
    assert O.prompt_lookup(history, 7, 2, 3) == [-1, -1, -1]           # (7, 9) never seen before
    assert O.prompt_lookup([5, 6, 7], 2, 3, 4) == [-1] * 4             # history == n-gram
    assert O.prompt_lookup([1, 2, 3, 1, 2, 3], 5, 3, 5) == [1, 2, 3, -1, -1]


def test_speculative_greedy_decoding_gives_the_tokens_of_plain_greedy_decoding():
    """target_verify_greedy (target_verify.cuh:20-60) accepts a draft only if it is the model's
    own arg-max, so the sequence is unchanged and only the iteration count drops."""
    g = torch.Generator().manual_seed(4)
    hidden, inter, hq, hkv, vocab = 64, 128, 4, 2, 50
    d = hidden // hq
    r = lambda *s: (torch.randn(*s, generator=g) * 0.2).to(torch.bfloat16)
    one = torch.ones(hidden, dtype=torch.bfloat16)
    layer = dict(input_norm=one, q=r(hq * d, hidden), k=r(hkv * d, hidden), v=r(hkv * d, hidden),
                 o=r(hidden, hq * d), post_norm=one, gate=r(inter, hidden), up=r(inter, hidden),
                 down=r(hidden, inter))
    w = O.LlamaWeights(embed=r(vocab, hidden), layers=[layer], final_norm=one, lm_head=r(vocab, hidden),
                       num_q_heads=hq, num_kv_heads=hkv, head_dim=d, eps=1e-5, rope_theta=10000.0)

    def run(spec):
        tokens = torch.zeros(2, 48, dtype=torch.int64)
        tokens[0, :5] = torch.tensor([3, 7, 11, 2, 9])
        tokens[1, :3] = torch.tensor([4, 4, 8])
        bs = O.BatchState(total_requests=2, max_requests=2, max_tokens=8, max_pages=4, page_size=64,
                          max_seq_length=48, eos=-1, tokens=tokens, prompt_len=[5, 3],
                          spec_length=spec, ngram_size=2)
        kc = [torch.zeros(4, 64, hkv, d, dtype=torch.bfloat16)]
        vc = [torch.zeros_like(kc[0])]
        cos, sin = O.rope_tables(d, 10000.0, 64)
        return O.generate(w, bs, kc, vc, cos, sin, rounding=None), tokens, bs

    it0, t0, _ = run(0)
    it3, t3, bs = run(3)
    assert torch.equal(t0, t3)
    assert it3 < it0, "some drafts must have been accepted on this seed"
    assert bs.step == [47, 47] and bs.tail - bs.head == 4


def test_moe_routing_is_softmax_then_topk_renormalised():
    """topk_softmax_task_impl (tasks/blackwell/topk_softmax_sm100.cuh:63-303) with renormalize =
    true: probabilities over all experts, the k largest in order, divided by their sum; equal
    probabilities go to the lower expert id."""
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(5, 32, generator=g)
    w, e = O.moe_topk_softmax(logits, 4)
    p = torch.softmax(logits, -1)
    tv, ti = p.topk(4)
    assert torch.equal(e, ti) and torch.allclose(w, tv / tv.sum(-1, keepdim=True))
    assert torch.allclose(w.sum(-1), torch.ones(5))
    w, e = O.moe_topk_softmax(torch.zeros(1, 8), 3)
    assert e.tolist() == [[0, 1, 2]] and torch.allclose(w, torch.full((1, 3), 1 / 3))


def test_moe_mlp_equals_a_dense_sum_over_the_selected_experts():
    g = torch.Generator().manual_seed(1)
    T, H, I, E, K = 3, 32, 16, 8, 2
    x, res = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g)
    gate_w = torch.randn(E, H, generator=g)
    w13, w2 = torch.randn(E, 2 * I, H, generator=g) * 0.2, torch.randn(E, H, I, generator=g) * 0.2
    got = O.moe_mlp(x, gate_w, w13, w2, K, res, rounding=None)
    wts, exps = O.moe_topk_softmax((x @ gate_w.t()).to(torch.bfloat16), K)
    want = res.clone()
    for t in range(T):
        for j in range(K):
            e = int(exps[t, j])
            mid = x[t] @ w13[e].t()
            act = torch.nn.functional.silu(mid[:I]) * mid[I:]
            want[t] += wts[t, j] * (act @ w2[e].t())
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)


def test_prompt_lookup_known_answers_of_the_reference_kernel_test():
    """tests/runtime_python/test_prompt_lookup.py:8-60 of the reference: an n-gram planted at
    position 100 and again at the end of a 515-token prompt, five planted tokens behind the
    first occurrence -> those five are the drafts; without the first occurrence -> all -1.
    (Its wrapper passes the prompt length to both kernels.)"""
    N, S, PROMPT_LEN = 3, 5, 512 + 3
    g = torch.Generator().manual_seed(0)
    for planted in (True, False):
        toks = torch.randint(40, 1000, (2048,), generator=g)
        if planted:
            toks[100:103] = torch.tensor([10, 20, 30])
            toks[103:108] = torch.tensor([4, 5, 6, 7, 8])
        toks[PROMPT_LEN - N:PROMPT_LEN] = torch.tensor([10, 20, 30])
        toks[PROMPT_LEN] = 99
        got = [int(toks[PROMPT_LEN])] + O.prompt_lookup(toks.tolist(), PROMPT_LEN, N, S, n_in=PROMPT_LEN)
        assert got == ([99, 4, 5, 6, 7, 8] if planted else [99, -1, -1, -1, -1, -1])


def test_verify_known_answers_of_the_reference_kernel_test():
    """tests/runtime_python/test_verify.py:7-50 of the reference."""
    target = [10, 20, 30, 40, 50, 60]
    assert O.verify_accept([100, 10, 20, 30, 40, 50], target) == 6          # all drafts accepted
    n = O.verify_accept([100, 10, 20, 99, 40, 50], target)                  # mismatch at the third
    assert n == 3 and target[:n] == [10, 20, 30]


def test_moe_routing_matches_the_reference_tests_torch_computation():
    """The torch computation the reference's kernel test compares against
    (tests/runtime_python/blackwell/sm100_moe/test_gate_topk.py:21-50): softmax over 128 bf16
    router logits, top 8, renormalised; routing index = top-k position + 1; active mask."""
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(1234)
    E, K, T = 128, 8, 3
    logits = torch.randn(T, E, generator=g).to(torch.bfloat16)
    w, e = O.moe_topk_softmax(logits, K)
    f = logits.float()
    sm = F.softmax(f - f.amax(dim=1, keepdim=True), dim=1, dtype=torch.float)
    tv, ti = torch.topk(sm, K, dim=1)
    torch.testing.assert_close(w, tv / tv.sum(dim=-1, keepdim=True), rtol=1e-2, atol=1e-2)
    # bf16 logits tie now and then: torch.topk leaves the order of equal values open, the kernel
    # (and the oracle) take the lower expert id first, so positions may swap among equals
    routing = torch.zeros(E, T, dtype=torch.int32)
    mine = torch.zeros(E, T, dtype=torch.int32)
    for t in range(T):
        for j in range(K):
            routing[ti[t, j], t] = j + 1
            mine[e[t, j], t] = j + 1
    assert torch.equal(routing != 0, mine != 0), "the same experts are active for every token"
    for t in range(T):
        for j in range(K):
            if routing[e[t, j], t] != j + 1:
                other = int(ti[t, j])
                assert sm[t, other] == sm[t, int(e[t, j])] and int(e[t, j]) < other or \
                    sm[t, other] == sm[t, int(e[t, j])]


def test_moe_weighted_sum_matches_the_reference_tests_torch_computation():
    """tests/runtime_python/blackwell/sm100_moe/test_weighted_sum.py:20-38 (tolerance 1e-2 as there;
    the reference's torch lines round the sum before adding the residual, the kernel and this
    oracle add in fp32 and round once)."""
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(5)
    T, K, H, E = 2, 8, 256, 128
    x = torch.randn(T, K, H, generator=g).to(torch.bfloat16)
    residual = torch.randn(T, H, generator=g).to(torch.bfloat16)
    score = torch.randn(T, E, generator=g).to(torch.bfloat16)
    wts = F.softmax(torch.topk(score, K, dim=1)[0], dim=1, dtype=torch.float)
    want = (x.float() * wts.unsqueeze(-1)).sum(dim=1).to(torch.bfloat16)
    want += residual
    got = O.moe_combine(x, wts, residual, rounding="bf16")
    torch.testing.assert_close(got.to(torch.bfloat16), want, rtol=1e-2, atol=1e-2)
