"""Shared helpers of the GPU parity tests: one-pass PersistentKernel graphs around a single
operator, seeded inputs, tolerance check."""
import torch

import yirage_b200 as yr
from oracle import decode_oracle as O


def randn(shape, seed, std=1.0, dtype=torch.bfloat16, device="cuda", mean=0.0):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * std + mean).to(dtype).to(device)


def onepass_kernel(max_tokens, meta=None, max_requests=1, max_pages=1, page_size=64,
                   max_seq_length=64):
    return yr.PersistentKernel(
        mode="onepass", world_size=1, mpi_rank=0, num_workers=128, num_local_schedulers=0,
        num_remote_schedulers=0, max_seq_length=max_seq_length,
        max_num_batched_requests=max_requests, max_num_batched_tokens=max_tokens,
        max_num_pages=max_pages, page_size=page_size, eos_token_id=-1, meta_tensors=meta or {},
        profiler_tensor=None, trace_name="", spec_decode_config=None, use_cutlass_kernel=True)


def assert_close(got, want, what=""):
    ok, max_abs, ratio = O.within_tolerance(got.float().cpu(), want.float().cpu())
    assert ok, f"{what}: max abs err {max_abs:.4g}, worst err/bound {ratio:.3g}"


def oracle_weights(shape, w):
    """Device weight dictionary (unsharded) -> oracle LlamaWeights on CPU."""
    c = lambda t: t.detach().cpu()
    return O.LlamaWeights(
        embed=c(w["embed"]), layers=[{k: c(v) for k, v in L.items()} for L in w["layers"]],
        final_norm=c(w["final_norm"]), lm_head=c(w["lm_head"]),
        num_q_heads=shape.num_attention_heads, num_kv_heads=shape.num_key_value_heads,
        head_dim=shape.head_dim, eps=shape.rms_norm_eps, rope_theta=shape.rope_theta,
        experts_per_token=getattr(shape, "experts_per_token", 0))


def replay_against_oracle(shape, ow, device_tokens, prompt_lens, *, max_seq, max_requests,
                          max_tokens, max_pages, page_size, max_new_per_request=None, rounding=None,
                          check_tokens=True, decode_tokens=None, spec=None):
    """Teacher-forced replay: the fp32 oracle runs the same batcher and graph but sees the
    device's own token history, so every iteration is checked on identical inputs and one
    flipped near-tie cannot cascade.  Every device token must be the oracle arg-max or tie
    with it inside the activation tolerance.  Returns (iterations, batch state, logits of
    the last iteration, exact matches, sampled tokens).

    A request brings at most `max_new_per_request` new tokens per iteration: by default what one
    attention task takes (8, or 32 // q-heads-per-kv-head) in graphs of at most 8 tokens and
    min(64, max_tokens) in larger ones.  `decode_tokens`: the run is a prefill/decode pair: once
    a batch of at most that many tokens has been formed (not the first), the batcher goes on
    under the small graph's limits.  `spec` = (ngram_size, spec_length): prompt-lookup
    speculative decoding; the drafts are looked up in the (device's) token history, the
    verification runs on the device's tokens, and the rows behind the first rejected draft are
    not compared (the device wrote nothing for them)."""
    G = ow.num_q_heads // ow.num_kv_heads
    small = min(8, 32 // G)
    if max_new_per_request is None:
        max_new_per_request = small if max_tokens <= 8 else min(64, max_tokens)
    R = len(prompt_lens)
    tokens_ref = torch.zeros(R, max_seq, dtype=torch.int64)
    for r, n in enumerate(prompt_lens):
        tokens_ref[r, :n] = device_tokens[r, :n]
    bs = O.BatchState(total_requests=R, max_requests=max_requests, max_tokens=max_tokens,
                      max_pages=max_pages, page_size=page_size, max_seq_length=max_seq, eos=-1,
                      tokens=tokens_ref, prompt_len=list(prompt_lens),
                      max_new_per_request=max_new_per_request,
                      ngram_size=spec[0] if spec else 3, spec_length=spec[1] if spec else 0)
    L = len(ow.layers)
    kc = [torch.zeros(max_pages, page_size, ow.num_kv_heads, ow.head_dim, dtype=torch.bfloat16)
          for _ in range(L)]
    vc = [torch.zeros_like(k) for k in kc]
    cos, sin = O.rope_tables(ow.head_dim, ow.rope_theta, max(max_seq, 64))
    iters, exact, total, out, last_logits = 0, 0, 0, None, None
    while True:
        ntok = bs.prepare_next_batch(out)
        if ntok == 0:
            break
        if decode_tokens is not None and iters > 0 and ntok <= decode_tokens:
            bs.max_tokens, bs.max_new_per_request = decode_tokens, small
            decode_tokens = None
        trace = []
        O.fill_drafts(bs)
        pred = O.decode_iteration(ow, bs, kc, vc, cos, sin, rounding=rounding, logits_out=trace)
        logits = trace[0]
        out = list(pred)
        for i in range(max_requests):
            req = bs.request_ids[i]
            if req < 0:
                continue
            a, b = bs.qo_indptr[i], bs.qo_indptr[i + 1]
            drafts = bs.spec_length > 0 and bs.step[req] >= prompt_lens[req] and b - a > 1
            for j in range(a, b):
                pos = bs.step[req] + (j - a) + 1
                if pos >= prompt_lens[req] and pos < max_seq:
                    dev_tok = int(device_tokens[req, pos])
                    total += 1
                    exact += int(dev_tok == pred[j])
                    gap = float(logits[j].max() - logits[j, dev_tok])
                    assert not check_tokens or gap <= O.ATOL + O.RTOL * float(logits[j].max().abs()), \
                        f"request {req} position {pos}: device token {dev_tok} is {gap:.3f} below the max"
                    out[j] = dev_tok
                if drafts and j + 1 < b and bs.input_tokens[j + 1] != out[j]:
                    break       # draft rejected: the device's iteration ended here for this request
        O.verify_greedy(bs, out)
        last_logits = logits
        iters += 1
    return iters, bs, last_logits, exact, total
