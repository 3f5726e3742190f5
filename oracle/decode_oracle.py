"""CPU oracle for the persistent-kernel decode path.  TEST INFRASTRUCTURE ONLY: imported by
tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline / reference legs as the
checker; the product (yirage_b200) never imports it.

Each function restates, in plain torch-on-CPU fp32 arithmetic, what the reference computes
for one piece of the path; the docstrings give the reference file:line followed.

Pinning.  The reference commits no golden vectors for this path and its native library
cannot be built here (needs Rust, CUTLASS and json submodules that are empty in the tree).
What can run here is the reference's PyTorch model code
(demo/llama3/models/modeling_llama3.py): Llama3RMSNorm, Llama3MLP, naive_attention,
Llama3RotaryEmbedding.  tests/golden/make_golden.py imports those from the reference tree,
runs them on seeded inputs and stores inputs+outputs under tests/golden/; the tests check
this oracle against those fixtures.  The same script also covers what has a counterpart on a
CPU: the rotate-half RoPE application, the paged-KV indexing with its in-place K update, the
causal window among several new tokens and the q/k RMSNorm inside attention are pinned by
the torch functions the reference's own kernel tests compare against
(tests/runtime_python/test_paged_attention.py, test_multitoken_paged_attention.py,
test_decoding_w_norm.py), whose definitions make_golden.py takes out of those scripts and
runs on CPU.  Still "parity unpinned" (CUDA-only in the reference, followed by reading): the
continuous batcher, the all-reduce order and the arg-max tie order.

`rounding="bf16"` reproduces the rounding points of the reference's bf16 pipeline (every
operator output rounded to bf16); `rounding=None` keeps fp32 throughout and is the fp32
reference the tolerance (max-abs 2e-2, relative 1e-2) is stated against.
"""
import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

ATOL = 2e-2
RTOL = 1e-2


def rnd(x: torch.Tensor, rounding):
    if rounding == "bf16":
        return x.to(torch.bfloat16).to(torch.float32)
    if rounding == "fp16":
        return x.to(torch.float16).to(torch.float32)
    return x


def within_tolerance(got: torch.Tensor, want: torch.Tensor, atol=ATOL, rtol=RTOL):
    """|got - want| <= atol + rtol * |want| element-wise; returns (ok, max_abs, worst_ratio)."""
    got, want = got.double(), want.double()
    err = (got - want).abs()
    bound = atol + rtol * want.abs()
    return bool((err <= bound).all()), float(err.max()), float((err / bound).max())


# ------------------------------------------------------------------ operators
def rmsnorm(x, w, eps, rounding=None):
    """y = x * rsqrt(mean(x^2) + eps) * w  (modeling_llama3.py:48-52; the persistent-kernel
    task does the same in fp32 and rounds once, tasks/hopper/rmsnorm_hopper.cuh:20-155).
    w may be None: the kernel-graph rms_norm has no weight and no eps
    (src/kernel/cuda/rms_norm_kernel.cu:30-60)."""
    x = x.float()
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    if w is not None:
        y = y * w.float()
    return rnd(y, rounding)


def linear(x, w, residual=None, rounding=None):
    """y = x @ w.T (+ residual); w is [N, K] as torch.nn.Linear.weight
    (modeling_llama3.py:103-111,200-202,251; linear_sm100_mpk.cuh:31-707)."""
    y = x.float() @ w.float().t()
    if residual is not None:
        y = y + residual.float()
    return rnd(y, rounding)


def silu_mul(g, u, rounding=None):
    """silu(g) * u with the task's rounding points when rounding is on: silu in fp32 rounded
    to bf16, product rounded to bf16 (tasks/ampere/silu_mul.cuh:33-40)."""
    g, u = g.float(), u.float()
    s = rnd(g * torch.sigmoid(g), rounding)
    return rnd(s * u, rounding)


def gated_mlp(x, w_gate, w_up, w_down, rounding=None):
    """down(silu(gate(x)) * up(x))  (modeling_llama3.py:103-111)."""
    g = linear(x, w_gate, rounding=rounding)
    u = linear(x, w_up, rounding=rounding)
    return linear(silu_mul(g, u, rounding), w_down, rounding=rounding)


def moe_topk_softmax(gate_logits, k: int, renormalize: bool = True):
    """Routing of a mixture-of-experts layer (topk_softmax_task_impl,
    tasks/blackwell/topk_softmax_sm100.cuh:63-303, registered with renormalize = true,
    src/kernel/task_register.cc:2119-2133): softmax over all experts in fp32, the k largest
    probabilities in order (lowest expert index on ties), divided by their sum.
    Returns (weights [T, k] fp32, experts [T, k] int64)."""
    p = torch.softmax(gate_logits.float(), dim=-1)
    T, E = p.shape
    weights = torch.zeros(T, k)
    experts = torch.zeros(T, k, dtype=torch.int64)
    for t in range(T):
        row = p[t].clone()
        for j in range(k):
            m = row.max()
            e = int((row == m).nonzero()[0])      # lowest index among equals
            weights[t, j], experts[t, j] = m, e
            row[e] = -10000.0
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    return weights, experts


def moe_combine(expert_out, weights, residual, rounding=None):
    """residual + sum_j weight_j * expert_out[:, j] accumulated in fp32 in slot order on top
    of the residual, rounded once (mul_sum_add_sm100_task_impl,
    tasks/blackwell/mul_sum_add_sm100.cuh:24-47).  expert_out [T, k, H], weights [T, k]."""
    acc = residual.float().clone()
    for j in range(expert_out.shape[1]):
        acc = acc + expert_out[:, j].float() * weights[:, j:j + 1].float()
    return rnd(acc, rounding)


def moe_mlp(x, gate_w, w13, w2, k: int, residual, rounding=None):
    """Mixture-of-experts MLP as the reference's task sequence computes it
    (demo/qwen3/demo_30B_A3B.py:598-645): router logits (a linear operator, 16-bit output),
    top-k softmax routing, per selected expert w13 = [gate; up] -> silu(gate) * up -> w2,
    then residual + sum_j weight_j * out_j accumulated in fp32 in slot order and rounded once
    (mul_sum_add_sm100_task_impl, tasks/blackwell/mul_sum_add_sm100.cuh:24-47).
    gate_w [E, H]; w13 [E, 2I, H]; w2 [E, H, I]."""
    logits = linear(x, gate_w, rounding=rounding or "bf16")   # moe_gate_out is a 16-bit tensor
    weights, experts = moe_topk_softmax(logits, k)
    T = x.shape[0]
    inter = w13.shape[1] // 2
    eo = torch.zeros(T, k, w2.shape[1])
    for t in range(T):
        for j in range(k):
            e = int(experts[t, j])
            mid = linear(x[t:t + 1], w13[e], rounding=rounding)
            act = silu_mul(mid[:, :inter], mid[:, inter:], rounding)
            eo[t, j] = linear(act, w2[e], rounding=rounding)[0]
    return moe_combine(eo, weights, residual, rounding)


def rope_tables(head_dim: int, theta: float, max_pos: int):
    """cos/sin tables [max_pos, head_dim] in bf16: fp32 angles pos * theta^(-2i/d), the half
    table repeated twice (modeling_llama3.py:71-89 with the default rope init of
    transformers: inv_freq = 1 / theta^(arange(0, d, 2) / d))."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    pos = torch.arange(max_pos, dtype=torch.float32)
    freqs = pos[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)


def apply_rope(x, cos, sin, rounding=None):
    """Rotate-half: first half  x1*cos - x2*sin, second half  x2*cos + x1*sin
    (demo/llama3/models/rope.py:79-126; rotary_embedding_sm100.cuh:56-73).
    x: [..., head_dim]; cos/sin broadcastable [..., head_dim]."""
    x = x.float()
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos.float(), sin.float()
    out = torch.cat((x1 * c[..., :d] - x2 * s[..., :d], x2 * c[..., d:] + x1 * s[..., d:]), dim=-1)
    return rnd(out, rounding)


def attention_rows(q, k, v, causal_offset=None):
    """softmax(q k^T / sqrt(d)) v for one kv head.  q: [rows, d]; k, v: [L, d].
    causal_offset[i] = number of keys row i may see (None: all)
    (modeling_llama3.py:114-135; attention_sm100.cuh:81 for the scale)."""
    q, k, v = q.float(), k.float(), v.float()
    s = (q @ k.t()) / math.sqrt(q.shape[-1])
    if causal_offset is not None:
        L = k.shape[0]
        mask = torch.arange(L)[None, :] >= torch.as_tensor(causal_offset)[:, None]
        s = s.masked_fill(mask, float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def shuffle_rows(sources: List[torch.Tensor], num_groups: int):
    """Row interleave of shuffle_tensors: group g holds rows [g*n_i/G, (g+1)*n_i/G) of every
    source in turn (src/kernel/graph.cc:398-437, runtime.cc:804-842)."""
    parts = []
    for g in range(num_groups):
        for s in sources:
            n = s.shape[0] // num_groups
            parts.append(s[g * n:(g + 1) * n])
    return torch.cat(parts, 0)


def argmax_lowest(logits):
    """Index of the maximum, lowest index on ties (torch.argmax semantics; the reference's
    warp reduction does not define the tie order, argmax_sm100.cuh:78-167)."""
    m = logits.max(dim=-1, keepdim=True).values
    idx = torch.arange(logits.shape[-1]).expand_as(logits)
    big = torch.full_like(idx, logits.shape[-1])
    return torch.where(logits == m, idx, big).min(dim=-1).values


def allreduce_sum(partials: List[torch.Tensor], rounding="bf16"):
    """Sum over ranks in rank order with fp32 accumulation, one rounding at the end
    (tasks/ampere/reduction.cuh:139-166)."""
    acc = torch.zeros_like(partials[0], dtype=torch.float32)
    for p in partials:
        acc = acc + p.float()
    return rnd(acc, rounding)


# ------------------------------------------------------------------ paged KV + batcher
@dataclass
class BatchState:
    """Host model of the on-device continuous batcher (persistent_kernel.cuh:107-132,
    169-322) with this build's two deliberate differences: paged_kv_last_page_len lies in
    [1, page_size] and a request contributes at most max_new_per_request new tokens per
    iteration (8, or 32 // q-heads-per-kv-head if that is smaller)."""
    total_requests: int
    max_requests: int
    max_tokens: int
    max_pages: int
    page_size: int
    max_seq_length: int
    eos: int
    tokens: torch.Tensor            # [total_requests, max_seq_length] int64
    prompt_len: List[int]
    max_new_per_request: int = 8
    # prompt-lookup speculative decoding: a request that is past its prompt brings its last
    # token plus `spec_length` draft tokens per iteration (0: off); `num_new_tokens[req]` is
    # what the verification accepted (target_verify.cuh:20-60), read by the next
    # prepare_next_batch as the reference's online batcher does (persistent_kernel.cuh:325-352)
    spec_length: int = 0
    ngram_size: int = 3
    num_new_tokens: List[int] = field(default_factory=list)
    step: List[int] = field(default_factory=list)
    request_ids: List[int] = field(default_factory=list)
    qo_indptr: List[int] = field(default_factory=list)
    kv_indptr: List[int] = field(default_factory=list)
    kv_indices: List[int] = field(default_factory=list)
    kv_last_len: List[int] = field(default_factory=list)
    input_tokens: List[int] = field(default_factory=list)
    next_request: int = 0
    page_queue: List[int] = field(default_factory=list)
    head: int = 0
    tail: int = 0

    def __post_init__(self):
        self.step = [0] * self.total_requests
        self.num_new_tokens = [1] * self.total_requests
        self.request_ids = [-1] * self.max_requests
        self.qo_indptr = [0] * (self.max_requests + 1)
        self.kv_indptr = [0] * (self.max_requests + 1)
        self.kv_indices = [0] * self.max_pages
        self.kv_last_len = [0] * self.max_requests
        self.input_tokens = [0] * self.max_tokens
        self.page_queue = list(range(self.max_pages))
        self.head, self.tail = 0, self.max_pages

    def prepare_next_batch(self, output_tokens: Optional[List[int]]):
        MR, MT, MP, PS = self.max_requests, self.max_tokens, self.max_pages, self.page_size
        # 1. retire / advance the previous batch
        for i in range(MR):
            req = self.request_ids[i]
            if req < 0:
                continue
            step = self.step[req]
            qo = self.qo_indptr[i]
            ntok = self.qo_indptr[i + 1] - qo
            plen = self.prompt_len[req]
            if self.spec_length > 0 and step >= plen and ntok > 1:
                # drafts were verified: only the accepted outputs count
                ntok = max(1, min(ntok, self.num_new_tokens[req]))
            for j in range(ntok):
                if step + j + 1 >= plen and step + j + 1 < self.max_seq_length:
                    self.tokens[req, step + j + 1] = output_tokens[qo + j]
            self.step[req] = step + ntok
            full = step + ntok + 1 >= self.max_seq_length
            eos = (step + ntok >= plen and step + ntok < self.max_seq_length
                   and int(self.tokens[req, step + ntok]) == self.eos)
            if full or eos:
                self.request_ids[i] = -1
                kv = self.kv_indptr[i]
                for j in range(self.kv_indptr[i + 1] - kv):
                    self.page_queue[self.tail % MP] = self.kv_indices[kv + j]
                    self.tail += 1
        old_indices = list(self.kv_indices)
        old_indptr = list(self.kv_indptr)
        old_ids = list(self.request_ids)
        nreq = ntok = npages = 0
        # 2. surviving requests
        for i in range(MR):
            req = old_ids[i]
            if req < 0:
                continue
            kv = old_indptr[i]
            nold = old_indptr[i + 1] - kv
            step = self.step[req]
            nnew = self.prompt_len[req] - step
            if nnew > 0:
                nnew = min(nnew, MT - ntok, self.max_new_per_request)
            else:
                nnew = min(1, MT - ntok)
                want = 1 + self.spec_length
                if (self.spec_length > 0 and MT - ntok >= want and want <= self.max_new_per_request
                        and step + want < self.max_seq_length):
                    nnew = want      # the last token and the draft slots (filled by fill_drafts)
            self.request_ids[nreq] = req
            self.qo_indptr[nreq] = ntok
            self.kv_indptr[nreq] = npages
            for j in range(nold):
                self.kv_indices[npages + j] = old_indices[kv + j]
            for j in range(nnew):
                past_prompt = self.prompt_len[req] - step <= 0
                self.input_tokens[ntok + j] = int(self.tokens[req, step + j]) if not (past_prompt and j > 0) else -1
            total = step + nnew
            need = (total + PS - 1) // PS
            if need > nold and (self.tail - self.head < need - nold or npages + need > MP):
                raise RuntimeError("KV page pool exhausted")   # the device raises YPK_ERR_STATE
            for j in range(nold, need):
                self.kv_indices[npages + j] = self.page_queue[self.head % MP]
                self.head += 1
            self.kv_last_len[nreq] = (total - 1) % PS + 1 if total > 0 else 0
            npages += max(need, nold)
            ntok += nnew
            nreq += 1
        # 3. admit new requests
        while nreq < MR and ntok < MT:
            req = self.next_request
            if req >= self.total_requests:
                break
            s0 = max(0, min(self.step[req], self.max_seq_length - 2))   # tokens taken as cached
            left = self.prompt_len[req] - s0
            nnew = min(left, MT - ntok, self.max_new_per_request) if left > 0 else min(1, MT - ntok)
            need = (s0 + nnew + PS - 1) // PS
            if npages + need > MP or (self.tail - self.head) < need:
                break
            self.request_ids[nreq] = req
            self.qo_indptr[nreq] = ntok
            self.kv_indptr[nreq] = npages
            for j in range(nnew):
                self.input_tokens[ntok + j] = int(self.tokens[req, s0 + j])
            for j in range(need):
                self.kv_indices[npages + j] = self.page_queue[self.head % MP]
                self.head += 1
            self.kv_last_len[nreq] = (s0 + nnew - 1) % PS + 1 if s0 + nnew > 0 else 0
            npages += need
            ntok += nnew
            nreq += 1
            self.next_request = req + 1
        for i in range(nreq, MR):
            self.request_ids[i] = -1
        for i in range(nreq, MR + 1):
            self.qo_indptr[i] = ntok
            self.kv_indptr[i] = npages
        return ntok


def prompt_lookup(tokens_row, step: int, ngram_size: int, spec_length: int,
                  n_in: Optional[int] = None) -> List[int]:
    """Draft tokens of prompt-lookup decoding (find_ngram_partial_kernel +
    find_ngram_global_kernel, tasks/speculative_decoding/prompt_lookup.cuh:22-132): the last
    `ngram_size` tokens of the history tokens[0..n_in) are searched in the history before them;
    the tokens after the earliest match are the drafts, -1 where there is no match or the
    index would pass `step`.  The persistent kernel calls the two kernels with n_in = step + 1
    and step (src/kernel/task_register.cc:726-729,758-765), the default here; the reference's
    kernel test calls both with the prompt length (tests/runtime_python/
    runtime_kernel_wrapper.cu:1388-1406)."""
    if n_in is None:
        n_in = step + 1
    drafts = [-1] * spec_length
    if n_in <= ngram_size:
        return drafts
    row = [int(t) for t in tokens_row[:n_in]]
    ngram = row[n_in - ngram_size:]
    for idx in range(n_in - ngram_size):
        if row[idx:idx + ngram_size] == ngram:
            for t in range(spec_length):
                j = idx + ngram_size + t
                drafts[t] = row[j] if j <= step else -1
            break
    return drafts


def verify_accept(spec_tokens, target_tokens) -> int:
    """target_verify_greedy_kernel (tasks/speculative_decoding/target_verify.cuh:20-60):
    spec_tokens[0] is the request's own last token, [1:] the drafts; draft i + 1 is accepted
    while it equals target_tokens[i].  Returns the number of new tokens: accepted drafts + 1
    (the first `that many` target tokens are the new tokens)."""
    n = len(spec_tokens) - 1
    acc = n
    for i in range(n):
        if int(spec_tokens[i + 1]) != int(target_tokens[i]):
            acc = i
            break
    return acc + 1


def fill_drafts(bs: BatchState):
    """The draft slots of every request that is past its prompt (the batcher left -1 there)."""
    for i in range(bs.max_requests):
        req = bs.request_ids[i]
        if req < 0:
            continue
        a, b = bs.qo_indptr[i], bs.qo_indptr[i + 1]
        if bs.spec_length > 0 and bs.step[req] >= bs.prompt_len[req] and b - a > 1:
            d = prompt_lookup(bs.tokens[req], bs.step[req], bs.ngram_size, b - a - 1)
            bs.input_tokens[a + 1:b] = d


def verify_greedy(bs: BatchState, output_tokens: List[int]):
    """target_verify_greedy_kernel (tasks/speculative_decoding/target_verify.cuh:20-60): draft
    i + 1 is accepted while it equals the model's output for position i; the count of new
    tokens is the accepted drafts plus the model's own next token."""
    for i in range(bs.max_requests):
        req = bs.request_ids[i]
        if req < 0:
            continue
        a, b = bs.qo_indptr[i], bs.qo_indptr[i + 1]
        n = b - a
        if bs.spec_length > 0 and bs.step[req] >= bs.prompt_len[req] and n > 1:
            bs.num_new_tokens[req] = verify_accept(bs.input_tokens[a:b], output_tokens[a:b])
        else:
            bs.num_new_tokens[req] = n


@dataclass
class LlamaWeights:
    """Per-rank weights of a Llama-style decoder, layout as torch.nn.Linear ([out, in])."""
    embed: torch.Tensor
    layers: List[dict]     # input_norm, q, k, v, o, post_norm, gate, up, down; a mixture-of-
                           # experts layer has moe_gate [E, H], w13 [E, 2I, H], w2 [E, H, I] instead
    final_norm: torch.Tensor
    lm_head: torch.Tensor
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    eps: float
    rope_theta: float
    experts_per_token: int = 0


def paged_attention_step(q, k_new, v_new, k_cache, v_cache, pages, seq_len, page_size,
                         num_q_heads, num_kv_heads, cos, sin, rounding="bf16",
                         q_norm_w=None, k_norm_w=None, qk_eps=1e-6):
    """Attention of T new tokens of one request against its paged cache, updating the cache
    in place.  q: [T, Hq, d]; k_new, v_new: [T, Hkv, d]; caches: [pages, page_size, Hkv, d];
    `pages` the request's page list; seq_len counts the new tokens
    (tests/runtime_python/test_multitoken_paged_attention.py:51-122 for the in-place update
    and causal windows; attention_sm100.cuh:86-102,254-269,412-427 for the indexing).
    q_norm_w / k_norm_w [d]: RMSNorm over the head dimension of every new q head and of the
    new k before the rotation, its result rounded like an operator output (Qwen3;
    attention_sm100.cuh:349-379, norm_sm100.cuh; test_decoding_w_norm.py:38-72)."""
    T = q.shape[0]
    G = num_q_heads // num_kv_heads
    pos0 = seq_len - T
    out = torch.zeros(T, num_q_heads, q.shape[-1])
    positions = torch.arange(pos0, seq_len)
    if q_norm_w is not None:
        q = rmsnorm(q, q_norm_w.reshape(-1), qk_eps, rounding)
        k_new = rmsnorm(k_new, k_norm_w.reshape(-1), qk_eps, rounding)
    if cos is not None:
        c, s = cos[positions][:, None, :], sin[positions][:, None, :]
        q = apply_rope(q, c, s, rounding)
        k_new = apply_rope(k_new, c, s, rounding)
    for t in range(T):
        p = pos0 + t
        pg = pages[p // page_size]
        k_cache[pg, p % page_size] = k_new[t].to(k_cache.dtype)
        v_cache[pg, p % page_size] = v_new[t].to(v_cache.dtype)
    idx_pages = torch.tensor([pages[p // page_size] for p in range(seq_len)])
    idx_slots = torch.tensor([p % page_size for p in range(seq_len)])
    K = k_cache[idx_pages, idx_slots].float()   # [seq, Hkv, d]
    V = v_cache[idx_pages, idx_slots].float()
    visible = [pos0 + t + 1 for t in range(T)]
    for h in range(num_kv_heads):
        qh = q[:, h * G:(h + 1) * G, :].reshape(T * G, -1)
        vis = [visible[t] for t in range(T) for _ in range(G)]
        o = attention_rows(qh, K[:, h], V[:, h], vis)
        out[:, h * G:(h + 1) * G, :] = o.reshape(T, G, -1)
    return rnd(out, rounding)


def decode_iteration(w: LlamaWeights, bs: BatchState, k_caches, v_caches, cos, sin,
                     rounding="bf16", num_tokens=None, logits_out=None, world=None):
    """One pass of the decode graph over the batch the batcher prepared: embedding, 32x
    (norm, qkv, paged attention, o_proj+residual, norm, gated MLP+residual), final norm,
    lm_head, arg-max.  Mirrors the layer sequence the demo builds
    (demo/llama3/demo.py:472-747) and the reference model's forward
    (modeling_llama3.py:188-298,363-393,421-445).  Returns the output token per batch row.
    `world`: list of LlamaWeights (one per tensor-parallel rank) replaces w for the sharded
    projections; partial sums are reduced with allreduce_sum."""
    ntok = bs.qo_indptr[bs.max_requests] if num_tokens is None else num_tokens
    ids = torch.tensor(bs.input_tokens[:ntok])
    valid = (ids >= 0) & (ids < w.embed.shape[0])        # an id outside the table embeds as zeros
    x = w.embed[ids.clamp(0, w.embed.shape[0] - 1)].float() * valid[:, None]
    d = w.head_dim
    for li, L in enumerate(w.layers):
        h = rmsnorm(x, L["input_norm"], w.eps, rounding)
        q = linear(h, L["q"], rounding=rounding).view(ntok, w.num_q_heads, d)
        k = linear(h, L["k"], rounding=rounding).view(ntok, w.num_kv_heads, d)
        v = linear(h, L["v"], rounding=rounding).view(ntok, w.num_kv_heads, d)
        attn = torch.zeros(ntok, w.num_q_heads, d)
        for i in range(bs.max_requests):
            if bs.request_ids[i] < 0:
                continue
            a, b = bs.qo_indptr[i], bs.qo_indptr[i + 1]
            if a == b:
                continue
            kv0, kv1 = bs.kv_indptr[i], bs.kv_indptr[i + 1]
            pages = bs.kv_indices[kv0:kv1]
            seq_len = (kv1 - kv0 - 1) * bs.page_size + bs.kv_last_len[i]
            attn[a:b] = paged_attention_step(q[a:b], k[a:b], v[a:b], k_caches[li], v_caches[li],
                                             pages, seq_len, bs.page_size, w.num_q_heads,
                                             w.num_kv_heads, cos, sin, rounding,
                                             q_norm_w=L.get("q_norm"), k_norm_w=L.get("k_norm"),
                                             qk_eps=w.eps)
        x = linear(attn.reshape(ntok, -1), L["o"], residual=x, rounding=rounding)
        h = rmsnorm(x, L["post_norm"], w.eps, rounding)
        if "moe_gate" in L:
            x = moe_mlp(h, L["moe_gate"], L["w13"], L["w2"], w.experts_per_token, x, rounding)
            continue
        g = linear(h, L["gate"], rounding=rounding)
        u = linear(h, L["up"], rounding=rounding)
        x = linear(silu_mul(g, u, rounding), L["down"], residual=x, rounding=rounding)
    h = rmsnorm(x, w.final_norm, w.eps, rounding)
    logits = linear(h, w.lm_head, rounding=rounding)
    if logits_out is not None:
        logits_out.append(logits)
    return argmax_lowest(logits).tolist()


def generate(w: LlamaWeights, bs: BatchState, k_caches, v_caches, cos, sin, rounding="bf16",
             max_iterations=None, logits_trace=None):
    """Run the batcher + decode graph until every request has retired (or for
    max_iterations).  tokens / step are updated in bs exactly as the device does."""
    out = None
    it = 0
    while True:
        ntok = bs.prepare_next_batch(out)
        if ntok == 0:
            break
        if max_iterations is not None and it >= max_iterations:
            break
        fill_drafts(bs)
        out = decode_iteration(w, bs, k_caches, v_caches, cos, sin, rounding,
                               logits_out=logits_trace)
        verify_greedy(bs, out)
        it += 1
    return it
