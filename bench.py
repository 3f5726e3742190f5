"""Benchmark of the persistent-kernel decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (BASELINE.json configs[3]): random-init Llama-3-8B, bf16, batch 1, a
512-token prompt of uniform-random ids, greedy decode; seed 3.  One "step" is one decode
iteration of the megakernel (one new token per sequence): the prompt is prefilled untimed, W
decode iterations warm up, then exactly K iterations are timed with CUDA events around one
persistent-kernel launch.  With N > 1 the same model runs under N-way tensor parallelism
(strong scaling).  Prints one JSON line (rank 0).

 value      tokens/s over the K timed iterations, inputs resident in HBM
 e2e        tokens/s of a whole generation through PersistentKernel.__call__: the prompt starts
            in pinned host memory, 256 tokens are generated (BASELINE's count, whatever
            --steps is), the ids are read back to the host; prefill inside the time, with
            prefill_ms / decode_ms and the decode-only rate beside it
 roofline   weight + KV bytes one iteration has to read / time per iteration, against the
            measured copy bandwidth in MEASURED_PEAKS.json
 kernels    (N = 1) the task kernels on BASELINE configs[0..2]: achieved GB/s and fraction
 batch16    (N = 1) configs[3] at batch 16
 parity     (N > 1) a small model generated under N-way tensor parallelism just before the
            timed runs: the ranks' tokens bit-equal, rank 0's replayed against the CPU oracle
 llama3_70b (N > 1) configs[4]: the 70B shape at batch 1 / 8 / 64, context 2048
 cpu_baseline / --impl reference
            the CPU oracle (port of the reference's PyTorch model code) timed on the host
            cores on a bounded sample of the same workload
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

DRAM_TRAFFIC_RATIO = 1.000   # (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes, ncu, profiles/
PROMPT_LEN = 512
E2E_NEW_TOKENS = 256         # BASELINE configs[3]: 256 greedy decode steps
SEED = 3
FALLBACK_HBM_GBS = 6650.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (invalid as a result)")
    ap.add_argument("--workload", default="decode",
                    choices=["decode", "rmsnorm_linear", "gated_mlp", "attention"],
                    help="decode = BASELINE configs[3] (the headline); the others time one task "
                         "kernel on BASELINE configs[0..2] as a chain of independent copies")
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "llama3-70b", "qwen3-30b-a3b"],
                    help="llama3-70b = BASELINE configs[4] (context 2048); needs --gpus >= 2.  "
                         "qwen3-30b-a3b = the mixture-of-experts shape of the reference's "
                         "demo/qwen3/demo_30B_A3B.py (no BASELINE config; one GPU)")
    ap.add_argument("--timeline", action="store_true",
                    help="print the per-operator device timeline of one decode iteration (rank 0) "
                         "instead of the benchmark line; the recording itself costs ~0.3 %%")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline line only: no kernels / batch16 / llama3_70b / parity sub-results")
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.proc, self.lines = device, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.device), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ CPU baseline (oracle)
def cpu_decode_sample(shape, ctx, budget_s=20.0):
    """The oracle's decode arithmetic on the host cores, bounded: one transformer layer
    (norm, q/k/v, attention over `ctx` cached tokens, o_proj, norm, gated MLP) at batch 1
    is timed and scaled by the layer count, plus the lm_head once.  Returns
    (seconds per token, description)."""
    from oracle import decode_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(SEED)
    h, f, d = shape.hidden_size, shape.intermediate_size, shape.head_dim
    hq, hkv = shape.num_attention_heads, shape.num_key_value_heads
    mk = lambda r, c: (torch.randn(r, c, generator=g) * 0.02).to(torch.bfloat16)
    L = {"input_norm": torch.ones(h, dtype=torch.bfloat16), "q": mk(hq * d, h), "k": mk(hkv * d, h),
         "v": mk(hkv * d, h), "o": mk(h, hq * d), "post_norm": torch.ones(h, dtype=torch.bfloat16),
         "gate": mk(f, h), "up": mk(f, h), "down": mk(h, f)}
    lm = mk(shape.vocab_size // 8, h)   # an eighth of the vocabulary, scaled below
    x = torch.randn(1, h, generator=g).to(torch.bfloat16)
    kc = torch.randn(ctx + 1, hkv, d, generator=g).to(torch.bfloat16)
    vc = torch.randn(ctx + 1, hkv, d, generator=g).to(torch.bfloat16)
    cos, sin = O.rope_tables(d, shape.rope_theta, ctx + 1)

    def lin(a, w, res=None):
        # bf16 GEMV as the reference model runs it (torch.nn.Linear on bf16 tensors)
        y = torch.nn.functional.linear(a, w)
        return y if res is None else y + res

    def layer(xx):
        hh = O.rmsnorm(xx, L["input_norm"], shape.rms_norm_eps, "bf16").to(torch.bfloat16)
        q = lin(hh, L["q"]).view(1, hq, d)
        k = lin(hh, L["k"]).view(1, hkv, d)
        v = lin(hh, L["v"]).view(1, hkv, d)
        c, s = cos[ctx][None, None], sin[ctx][None, None]
        q = O.apply_rope(q, c, s, "bf16")
        k = O.apply_rope(k, c, s, "bf16")
        kc[ctx], vc[ctx] = k[0].to(torch.bfloat16), v[0].to(torch.bfloat16)
        G = hq // hkv
        outs = [O.attention_rows(q[0, hh_ * G:(hh_ + 1) * G], kc[:, hh_], vc[:, hh_]) for hh_ in range(hkv)]
        a = torch.cat(outs, 0).reshape(1, hq * d).to(torch.bfloat16)
        xx = lin(a, L["o"], xx)
        hh = O.rmsnorm(xx, L["post_norm"], shape.rms_norm_eps, "bf16").to(torch.bfloat16)
        act = O.silu_mul(lin(hh, L["gate"]), lin(hh, L["up"]), "bf16").to(torch.bfloat16)
        return lin(act, L["down"], xx)

    layer(x)  # warm-up
    t0 = time.perf_counter()
    reps = 0
    while True:
        layer(x)
        reps += 1
        if time.perf_counter() - t0 > budget_s * 0.6 or reps >= 16:
            break
    t_layer = (time.perf_counter() - t0) / reps
    lin(x, lm)
    t0 = time.perf_counter()
    for _ in range(2):
        lin(x, lm)
    t_lm = (time.perf_counter() - t0) / 2 * 8
    per_token = t_layer * shape.num_hidden_layers + t_lm
    desc = (f"oracle decode arithmetic, batch 1, ctx {ctx}: 1 of {shape.num_hidden_layers} layers x "
            f"{reps} reps + 1/8 of the lm_head, scaled to a full token")
    return per_token, desc


def cpu_prefill_sample(shape, prompt_len, chunk=64):
    """Host time to prefill `prompt_len` tokens with the same arithmetic: the projections of
    one layer on a chunk of tokens (causal attention inside the chunk left out: under 2 % of
    the flops at these lengths), scaled to all chunks and layers.  Returns seconds."""
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(SEED)
    h, f, d = shape.hidden_size, shape.intermediate_size, shape.head_dim
    hq, hkv = shape.num_attention_heads, shape.num_key_value_heads
    mk = lambda r, c: (torch.randn(r, c, generator=g) * 0.02).to(torch.bfloat16)
    ws = [mk((hq + 2 * hkv) * d, h), mk(h, hq * d), mk(2 * f, h), mk(h, f)]
    x = torch.randn(chunk, h, generator=g).to(torch.bfloat16)
    a = torch.randn(chunk, f, generator=g).to(torch.bfloat16)

    def layer():
        torch.nn.functional.linear(x, ws[0])
        torch.nn.functional.linear(x, ws[1])
        torch.nn.functional.linear(x, ws[2])
        torch.nn.functional.linear(a, ws[3])

    layer()
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 3.0 and reps < 8:
        layer()
        reps += 1
    t_layer = (time.perf_counter() - t0) / reps
    return t_layer * shape.num_hidden_layers * ((prompt_len + chunk - 1) // chunk)


# ------------------------------------------------------------------ reference arm
def run_reference(args):
    from yirage_b200 import llama
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    shape = llama.LlamaShape.llama3_8b()
    K, W = max(1, args.steps), args.warmup
    # each "step" is a bounded sample of a decode token; keep the whole run to ~a minute
    budget = max(2.0, min(20.0, 60.0 / (K + W)))
    per = []
    nsamples = min(K + W, 3)
    for i in range(nsamples):
        t, desc = cpu_decode_sample(shape, PROMPT_LEN, budget_s=budget)
        per.append(t)
    t_tok = sorted(per)[len(per) // 2]
    t_prefill = cpu_prefill_sample(shape, PROMPT_LEN)
    val = args.batch / t_tok
    e2e_val = E2E_NEW_TOKENS / (t_prefill + E2E_NEW_TOKENS * t_tok)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_second", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": t_tok * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "scaled_from_sample": True,
        "config": {"workload": "llama3-8b decode, batch 1, prompt 512, greedy (BASELINE configs[3])",
                   "note": "CPU port of the reference's PyTorch model code (the reference's native "
                           "library cannot be built here and its model code needs a GPU); the value "
                           f"is the median of {nsamples} samples, each one layer timed and scaled to "
                           "a token, not K full steps"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": desc},
        "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "prefill_ms": t_prefill * 1e3, "decode_ms": E2E_NEW_TOKENS * t_tok * 1e3,
                "new_tokens": E2E_NEW_TOKENS,
                "note": f"{E2E_NEW_TOKENS} tokens after a {PROMPT_LEN}-token prompt: prefill estimated "
                        "from one layer's projections on a 64-token chunk, decode from the sample above"},
        "e2e_decode_only": {"value": val, "unit": "tokens/s"},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ our arm
def _dist():
    import torch.distributed as dist
    return dist


def max_over_ranks(value, dev, world):
    if world == 1:
        return value
    t = torch.tensor([value], device=dev, dtype=torch.float64)
    _dist().all_reduce(t, op=_dist().ReduceOp.MAX)
    return float(t)


def tp_parity_prelude(world, rank, dev):
    """Correct tokens under N-way tensor parallelism, checked right here because the GPU test
    box has one GPU: a 2-layer 512-wide model (16 q / 8 kv heads so that it shards 8 ways)
    generates from three prompts through two request slots; every rank's token matrix must be
    bit-equal, and rank 0's is replayed iteration by iteration against the CPU oracle on the
    unsharded weights (each sampled token the oracle arg-max or inside the tolerance of it)."""
    dist = _dist()
    from yirage_b200 import llama
    shape = llama.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                             num_attention_heads=16, num_key_value_heads=8, vocab_size=3000)
    w = llama.init_weights(shape, dev, 3, world_size=world, rank=rank)
    prompt_lens, max_seq = [9, 14, 5], 30
    g = torch.Generator().manual_seed(3)
    tokens = torch.zeros(len(prompt_lens), max_seq, dtype=torch.int64)
    for r, n in enumerate(prompt_lens):
        tokens[r, :n] = torch.randint(0, shape.vocab_size, (n,), generator=g)
    tokens = tokens.to(dev)
    plen = torch.tensor(prompt_lens, dtype=torch.int32, device=dev)
    ypk, st = llama.build_decode_kernel(
        shape, w, tokens=tokens, prompt_lengths=plen, max_num_batched_requests=2,
        max_num_batched_tokens=8, max_num_pages=4, page_size=64, world_size=world, rank=rank)
    dist.barrier()
    ypk()
    torch.cuda.synchronize()
    status = ypk.status()
    every = [torch.empty_like(tokens) for _ in range(world)]
    dist.all_gather(every, tokens)
    agree = all(torch.equal(every[0], t) for t in every[1:])
    res = {"ranks_agree": bool(agree), "device_error": int(status.error), "world": world}
    if rank == 0:
        from tests.util import oracle_weights, replay_against_oracle
        full = llama.init_weights(shape, dev, 3)
        try:
            iters, bs, _, exact, total = replay_against_oracle(
                shape, oracle_weights(shape, full), tokens.cpu(), prompt_lens, max_seq=max_seq,
                max_requests=2, max_tokens=8, max_pages=4, page_size=64)
            ok = status.iterations == iters and st["meta"]["step"].cpu().tolist() == bs.step
            res.update(oracle_ok=bool(ok and status.error == 0), tokens=int(total),
                       exact_argmax_matches=int(exact), iterations=int(iters))
        except AssertionError as e:
            res.update(oracle_ok=False, tokens=0, failure=str(e)[:200])
        del full
    dist.barrier()
    ypk.finalize()
    del w, ypk, st
    torch.cuda.empty_cache()
    return res


def time_decode(ypk, st, K, W, B, prompt_len, shape, dev, world, rank, sample_clocks=False,
                synthetic_context=False):
    """Bring every request to the decode phase (untimed), W warm-up iterations, then exactly K
    iterations in one launch between two CUDA events; max over ranks.  Returns (ms, clocks)."""
    dist = _dist()
    ypk.reset()
    if synthetic_context:
        # the requests enter with `prompt_len` tokens taken as cached: their pages keep
        # whatever the cache tensors hold (random values), no prefill is run
        st["meta"]["step"].fill_(prompt_len - 1)
    else:
        # run the prompts: the launch returns once a batch of B tokens (one per request) waits
        ypk.set_pause_below(B)
        ypk()
        ypk.set_pause_below(0)
    ypk(max_iterations=W)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(dev.index) if (sample_clocks and rank == 0) else None
    if sampler:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = st["meta"]["step"].clone()
    time_decode.mean_context = float(before.float().mean()) + K / 2.0   # over the timed steps
    torch.cuda.synchronize()
    ev0.record()
    ypk(max_iterations=K)
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if sampler else None
    done = int((st["meta"]["step"] - before).sum())
    assert done == K * B, f"timed region ran {done} token-steps, expected {K * B}"
    assert ypk.status().error == 0
    return max_over_ranks(ms, dev, world), clocks


def decode_bytes(shape, world, B, ctx):
    """Algorithmic HBM bytes of one decode iteration on one GPU: its shard of every weight
    (lm_head padded and split by vocabulary rows) + the K/V of its kv heads over `ctx` tokens."""
    from yirage_b200 import llama
    wbytes = shape.decode_weight_bytes(1, llama.padded_vocab(shape.vocab_size)) / world
    kv = B * ctx * shape.num_hidden_layers * shape.num_key_value_heads * shape.head_dim * 2 * 2 / world
    return wbytes, kv


def run_ours(args):
    from yirage_b200 import llama
    dist = _dist()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    K, W, B = args.steps, max(args.warmup, 3), args.batch
    big = args.model == "llama3-70b"
    moe = args.model == "qwen3-30b-a3b"
    shape = (llama.LlamaShape.llama3_70b() if big else llama.LlamaShape.qwen3_30b_a3b() if moe
             else llama.LlamaShape.llama3_8b())
    if moe and world != 1:
        raise SystemExit("the mixture-of-experts graph is built for one GPU")
    prompt_len = 2048 if big else PROMPT_LEN
    if big and world < 2:
        raise SystemExit("llama3-70b (140 GB of weights) is a tensor-parallel configuration: --gpus 2/4/8")
    if args.layers:
        shape.num_hidden_layers = args.layers
    extras = not args.no_extras and not args.layers and not big and not moe

    parity = tp_parity_prelude(world, rank, dev) if (world > 1 and not args.no_extras) else None

    # ---- headline: 8 prompt tokens per request and iteration; all requests prefill in lockstep
    MT = 8 * B
    # a request retires at max_seq_length - 1 tokens: with this length the end-to-end run
    # below generates exactly E2E_NEW_TOKENS per request on the same kernel
    gen_seq = prompt_len + E2E_NEW_TOKENS
    max_seq = gen_seq if W + K + 2 <= E2E_NEW_TOKENS else prompt_len + W + K + 2
    page = 64
    pages_per_req = (max_seq + page - 1) // page
    g = torch.Generator().manual_seed(SEED)
    host_tokens = torch.zeros(B, max_seq, dtype=torch.int64)
    host_tokens[:, :prompt_len] = torch.randint(0, shape.vocab_size, (B, prompt_len), generator=g)
    host_tokens = host_tokens.pin_memory()
    host_plen = torch.full((B,), prompt_len, dtype=torch.int32).pin_memory()
    tokens, plen = host_tokens.to(dev), host_plen.to(dev)
    # N > 1: tensor parallelism over the N GPUs (column-split qkv / gate / up, row-split
    # o_proj / down_proj, in-kernel all-reduce over NVLink after each row-split projection;
    # lm_head split by vocabulary rows, arg-max winners exchanged).  Total work is fixed.
    weights = llama.init_weights(shape, dev, SEED, world_size=world, rank=rank)
    # One GPU, at most 8 token slots: the decode graph is paired with a 64-token graph over the
    # same requests and caches, which runs the prompt in the end-to-end measurement below.
    pair = None
    use_pair = MT <= 8 and not args.no_e2e
    if use_pair and max_seq == gen_seq:
        pair = llama.build_prefill_decode_pair(
            shape, weights, tokens=tokens, prompt_lengths=plen, max_num_batched_requests=B,
            max_num_pages=pages_per_req * B, page_size=page, prefill_tokens=64, decode_tokens=MT,
            world_size=world, rank=rank)
        ypk, st = pair.decode, pair.state
    else:
        ypk, st = llama.build_decode_kernel(
            shape, weights, tokens=tokens, prompt_lengths=plen, max_num_batched_requests=B,
            max_num_batched_tokens=MT, max_num_pages=pages_per_req * B, page_size=page,
            world_size=world, rank=rank)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms, clocks = time_decode(ypk, st, K, W, B, prompt_len, shape, dev, world, rank, sample_clocks=True)

    # ---- end to end: one whole generation through the public call, host buffers in and out,
    # always E2E_NEW_TOKENS new tokens per request (max_seq_length ends the generation)
    e2e = e2e_decode_only = None
    if not args.no_e2e:
        if max_seq == gen_seq:
            ypk2, st2, pair2, e_tokens, e_host = ypk, st, pair, tokens, host_tokens
        else:       # more timed steps than the generation is long: a second kernel of the right length
            e_tokens = torch.zeros(B, gen_seq, dtype=torch.int64, device=dev)
            e_host = torch.zeros(B, gen_seq, dtype=torch.int64)
            e_host[:, :prompt_len] = host_tokens[:, :prompt_len]
            e_host = e_host.pin_memory()
            pair2 = None
            kw2 = dict(tokens=e_tokens, prompt_lengths=plen, max_num_batched_requests=B,
                       max_num_pages=((gen_seq + page - 1) // page) * B, page_size=page)
            if use_pair:
                pair2 = llama.build_prefill_decode_pair(shape, weights, prefill_tokens=64,
                                                        decode_tokens=MT, world_size=world,
                                                        rank=rank, **kw2)
                ypk2, st2 = pair2.decode, pair2.state
            else:
                ypk2, st2 = llama.build_decode_kernel(shape, weights, max_num_batched_tokens=MT,
                                                      world_size=world, rank=rank, **kw2)
        host_out = torch.empty_like(e_host).pin_memory()
        host_step = torch.empty(B, dtype=torch.int32).pin_memory()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        e_tokens.copy_(e_host, non_blocking=True)
        plen.copy_(host_plen, non_blocking=True)
        if pair2 is not None:
            # the prompt on the 64-token graph (a launch that returns once a batch of at most
            # MT tokens waits), the rest on the decode graph
            pair2.reset()
            pair2.prefill()
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            pair2.decode.adopt(pair2.prefill)
            pair2.decode()
            prefill_iters = int(pair2.prefill.status().iterations)
            launches = 2
        else:
            ypk2.reset()
            ypk2.set_pause_below(B)                  # returns when every request is past its prompt
            ypk2()
            ypk2.set_pause_below(0)
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            prefill_iters = int(ypk2.status().iterations)
            ypk2()                                   # decode until every request has retired
            launches = 2
        host_out.copy_(e_tokens, non_blocking=True)
        host_step.copy_(st2["meta"]["step"], non_blocking=True)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        gen = int((host_step.to(torch.int64) + 1 - prompt_len).sum())
        iters = int(ypk2.status().iterations) + (prefill_iters if pair2 is not None else 0)
        dt = max_over_ranks(t2 - t0, dev, world)
        t_pre = max_over_ranks(t1 - t0, dev, world)
        h2d = e_host.numel() * 8 + host_plen.numel() * 4
        d2h = host_out.numel() * 8 + host_step.numel() * 4
        e2e = {"value": gen / dt, "unit": "tokens/s",
               "h2d_bytes_per_step": h2d / max(1, iters), "d2h_bytes_per_step": d2h / max(1, iters),
               "new_tokens": gen, "iterations": iters,
               "prefill_ms": t_pre * 1e3, "decode_ms": (dt - t_pre) * 1e3,
               "prefill_iterations": prefill_iters, "gpu_launches": launches,
               "prefill_graph": ("64 token slots, attention over query tiles, LINEAR on tcgen05"
                                 if pair2 is not None else f"the decode graph itself, {MT} token slots"),
               "note": f"{gen} generated tokens after a {prompt_len}-token prompt ({prefill_iters} chunked-"
                       "prefill iterations), prompt copied from pinned host memory, token matrix and step "
                       "counters read back; independent of --steps"}
        e2e_decode_only = {"value": gen / max(1e-9, dt - t_pre), "unit": "tokens/s",
                           "note": "same run, prefill time taken out (the device->host read-back stays in)"}
        if ypk2 is not ypk:
            (pair2 or ypk2).finalize()
        del ypk2, st2, e_tokens, pair2

    sub = {}
    if extras and world == 1:
        # ---- BASELINE configs[3] at batch 16 (same weights): 16 requests over 64 token slots
        try:
            B16, K16 = 16, max(8, min(K, 48))
            # the requests run their prompts one after the other (64 tokens per iteration), so
            # the first ones have decoded ~9 tokens per later request before the timing starts
            mseq = prompt_len + 12 * B16 + W + K16 + 8
            tk = torch.zeros(B16, mseq, dtype=torch.int64)
            tk[:, :prompt_len] = torch.randint(0, shape.vocab_size, (B16, prompt_len), generator=g)
            tk = tk.to(dev)
            pl16 = torch.full((B16,), prompt_len, dtype=torch.int32, device=dev)
            y16, s16 = llama.build_decode_kernel(
                shape, weights, tokens=tk, prompt_lengths=pl16, max_num_batched_requests=B16,
                max_num_batched_tokens=64, max_num_pages=((mseq + page - 1) // page) * B16,
                page_size=page)
            ms16, _ = time_decode(y16, s16, K16, W, B16, prompt_len, shape, dev, 1, 0)
            wb, kvb = decode_bytes(shape, 1, B16, time_decode.mean_context)
            hbm, src = peaks()
            ach = (wb + kvb) / (ms16 / 1e3 / K16) / 1e9
            sub["batch16"] = {"ms_per_step": ms16 / K16, "tokens_per_s": K16 * B16 / (ms16 / 1e3),
                              "steps": K16, "achieved_gbs": ach, "frac": ach / hbm,
                              "frac_of": f"{src} copy bandwidth",
                              "tensor_core_tasks": int(y16.status().tensor_core_tasks),
                              "mean_context": time_decode.mean_context,
                              "workload": "llama3-8b decode, batch 16, prompt 512 (BASELINE configs[3])"}
            y16.finalize()
            del y16, s16, tk
        except Exception as e:   # a sub-result must not take the headline down
            sub["batch16"] = {"error": str(e)[:300]}
    (pair or ypk).finalize()
    del ypk, st, weights, pair
    torch.cuda.empty_cache()

    if extras and world == 1:
        ks = {}
        for key, wl, b in (("rmsnorm_linear", "rmsnorm_linear", 8), ("gated_mlp_b8", "gated_mlp", 8),
                           ("gated_mlp_b16", "gated_mlp", 16), ("gated_mlp_b64", "gated_mlp", 64),
                           ("attention", "attention", 8)):
            try:
                r = measure_kernel(wl, b, steps=20, warmup=3)
                ks[key] = {"gbs": r["achieved"], "frac": r["frac"], "us_per_operator": r["us_per_operator"],
                           "ms_per_step": r["ms"], "tensor_core_tasks": r["tensor_core_tasks"],
                           "workload": r["name"]}
            except Exception as e:
                ks[key] = {"error": str(e)[:300]}
            torch.cuda.empty_cache()
        sub["kernels"] = ks

    if extras and world > 1:
        # ---- BASELINE configs[4]: Llama-3-70B shape, context 2048, batch 1 / 8 / 64
        try:
            sub["llama3_70b"] = run_70b(world, rank, dev, steps=max(4, min(K, 16)), warmup=3)
        except Exception as e:
            sub["llama3_70b"] = {"error": str(e)[:300]}

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    hbm, src = peaks()
    wbytes, kv_bytes = decode_bytes(shape, world, B, prompt_len + W + K / 2.0)
    alg = wbytes + kv_bytes
    per_iter_s = ms / 1e3 / K
    achieved = alg / per_iter_s / 1e9
    line = {
        "metric": "decode_tokens_per_second", "value": K * B / (ms / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
        "us_per_token": ms * 1e3 / K / B,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.model} decode, batch {B}, prompt {prompt_len}, greedy "
                               + ("(no BASELINE config)" if moe else f"(BASELINE configs[{4 if big else 3}])"),
                   "layers": shape.num_hidden_layers, "page_size": page,
                   "parallelism": f"tp{world}" if world > 1 else "single",
                   "l2": f"weights streamed per iteration and GPU are {wbytes / 1e9:.1f} GB, far larger than the 126 MB L2"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                     "frac": achieved / hbm, "frac_of": f"{src} copy bandwidth, per GPU",
                     "frac_of_nominal_8TBs": achieved / 8000.0,
                     "algorithmic_bytes_per_iteration": alg,
                     "algorithmic_bytes_per_launch": alg * K,
                     # ncu on the 4-layer case of this kernel (profiles/): dram read + write =
                     # 0.998 x the algorithmic bytes of the captured launch; the traffic grows
                     # with the weights streamed, so the ratio carries over to the full launch
                     "traffic": DRAM_TRAFFIC_RATIO * alg * K,
                     "traffic_note": "scaled from the ncu capture of the 4-layer case (read + write = 1.000 x the algorithmic bytes), per launch of K iterations",
                     "kernel": "ypk_megakernel (one launch covers all K iterations)"},
        "clocks": clocks,
        "gpu_launches": 1,
    }
    if e2e is not None:
        line["e2e"] = e2e
        line["e2e_decode_only"] = e2e_decode_only
    if parity is not None:
        line["parity"] = parity
    line.update(sub)
    if not args.no_cpu_baseline and world == 1:
        t_tok, desc = cpu_decode_sample(shape, prompt_len, budget_s=15.0)
        line["cpu_baseline"] = {"value": 1.0 / t_tok, "unit": "tokens/s", "cores": os.cpu_count(),
                                "kind": "port", "sample": desc}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_70b(world, rank, dev, steps, warmup):
    """BASELINE configs[4] on the N GPUs of this run: Llama-3-70B shape (weights generated on
    the device per shard, ~139 GB / N per GPU), context 2048, batch 1, 8 and 64.  The context
    is synthetic: the requests enter the batcher with 2048 tokens taken as cached and the
    cache tensors hold random values, so no prefill of 2048 x batch tokens is run (at batch
    64 it would take minutes); the timed iterations read weights and 2048 tokens of K/V per
    request exactly as after a real prefill."""
    from yirage_b200 import llama
    dist = _dist()
    shape = llama.LlamaShape.llama3_70b()
    ctx, page = 2048, 64
    weights = llama.init_weights(shape, dev, 4, world_size=world, rank=rank)
    torch.cuda.empty_cache()      # the library allocates with cudaMalloc, outside torch's cache
    hbm, src = peaks()
    out = {"workload": "llama3-70b shape decode, context 2048 (BASELINE configs[4]), synthetic context",
           "parallelism": f"tp{world}", "steps": steps, "batch": {}}
    free_b, _ = torch.cuda.mem_get_info()
    def all_ok(flag):
        """Every rank must take the same path: the minimum of the ranks' flags."""
        t = torch.tensor([1 if flag else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(int(t))

    # the fused qkv / gate-up copies the library makes of the shard's weights
    h_, f_, d_ = shape.hidden_size, shape.intermediate_size, shape.head_dim
    copies = 2 * shape.num_hidden_layers * h_ * ((shape.num_attention_heads + 2 * shape.num_key_value_heads) * d_
                                                   + 2 * f_) // world
    for B in (1, 8, 64):
        ypk = None
        try:
            mseq = ctx + warmup + steps + 2
            pages = ((mseq + page - 1) // page) * B
            hkv = shape.num_key_value_heads // world
            kv_need = 2 * shape.num_hidden_layers * pages * page * hkv * shape.head_dim * 2
            torch.cuda.empty_cache()
            free_b, _ = torch.cuda.mem_get_info()
            if not all_ok(kv_need + copies < 0.92 * free_b):
                out["batch"][str(B)] = {"skipped": f"KV cache of {kv_need / 1e9:.0f} GB and {copies / 1e9:.0f} GB of fused "
                                                   f"weight copies do not fit in the {free_b / 1e9:.0f} GB left beside the weights"}
                continue
            g = torch.Generator().manual_seed(4)
            tk = torch.zeros(B, mseq, dtype=torch.int64)
            tk[:, :ctx] = torch.randint(0, shape.vocab_size, (B, ctx), generator=g)
            tk = tk.to(dev)
            pl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
            kc = torch.empty(shape.num_hidden_layers, pages, page, hkv, shape.head_dim,
                             dtype=torch.bfloat16, device=dev).normal_()
            vc = torch.empty_like(kc).normal_()
            try:
                ypk, st = llama.build_decode_kernel(
                    shape, weights, tokens=tk, prompt_lengths=pl, max_num_batched_requests=B,
                    max_num_batched_tokens=max(8, B), max_num_pages=pages, page_size=page,
                    world_size=world, rank=rank, k_cache=kc, v_cache=vc, defer_connect=True)
                built = True
            except Exception as e:
                built, why = False, str(e)[:200]
            if not all_ok(built):
                out["batch"][str(B)] = {"error": "the kernel could not be built on every rank" +
                                                 ("" if built else f": {why}")}
                if ypk is not None:
                    ypk.finalize()
                continue
            from yirage_b200 import tensor_parallel
            tensor_parallel.connect(ypk._handle, world, rank)
            dist.barrier()
            ms, _ = time_decode(ypk, st, steps, warmup, B, ctx, shape, dev, world, rank,
                                synthetic_context=True)
            wb, kvb = decode_bytes(shape, world, B, ctx + warmup + steps / 2.0)
            ach = (wb + kvb) / (ms / 1e3 / steps) / 1e9
            out["batch"][str(B)] = {"ms_per_step": ms / steps, "tokens_per_s": steps * B / (ms / 1e3),
                                    "us_per_token": ms * 1e3 / steps / B,
                                    "achieved_gbs_per_gpu": ach, "frac": ach / hbm,
                                    "frac_of": f"{src} copy bandwidth, per GPU",
                                    "tensor_core_tasks": int(ypk.status().tensor_core_tasks)}
            ypk.finalize()
            del ypk, st, kc, vc, tk
            torch.cuda.empty_cache()
        except Exception as e:
            out["batch"][str(B)] = {"error": str(e)[:300]}
            # every rank must take the same path afterwards: stop here
            break
    del weights
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------ task-kernel workloads
def measure_kernel(workload, batch, steps, warmup):
    """BASELINE configs[0..2] on one GPU.  One launch of a few microseconds cannot be timed
    from the host, so a step is a chain of `reps` independent copies of the operator (own
    weights / own KV cache each, several GB in total, far beyond L2) executed by one
    persistent-kernel launch; the figure is bytes the chain has to read / time."""
    import yirage_b200 as yr
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    K, W, B = steps, max(warmup, 3), batch
    g = torch.Generator(device=dev)

    def rn(shape, std, dtype, mean=0.0):
        return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std + mean).to(dtype)

    def pk(max_tokens, meta=None, **kw):
        return yr.PersistentKernel(
            mode="onepass", world_size=1, mpi_rank=0, num_workers=128, num_local_schedulers=0,
            num_remote_schedulers=0, max_seq_length=kw.get("max_seq", 64),
            max_num_batched_requests=kw.get("max_req", 1), max_num_batched_tokens=max_tokens,
            max_num_pages=kw.get("max_pages", 1), page_size=64, eos_token_id=-1,
            meta_tensors=meta or {}, profiler_tensor=None, trace_name="", spec_decode_config=None,
            use_cutlass_kernel=True)

    keep = []
    if workload == "rmsnorm_linear":
        g.manual_seed(0)
        reps, H, dt, ydt = 64, 4096, torch.float16, yr.float16
        ypk = pk(B)
        x = ypk.attach_input(rn((B, H), 1.0, dt), "x")
        alg = 0
        for i in range(reps):
            nw, w = rn((H,), 0.1, dt, 1.0), rn((H, H), 0.02, dt)
            keep += [nw, w]
            tmp = ypk.new_tensor(dims=(B, H), dtype=ydt, name=f"n{i}")
            out = ypk.new_tensor(dims=(B, H), dtype=ydt, name=f"o{i}")
            ypk.rmsnorm_layer(x, ypk.attach_input(nw, f"nw{i}"), tmp, (B, 1, 1), (128, 1, 1), eps=1e-6)
            ypk.linear_layer(tmp, ypk.attach_input(w, f"w{i}"), out, (64, 1, 1), (128, 1, 1))
            alg += H * H * 2 + 2 * B * H * 2 + H * 2
        name = f"RMSNorm->linear, X[{B},4096] fp16, W[4096,4096] (BASELINE configs[0]) x {reps} independent copies"
        dtype = "f16"
    elif workload == "gated_mlp":
        g.manual_seed(1)
        reps, H, I, dt = 6, 4096, 14336, torch.bfloat16
        ypk = pk(B)
        x = ypk.attach_input(rn((B, H), 1.0, dt), "x")
        alg = 0
        for i in range(reps):
            wg, wu, wd = rn((I, H), 0.02, dt), rn((I, H), 0.02, dt), rn((H, I), 0.02, dt)
            keep += [wg, wu, wd]
            wgu = ypk.shuffle_tensors([ypk.attach_input(wg, f"g{i}"), ypk.attach_input(wu, f"u{i}")], 0, 32, f"gu{i}")
            mid = ypk.new_tensor(dims=(B, 2 * I), name=f"mid{i}")
            act = ypk.new_tensor(dims=(B, I), name=f"act{i}")
            out = ypk.new_tensor(dims=(B, H), name=f"out{i}")
            ypk.linear_layer(x, wgu, mid, (64, 1, 1), (128, 1, 1))
            ypk.silu_mul_layer(mid, act, (32, 1, 1), (128, 1, 1))
            ypk.linear_layer(act, ypk.attach_input(wd, f"d{i}"), out, (64, 1, 1), (128, 1, 1))
            alg += 3 * I * H * 2 + B * (2 * H + I * 2) * 2
        name = f"SiLU-gated MLP, X[{B},4096] bf16, 4096x14336 (BASELINE configs[1]) x {reps} copies"
        dtype = "bf16"
    else:
        g.manual_seed(2)
        R, HQ, HKV, D, CTX, reps = 8, 32, 8, 128, 4096, 12
        B = R
        pages = (CTX + 1 + 63) // 64
        perm = torch.randperm(R * pages, generator=torch.Generator().manual_seed(2)).tolist()
        i32 = dict(dtype=torch.int32, device=dev)
        meta = {"qo_indptr_buffer": torch.arange(R + 1, **i32),
                "paged_kv_indptr_buffer": torch.arange(R + 1, **i32) * pages,
                "paged_kv_indices_buffer": torch.tensor(perm, **i32),
                "paged_kv_last_page_len_buffer": torch.full((R,), (CTX + 1 - 1) % 64 + 1, **i32)}
        ypk = pk(R, meta, max_req=R, max_pages=R * pages, max_seq=CTX + 1)
        from yirage_b200 import llama
        cos, sin = llama.rope_tables(llama.LlamaShape(), CTX + 64, dev)
        cos_t, sin_t = ypk.attach_input(cos, "cos"), ypk.attach_input(sin, "sin")
        qkv = ypk.attach_input(rn((R, (HQ + 2 * HKV) * D), 1.0, torch.bfloat16), "qkv")
        alg = 0
        for i in range(reps):
            kc, vc = rn((R * pages, 64, HKV, D), 1.0, torch.bfloat16), rn((R * pages, 64, HKV, D), 1.0, torch.bfloat16)
            keep += [kc, vc]
            out = ypk.new_tensor(dims=(R, HQ * D), name=f"o{i}")
            ypk.paged_attention_layer(qkv, ypk.attach_input(kc, f"k{i}"), ypk.attach_input(vc, f"v{i}"), None,
                                      None, cos_t, sin_t, out, (R, HKV, 1), (128, 1, 1))
            alg += R * CTX * HKV * D * 2 * 2
        name = (f"GQA decode attention, batch 8, 32q/8kv heads, ctx {CTX} in 64-token pages, random page "
                f"order (BASELINE configs[2]) x {reps} copies")
        dtype = "bf16"
    ypk.compile()
    for _ in range(W):
        ypk(batch=B)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    # one event pair per launch, recorded around the enqueue (the synchronous call would put
    # the host's wake-up and status read-back between the kernel's end and the second event)
    total = 0.0
    for _ in range(K):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        ypk.launch_async(batch=B)
        ev1.record()
        ypk.wait()
        total += ev0.elapsed_time(ev1)
    ms = total / K
    clocks = sampler.stop()
    hbm, src = peaks()
    achieved = alg / (ms / 1e3) / 1e9
    res = {"name": name, "dtype": dtype, "batch": B, "ms": ms, "us_per_operator": ms * 1e3 / reps,
           "alg": alg, "achieved": achieved, "frac": achieved / hbm, "src": src, "hbm": hbm,
           "clocks": clocks, "tensor_core_tasks": int(ypk.status().tensor_core_tasks)}
    ypk.finalize()
    del keep
    return res


def run_kernel_workload(args):
    B = args.batch if args.batch != 1 else 8
    r = measure_kernel(args.workload, B, args.steps, args.warmup)
    print(json.dumps({
        "metric": "task_kernel_hbm_gbs", "value": r["achieved"], "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": r["ms"],
        "us_per_operator": r["us_per_operator"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": r["dtype"], "data": "synthetic",
        "config": {"workload": r["name"], "batch": r["batch"],
                   "l2": f"{r['alg'] / 1e9:.2f} GB read per step, far larger than the 126 MB L2",
                   "note": "one cooperative launch per step; its launch latency is inside the time"},
        "roofline": {"bound": "hbm", "achieved": r["achieved"], "peak": r["hbm"], "unit": "GB/s",
                     "frac": r["frac"], "frac_of": f"{r['src']} copy bandwidth",
                     "algorithmic_bytes_per_step": r["alg"], "traffic": None},
        "tensor_core_tasks": r["tensor_core_tasks"],
        "clocks": r["clocks"], "gpu_launches": args.steps}), flush=True)


def run_timeline(args):
    """Per-operator device timeline of a decode iteration of the headline workload (first two
    layers and the tail): span = from the previous operator's last task to this one's, wait /
    exec = mean time a task waited for its dependency / ran, stage_in / stream / finish = the
    LINEAR phases (inputs staged, weights streamed, epilogue).  Microseconds."""
    from yirage_b200 import llama
    dist = _dist()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    B = args.batch
    MT = 8 if B <= 8 else 64
    shape = (llama.LlamaShape.qwen3_30b_a3b() if args.model == "qwen3-30b-a3b"
             else llama.LlamaShape.llama3_8b())
    if args.layers:
        shape.num_hidden_layers = args.layers
    max_seq = PROMPT_LEN + 12 * B + 64
    g = torch.Generator().manual_seed(SEED)
    tokens = torch.zeros(B, max_seq, dtype=torch.int64)
    tokens[:, :PROMPT_LEN] = torch.randint(0, shape.vocab_size, (B, PROMPT_LEN), generator=g)
    tokens = tokens.to(dev)
    plen = torch.full((B,), PROMPT_LEN, dtype=torch.int32, device=dev)
    weights = llama.init_weights(shape, dev, SEED, world_size=world, rank=rank)
    prof = torch.zeros(3000 * 128, dtype=torch.int64, device=dev)
    ypk, st = llama.build_decode_kernel(
        shape, weights, tokens=tokens, prompt_lengths=plen, max_num_batched_requests=B,
        max_num_batched_tokens=MT, max_num_pages=((max_seq + 63) // 64) * B, page_size=64,
        world_size=world, rank=rank, profiler_tensor=prof)
    ypk.set_pause_below(B)
    ypk()
    ypk.set_pause_below(0)
    ypk(max_iterations=8)
    torch.cuda.synchronize()
    rows = ypk.profile_summary()
    if rank == 0:
        print(f"# {args.model} decode, batch {B}, tp{world}, graph of {MT} token slots; microseconds")
        print("op  kind            tasks   span   wait   exec  stage_in stream finish")
        prev = 0.0
        per_layer = (len(rows) - 4) // shape.num_hidden_layers if shape.num_hidden_layers else 0
        for i, r in enumerate(rows):
            if 1 + per_layer <= i < 1 + 2 * per_layer or i >= len(rows) - 3 or i == 0:
                print(f"{r['op']:3d} {r['kind']:15s} {r['n']:5d} {(r['last_done'] - prev):6.1f} {r['wait']:6.1f} "
                      f"{r['exec']:6.1f} {r.get('stage_in', 0):8.1f} {r.get('stream', 0):6.1f} {r.get('finish', 0):6.1f}")
            prev = r["last_done"]
        print(f"iteration: {rows[-1]['last_done']:.1f}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse()
    if args.timeline:
        run_timeline(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload != "decode":
        run_kernel_workload(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
