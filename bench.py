"""Benchmark of the persistent-kernel decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[3]): random-init Llama-3-8B, bf16, batch 1, a 512-token
prompt of uniform-random ids, greedy decode; seed 3.  One "step" is one decode iteration
of the megakernel (one new token per sequence): the prompt is prefilled untimed, W decode
iterations warm up, then exactly K iterations are timed with CUDA events around one
persistent-kernel launch.  Prints one JSON line (rank 0).

 value      tokens/s over the K timed iterations, inputs resident in HBM
 e2e        tokens/s of a whole generation through PersistentKernel.__call__ with the
            prompt starting in pinned host memory and the generated ids read back to the
            host, prefill included in the time
 roofline   weight + KV bytes one iteration has to read / time per iteration, against the
            measured copy bandwidth in MEASURED_PEAKS.json
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

DRAM_TRAFFIC_RATIO = 0.998   # (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes, ncu, profiles/
PROMPT_LEN = 512
SEED = 3
FALLBACK_HBM_GBS = 6650.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (invalid as a result)")
    ap.add_argument("--workload", default="decode",
                    choices=["decode", "rmsnorm_linear", "gated_mlp", "attention"],
                    help="decode = BASELINE configs[3] (the headline); the others time one task "
                         "kernel on BASELINE configs[0..2] as a chain of independent copies")
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "llama3-70b"],
                    help="llama3-70b = BASELINE configs[4] (context 2048); needs --gpus >= 2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
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
    for i in range(min(K + W, 3)):
        t, desc = cpu_decode_sample(shape, PROMPT_LEN, budget_s=budget)
        per.append(t)
    t_tok = sorted(per)[len(per) // 2]
    val = args.batch / t_tok
    line = {
        "impl": "reference", "metric": "decode_tokens_per_second", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": t_tok * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "llama3-8b decode, batch 1, prompt 512 (BASELINE configs[3])",
                   "note": "CPU port of the reference's PyTorch model code; the reference's native "
                           "library cannot be built here and its model code needs a GPU"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": desc},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ our arm
def run_ours(args):
    import torch.distributed as dist
    from yirage_b200 import llama

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    K, W, B = args.steps, max(args.warmup, 3), args.batch
    global PROMPT_LEN
    big = args.model == "llama3-70b"
    shape = llama.LlamaShape.llama3_70b() if big else llama.LlamaShape.llama3_8b()
    if big:
        PROMPT_LEN = 2048      # BASELINE configs[4]: context 2048
        if world < 2:
            raise SystemExit("llama3-70b (140 GB of weights) is a tensor-parallel configuration: --gpus 2/4/8")
    if args.layers:
        shape.num_hidden_layers = args.layers
    # 8 prompt tokens per request and iteration: all requests prefill in lockstep and reach
    # the decode phase together (with fewer token slots the first requests would already be
    # hundreds of tokens into their generation when the last one finishes its prompt)
    MT = 8 * B
    max_seq = PROMPT_LEN + W + K + 2
    page = 64
    pages_per_req = (max_seq + page - 1) // page

    def fresh_tokens():
        g = torch.Generator().manual_seed(SEED)
        t = torch.zeros(B, max_seq, dtype=torch.int64)
        t[:, :PROMPT_LEN] = torch.randint(0, shape.vocab_size, (B, PROMPT_LEN), generator=g)
        return t

    host_tokens = fresh_tokens().pin_memory()
    host_plen = torch.full((B,), PROMPT_LEN, dtype=torch.int32).pin_memory()
    tokens = host_tokens.to(dev)
    plen = host_plen.to(dev)
    # N > 1: tensor parallelism over the N GPUs (column-split qkv / gate / up, row-split
    # o_proj / down_proj, in-kernel all-reduce over NVLink after each row-split projection;
    # lm_head split by vocabulary rows, arg-max winners exchanged).  The total work is fixed,
    # so the scaling is "strong".
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    weights = llama.init_weights(shape, dev, SEED, world_size=world, rank=rank)
    ypk, st = llama.build_decode_kernel(
        shape, weights, tokens=tokens, prompt_lengths=plen, max_num_batched_requests=B,
        max_num_batched_tokens=MT, max_num_pages=pages_per_req * B, page_size=page,
        world_size=world, rank=rank)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()

    # every request advances min(8, 32 / q-heads-per-kv-head) prompt tokens per iteration
    chunk = min(8, 32 // (shape.num_attention_heads // shape.num_key_value_heads))
    prefill_iters = (PROMPT_LEN + chunk - 1) // chunk

    def run_to_decode():
        """Prefill the prompts (untimed): iterate until every request is decoding."""
        ypk.reset()
        if prefill_iters is not None:
            ypk(max_iterations=prefill_iters)
        else:
            for _ in range(100000):
                ypk(max_iterations=1)
                if int(st["meta"]["step"].min()) >= PROMPT_LEN:
                    break

    if world > 1:
        dist.barrier()
    run_to_decode()
    ypk(max_iterations=W)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    step_before = st["meta"]["step"].clone()
    torch.cuda.synchronize()
    ev0.record()
    ypk(max_iterations=K)
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    done = int((st["meta"]["step"] - step_before).sum())
    assert done == K * B, f"timed region ran {done} token-steps, expected {K * B}"
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)

    # ---- end-to-end: whole generation through the public call, host buffers in and out
    e2e = None
    if not args.no_e2e:
        host_out = torch.empty_like(host_tokens).pin_memory()
        host_step = torch.empty(B, dtype=torch.int32).pin_memory()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        tokens.copy_(host_tokens, non_blocking=True)
        plen.copy_(host_plen, non_blocking=True)
        ypk.reset()
        ypk()
        host_out.copy_(tokens, non_blocking=True)
        host_step.copy_(st["meta"]["step"], non_blocking=True)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        gen = int((host_step.to(torch.int64) + 1 - PROMPT_LEN).sum())
        iters = int(ypk.status().iterations)
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t)
        h2d = host_tokens.numel() * 8 + host_plen.numel() * 4
        d2h = host_out.numel() * 8 + host_step.numel() * 4
        e2e = {"value": gen / dt, "unit": "tokens/s",
               "h2d_bytes_per_step": h2d / max(1, iters), "d2h_bytes_per_step": d2h / max(1, iters),
               "note": f"{gen} generated tokens, {iters} iterations incl. chunked prefill of the "
                       f"{PROMPT_LEN}-token prompt, host->device prompt copy and device->host token read-back inside the time"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    hbm, src = peaks()
    vpad = llama.padded_vocab(shape.vocab_size)
    # per GPU: its shard of every weight (the lm_head by vocabulary rows) + its kv heads
    wbytes = shape.decode_weight_bytes(1, vpad) / world
    ctx_mid = PROMPT_LEN + W + K / 2.0
    kv_bytes = B * ctx_mid * shape.num_hidden_layers * shape.num_key_value_heads * shape.head_dim * 2 * 2 / world
    alg = wbytes + kv_bytes
    per_iter_s = ms / 1e3 / K
    achieved = alg / per_iter_s / 1e9
    line = {
        "metric": "decode_tokens_per_second", "value": K * B / (ms / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
        "us_per_token": ms * 1e3 / K / B,
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.model} decode, batch {B}, prompt {PROMPT_LEN}, greedy "
                               f"(BASELINE configs[{4 if big else 3}])",
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
                     "traffic_note": "scaled from the ncu capture of the 4-layer case (ratio 0.998), per launch of K iterations",
                     "kernel": "ypk_megakernel (one launch covers all K iterations)"},
        "clocks": clocks,
        "gpu_launches": 1,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if not args.no_cpu_baseline:
        t_tok, desc = cpu_decode_sample(shape, PROMPT_LEN, budget_s=15.0)
        line["cpu_baseline"] = {"value": 1.0 / t_tok, "unit": "tokens/s", "cores": os.cpu_count(),
                                "kind": "port", "sample": desc}
    print(json.dumps(line), flush=True)
    ypk.finalize()
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------ task-kernel workloads
def run_kernel_workload(args):
    """BASELINE configs[0..2] on one GPU.  One launch of a few microseconds cannot be timed
    from the host, so a step is a chain of `reps` independent copies of the operator (own
    weights / own KV cache each, several GB in total, far beyond L2) executed by one
    persistent-kernel launch; the figure is bytes the chain has to read / time."""
    import yirage_b200 as yr
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    K, W, B = args.steps, max(args.warmup, 3), args.batch
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
    if args.workload == "rmsnorm_linear":
        g.manual_seed(0)
        B = B if args.batch != 1 else 8
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
        name = f"RMSNorm->linear, X[{B},4096] fp16, W[4096,4096] (BASELINE configs[0]) x {reps} copies"
        dtype = "f16"
    elif args.workload == "gated_mlp":
        g.manual_seed(1)
        B = B if args.batch != 1 else 8
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
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(K):
        ypk(batch=B)
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / K
    clocks = sampler.stop()
    hbm, src = peaks()
    achieved = alg / (ms / 1e3) / 1e9
    print(json.dumps({
        "metric": "task_kernel_hbm_gbs", "value": achieved, "unit": "GB/s", "n_gpus": 1, "steps": K,
        "warmup": W, "ms_per_step": ms, "us_per_operator": ms * 1e3 / reps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": name, "batch": B,
                   "l2": f"{alg / 1e9:.2f} GB read per step, far larger than the 126 MB L2",
                   "note": "launch overhead of one cooperative launch per step is inside the time"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                     "frac": achieved / hbm, "frac_of": f"{src} copy bandwidth",
                     "algorithmic_bytes_per_step": alg, "traffic": None},
        "clocks": clocks, "gpu_launches": K}), flush=True)
    ypk.finalize()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload != "decode":
        run_kernel_workload(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
