"""Llama-style decode graph on the PersistentKernel surface, plus synthetic weights.

build_decode_kernel() issues the same sequence of PersistentKernel calls as the
reference demo does for a Llama-3 model (demo/llama3/demo.py:325-349 attach inputs,
:351-465 intermediate tensors, :472-484 embedding, :487-684 one transformer layer,
:687-747 final norm / lm_head / arg-max, :750-812 compile), but takes plain tensors
instead of a Hugging Face module so that random-init models of any Llama shape can be
built directly on the GPU (the 70B-shaped configuration never exists on the host).
"""
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from . import core
from .persistent_kernel import PersistentKernel


@dataclass
class LlamaShape:
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    qk_norm: bool = False          # RMSNorm of q and k heads inside attention (Qwen3)
    num_experts: int = 0           # > 0: every MLP is a mixture of experts (Qwen3-MoE), whose
    experts_per_token: int = 0     # experts have intermediate_size columns each

    @staticmethod
    def llama3_8b():
        return LlamaShape()

    @staticmethod
    def qwen3_8b():
        """Dense Qwen3-8B: the Llama graph plus q/k RMSNorm in attention
        (demo/qwen3/demo.py:402-575)."""
        return LlamaShape(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                          num_attention_heads=32, num_key_value_heads=8, vocab_size=151936,
                          rms_norm_eps=1e-6, rope_theta=1000000.0, qk_norm=True)

    @staticmethod
    def qwen3_30b_a3b():
        """Qwen3-30B-A3B: 128 experts of 768 columns, 8 per token (demo/qwen3/demo_30B_A3B.py)."""
        return LlamaShape(hidden_size=2048, intermediate_size=768, num_hidden_layers=48,
                          num_attention_heads=32, num_key_value_heads=4, vocab_size=151936,
                          rms_norm_eps=1e-6, rope_theta=1000000.0, qk_norm=True, num_experts=128,
                          experts_per_token=8)

    @staticmethod
    def llama3_70b():
        return LlamaShape(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                          num_attention_heads=64, num_key_value_heads=8)

    def decode_weight_bytes(self, world_size=1, padded_vocab=None):
        """bf16 bytes of weights one rank streams per decode step (norm weights ignored)."""
        h, f = self.hidden_size, self.intermediate_size
        qkv = (self.num_attention_heads + 2 * self.num_key_value_heads) * self.head_dim * h
        o = self.num_attention_heads * self.head_dim * h
        mlp = 3 * f * h
        if self.num_experts:     # the router and the experts one token selects
            mlp = self.num_experts * h + self.experts_per_token * 3 * f * h
        per_layer = (qkv + o + mlp) // world_size
        v = padded_vocab or self.vocab_size
        return 2 * (self.num_hidden_layers * per_layer + v * h)


def padded_vocab(vocab_size: int) -> int:
    """The demo pads the lm_head to a multiple of 2048 rows (demo/llama3/demo.py:208)."""
    return (vocab_size + 2047) // 2048 * 2048


def rope_tables(shape: LlamaShape, max_pos: int, device):
    """bf16 cos/sin [max_pos, head_dim]: fp32 angles, half table repeated
    (demo/llama3/models/modeling_llama3.py:71-89)."""
    d = shape.head_dim
    inv_freq = 1.0 / (shape.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64,
                                                        device=device).float() / d))
    pos = torch.arange(max_pos, dtype=torch.float32, device=device)
    emb = torch.cat((pos[:, None] * inv_freq[None, :],) * 2, dim=-1)
    return emb.cos().to(torch.bfloat16).contiguous(), emb.sin().to(torch.bfloat16).contiguous()


def init_weights(shape: LlamaShape, device, seed: int, world_size: int = 1, rank: int = 0,
                 std: float = 0.02, dtype=torch.bfloat16) -> Dict:
    """Random-init weights ~N(0, std) (norm weights 1), already sharded for `rank`:
    q/k/v/gate/up split by output rows, o/down split by input columns
    (modeling_llama3.py:98-100,174-185).  Every rank draws the full tensor from the same
    seeded generator and keeps its slice, so the shards of all ranks form one model."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def full(rows, cols):
        return torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32).mul_(std).to(dtype)

    def rows_shard(t):
        n = t.shape[0] // world_size
        return t[rank * n:(rank + 1) * n].contiguous()

    def cols_shard(t):
        n = t.shape[1] // world_size
        return t[:, rank * n:(rank + 1) * n].contiguous()

    h, f, d = shape.hidden_size, shape.intermediate_size, shape.head_dim
    hq, hkv = shape.num_attention_heads, shape.num_key_value_heads
    w = {"embed": full(shape.vocab_size, h), "layers": []}
    for _ in range(shape.num_hidden_layers):
        L = {
            "input_norm": torch.ones(h, device=device, dtype=dtype),
            "q": rows_shard(full(hq * d, h)),
            "k": rows_shard(full(hkv * d, h)),
            "v": rows_shard(full(hkv * d, h)),
            "o": cols_shard(full(h, hq * d)),
            "post_norm": torch.ones(h, device=device, dtype=dtype),
        }
        if shape.num_experts:
            if world_size != 1:
                raise NotImplementedError("mixture-of-experts weights are built for one GPU")
            E = shape.num_experts
            L["moe_gate"] = full(E, h)
            # experts stacked as the demo does: [gate rows; up rows] per expert, then down
            L["w13"] = torch.stack([full(2 * f, h) for _ in range(E)])
            L["w2"] = torch.stack([full(h, f) for _ in range(E)])
        else:
            L.update(gate=rows_shard(full(f, h)), up=rows_shard(full(f, h)),
                     down=cols_shard(full(h, f)))
        if shape.qk_norm:
            L["q_norm"] = (1.0 + 0.1 * torch.randn(d, generator=g, device=device)).to(dtype)
            L["k_norm"] = (1.0 + 0.1 * torch.randn(d, generator=g, device=device)).to(dtype)
        w["layers"].append(L)
    w["final_norm"] = torch.ones(h, device=device, dtype=dtype)
    w["lm_head"] = full(shape.vocab_size, h)
    return w


def _divisor(n: int, want: int) -> int:
    """Largest divisor of n that is <= want (grid hints must divide the tiled dimension)."""
    return max(g for g in range(1, max(1, want) + 1) if n % g == 0)


def _gate_up_groups(rows: int) -> int:
    """Number of (gate|up) groups the demo asks shuffle_tensors for: half the task count
    its grid heuristic picks for the fused gate/up projection (demo/llama3/demo.py:120-130,
    617-624).  Only the layout of an unfused mlp_mid depends on it."""
    size = 2 * rows
    if size / 96 > 400 and size % 256 == 0:
        return size // 256 // 2
    for grid in (96, 80, 64, 48):
        if size % grid == 0 and (size // grid >= 128 or size // grid == 64):
            return max(1, grid // 2)
    return 1


def build_decode_kernel(shape: LlamaShape, weights: Dict, *, tokens: torch.Tensor,
                        prompt_lengths: torch.Tensor, max_num_batched_requests: int,
                        max_num_batched_tokens: int, max_num_pages: int, page_size: int,
                        eos_token_id: int = -1, world_size: int = 1, rank: int = 0,
                        num_workers: int = 128, use_model_eps: bool = True,
                        k_cache: Optional[torch.Tensor] = None,
                        v_cache: Optional[torch.Tensor] = None, compile: bool = True,
                        dry_run: bool = False, profiler_tensor: Optional[torch.Tensor] = None, handoff: Optional[str] = None,
                        vocab_parallel: Optional[bool] = None, defer_connect: bool = False,
                        meta: Optional[Dict] = None, spec_decode_config=None):
    """Build (and compile) the decode megakernel for `weights`.  Returns (ypk, state) where
    state holds the meta tensors, caches and rope tables the kernel works on.  `meta`, `k_cache`
    and `v_cache` of an earlier build may be passed in: the two kernels then serve the same
    requests (PersistentKernel.adopt); the token buffers of `meta` must hold at least
    max_num_batched_tokens entries.  `spec_decode_config` (speculative.PromptLookupConfig)
    adds the prompt-lookup draft and verification operators the way demo/qwen3/demo.py:377-384,
    457-470,625-632 does."""
    dev = tokens.device
    total_requests, max_seq_length = tokens.shape
    h, d = shape.hidden_size, shape.head_dim
    hq, hkv = shape.num_attention_heads // world_size, shape.num_key_value_heads // world_size
    inter = shape.intermediate_size // world_size
    vpad = padded_vocab(shape.vocab_size)
    MT, MR = max_num_batched_tokens, max_num_batched_requests
    i32 = dict(dtype=torch.int32, device=dev)
    if meta is not None:
        # same memory, this graph's token budget
        meta = dict(meta, input_tokens=meta["input_tokens"][:MT],
                    output_tokens=meta["output_tokens"][:MT])
    else:
        meta = {
            "step": torch.zeros(total_requests, **i32),
            "tokens": tokens,
            "input_tokens": torch.zeros(MT, 1, dtype=torch.int64, device=dev),
            "output_tokens": torch.zeros(MT, 1, dtype=torch.int64, device=dev),
            "num_new_tokens": torch.ones(total_requests, **i32),
            "prompt_lengths": prompt_lengths,
            "qo_indptr_buffer": torch.zeros(MR + 1, **i32),
            "paged_kv_indptr_buffer": torch.zeros(MR + 1, **i32),
            "paged_kv_indices_buffer": torch.zeros(max_num_pages, **i32),
            "paged_kv_last_page_len_buffer": torch.zeros(MR, **i32),
        }
    if k_cache is None:
        k_cache = torch.zeros(shape.num_hidden_layers, max_num_pages, page_size, hkv, d,
                              dtype=torch.bfloat16, device=dev)
        v_cache = torch.zeros_like(k_cache)
    cos, sin = rope_tables(shape, max(max_seq_length, 64), dev)
    lm_head = torch.cat((weights["lm_head"],
                         torch.zeros(vpad - shape.vocab_size, h, dtype=torch.bfloat16, device=dev)), 0)
    # Tensor parallelism: every rank keeps one slice of the vocabulary rows and the ranks
    # exchange their arg-max winners (vocab_parallel=False replicates the lm_head instead).
    if vocab_parallel is None:
        vocab_parallel = world_size > 1
    vocab_parallel = bool(vocab_parallel) and world_size > 1
    vslice = vpad // world_size if vocab_parallel else vpad
    if vocab_parallel:
        if vpad % world_size or vslice % num_workers:
            raise ValueError("the padded vocabulary does not split evenly over the ranks and workers")
        lm_head = lm_head[rank * vslice:(rank + 1) * vslice].contiguous()

    ypk = PersistentKernel(
        mode="offline", world_size=world_size, mpi_rank=rank, num_workers=num_workers,
        num_local_schedulers=0, num_remote_schedulers=0, max_seq_length=max_seq_length,
        max_num_batched_requests=MR, max_num_batched_tokens=MT, max_num_pages=max_num_pages,
        page_size=page_size, eos_token_id=eos_token_id, meta_tensors=meta,
        profiler_tensor=profiler_tensor, trace_name="", spec_decode_config=spec_decode_config,
        use_cutlass_kernel=True)
    if handoff is not None:
        ypk.handoff = handoff   # "event" | "ll" | "auto" (see lowering.lower)
    if use_model_eps:
        ypk.rms_norm_eps = shape.rms_norm_eps

    x_tok = ypk.attach_input(meta["input_tokens"], name="input_token")
    spec_tokens = None
    if spec_decode_config is not None:
        all_tokens = ypk.attach_input(meta["tokens"], name="all_tokens")
        spec_tokens = ypk.draft_forward_layer_dispatcher(
            spec_decode_config=spec_decode_config, tokens=all_tokens, grid_dim=(96, 1, 1),
            block_dim=(128, 1, 1))
        x_tok = spec_tokens
    cos_t = ypk.attach_input(cos, name="cos_position_embedding")
    sin_t = ypk.attach_input(sin, name="sin_position_embedding")
    embed_w = ypk.attach_input(weights["embed"], name="embed_tokens")

    def tmp(name, cols, dt=core.bfloat16, shared=False):
        return ypk.new_tensor(dims=(MT, cols), dtype=dt, name=name,
                              io_category="nvshmem_tensor" if shared and world_size > 1 else "cuda_tensor")

    embed_out = tmp("embed_out", h)
    rmsnorm_out = tmp("rmsnorm_out", h)
    attn_in = tmp("attn_in", (hq + 2 * hkv) * d)
    attn_out = tmp("attn_out", hq * d)
    attn_proj_out = tmp("attn_proj_out", h, shared=True)
    allreduce_buf = ypk.new_tensor(dims=(world_size, MT, h), dtype=core.bfloat16,
                                   name="all_reduce_buf",
                                   io_category="nvshmem_tensor" if world_size > 1 else "cuda_tensor")
    attn_allreduce_out = tmp("attn_allreduce_out", h, shared=True)
    mlp_mid = tmp("mlp_mid", 2 * inter)
    silu_mul_out = tmp("silu_mul_out", inter)
    mlp_out = tmp("mlp_out", h, shared=True)
    mlp_final = tmp("mlp_final", h, shared=True)
    argmax_in = tmp("argmax_in", vslice)
    argmax_part_value = tmp("argmax_part_value", num_workers)
    argmax_part_index = tmp("argmax_part_index", num_workers, dt=core.int64)
    argmax_out = ypk.attach_input(meta["output_tokens"], name="output_token")

    ypk.embed_layer(input=x_tok, weight=embed_w, output=embed_out, grid_dim=(1, 1, 1),
                    block_dim=(128, 1, 1), input_source=1)
    x = embed_out
    moe = None
    for li, L in enumerate(weights["layers"]):
        w_norm = ypk.attach_input(L["input_norm"], name=f"layer_{li}_input_layernorm")
        w_q = ypk.attach_input(L["q"], name=f"layer_{li}_q_proj")
        w_k = ypk.attach_input(L["k"], name=f"layer_{li}_k_proj")
        w_v = ypk.attach_input(L["v"], name=f"layer_{li}_v_proj")
        w_qkv = ypk.shuffle_tensors(inputs=[w_q, w_k, w_v], shuffled_dim=0, num_groups=hkv,
                                    name=f"layer_{li}_qkv_proj")
        ypk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(MT, 1, 1),
                          block_dim=(128, 1, 1))
        ypk.linear_layer(input=rmsnorm_out, weight=w_qkv, output=attn_in,
                         grid_dim=(_divisor(w_qkv.dims[0], 96), 1, 1),
                         block_dim=(128, 1, 1))
        kc = ypk.attach_input(k_cache[li], name=f"layer_{li}_k_cache")
        vc = ypk.attach_input(v_cache[li], name=f"layer_{li}_v_cache")
        qn = kn = None
        if "q_norm" in L:
            qn = ypk.attach_input(L["q_norm"], name=f"layer_{li}_q_norm")
            kn = ypk.attach_input(L["k_norm"], name=f"layer_{li}_k_norm")
        attention = (ypk.single_batch_extend_attention_layer if spec_decode_config is not None
                     else ypk.paged_attention_layer)
        attention(input=attn_in, k_cache=kc, v_cache=vc, q_norm=qn, k_norm=kn,
                  cos_pos_embed=cos_t, sin_pos_embed=sin_t, output=attn_out,
                  grid_dim=(MR, hkv, 1), block_dim=(128, 1, 1))
        w_o = ypk.attach_input(L["o"], name=f"layer_{li}_o_proj")
        ypk.linear_with_residual_layer(input=attn_out, weight=w_o, residual=x, output=attn_proj_out,
                                       grid_dim=(h // 64, 1, 1), block_dim=(128, 1, 1))
        x = attn_proj_out
        if world_size > 1:
            ypk.allreduce_layer(input=attn_proj_out, buffer=allreduce_buf, output=attn_allreduce_out,
                                grid_dim=(h // 64, 1, 1), block_dim=(128, 1, 1))
            x = attn_allreduce_out
        w_norm2 = ypk.attach_input(L["post_norm"], name=f"layer_{li}_post_attn_layernorm")
        if "moe_gate" in L:
            # demo/qwen3/demo_30B_A3B.py:564-645
            E, topk = shape.num_experts, shape.experts_per_token
            if moe is None:
                moe = {
                    "gate_out": tmp("moe_gate_out", E),
                    "routing": ypk.new_tensor(dims=(E, MT), dtype=core.int32, name="moe_routing_indices"),
                    "mask": ypk.new_tensor(dims=(E + 1,), dtype=core.int32, name="moe_mask"),
                    "topk_weight": ypk.new_tensor(dims=(MT, topk), dtype=core.float32, name="moe_topk_weight"),
                    "mid": ypk.new_tensor(dims=(MT, topk, 2 * inter), dtype=core.bfloat16, name="moe_mlp_mid"),
                    "act": ypk.new_tensor(dims=(MT, topk, inter), dtype=core.bfloat16, name="moe_silu_mul_out"),
                    "out": ypk.new_tensor(dims=(MT, topk, h), dtype=core.bfloat16, name="moe_mlp_out"),
                }
            w_router = ypk.attach_input(L["moe_gate"], name=f"layer_{li}_moe_gate")
            w13 = ypk.attach_input(L["w13"], name=f"layer_{li}_gateup_proj")
            w2 = ypk.attach_input(L["w2"], name=f"layer_{li}_down_proj")
            ypk.rmsnorm_layer(input=x, weight=w_norm2, output=rmsnorm_out, grid_dim=(MT, 1, 1),
                              block_dim=(128, 1, 1))
            ypk.linear_layer(input=rmsnorm_out, weight=w_router, output=moe["gate_out"],
                             grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
            ypk.moe_topk_softmax_routing_layer(
                input=moe["gate_out"], output=(moe["topk_weight"], moe["routing"], moe["mask"]),
                grid_dim=(1, 1, 1), block_dim=(256, 1, 1))
            ypk.moe_w13_linear_layer(input=rmsnorm_out, weight=w13, moe_routing_indices=moe["routing"],
                                     moe_mask=moe["mask"], output=moe["mid"], grid_dim=(1, _divisor(2 * inter, 12), 1),
                                     block_dim=(256, 1, 1))
            ypk.moe_silu_mul_layer(input=moe["mid"], output=moe["act"], grid_dim=(MT, topk, 1),
                                   block_dim=(256, 1, 1))
            ypk.moe_w2_linear_layer(input=moe["act"], weight=w2, moe_routing_indices=moe["routing"],
                                    moe_mask=moe["mask"], output=moe["out"], grid_dim=(1, _divisor(h, 16), 1),
                                    block_dim=(256, 1, 1))
            ypk.moe_mul_sum_add_layer(input=moe["out"], weight=moe["topk_weight"], residual=x,
                                      output=mlp_out, grid_dim=(MT, max(1, h // 256), 1),
                                      block_dim=(256, 1, 1))
            x = mlp_out
            continue
        w_gate = ypk.attach_input(L["gate"], name=f"layer_{li}_gate_proj")
        w_up = ypk.attach_input(L["up"], name=f"layer_{li}_up_proj")
        groups = _gate_up_groups(inter)
        w_gu = ypk.shuffle_tensors(inputs=[w_gate, w_up], shuffled_dim=0, num_groups=groups,
                                   name=f"layer_{li}_gatedup_proj")
        ypk.rmsnorm_layer(input=x, weight=w_norm2, output=rmsnorm_out, grid_dim=(MT, 1, 1),
                          block_dim=(128, 1, 1))
        ypk.linear_layer(input=rmsnorm_out, weight=w_gu, output=mlp_mid,
                         grid_dim=(2 * groups, 1, 1), block_dim=(128, 1, 1))
        ypk.silu_mul_layer(input=mlp_mid, output=silu_mul_out, grid_dim=(groups, 1, 1),
                           block_dim=(128, 1, 1))
        w_down = ypk.attach_input(L["down"], name=f"layer_{li}_down_proj")
        ypk.linear_with_residual_layer(input=silu_mul_out, weight=w_down, residual=x,
                                       output=mlp_out, grid_dim=(h // 64, 1, 1),
                                       block_dim=(128, 1, 1))
        x = mlp_out
        if world_size > 1:
            ypk.allreduce_layer(input=mlp_out, buffer=allreduce_buf, output=mlp_final,
                                grid_dim=(h // 64, 1, 1), block_dim=(128, 1, 1))
            x = mlp_final
    w_fn = ypk.attach_input(weights["final_norm"], name="model_norm_weight")
    w_lm = ypk.attach_input(lm_head, name="lm_head")
    ypk.rmsnorm_layer(input=x, weight=w_fn, output=rmsnorm_out, grid_dim=(MT, 1, 1),
                      block_dim=(128, 1, 1))
    ypk.linear_layer(input=rmsnorm_out, weight=w_lm, output=argmax_in,
                     grid_dim=(vslice // 256 if vslice % 256 == 0 else 1, 1, 1), block_dim=(128, 1, 1))
    # real vocabulary columns of this rank's logits (the lm_head is padded with zero rows,
    # whose logit 0.0 would win whenever every real logit is negative)
    v0 = rank * vslice if vocab_parallel else 0
    valid = max(0, min(vslice, shape.vocab_size - v0))
    ypk.argmax_partial_layer(input=argmax_in, output=(argmax_part_value, argmax_part_index),
                             grid_dim=(num_workers, 1, 1), block_dim=(128, 1, 1),
                             valid_cols=valid if valid > 0 else -1)
    ypk.argmax_reduce_layer(input=(argmax_part_value, argmax_part_index), output=argmax_out,
                            grid_dim=(1, 1, 1), block_dim=(128, 1, 1),
                            vocab_offset=rank * vslice if vocab_parallel else 0, exchange=vocab_parallel)
    if spec_decode_config is not None:
        ypk.verify_layer_dispatcher(spec_decode_config=spec_decode_config, spec_tokens=spec_tokens,
                                    target_output=argmax_out, grid_dim=(1, 1, 1),
                                    block_dim=(128, 1, 1))
    state = {"meta": meta, "k_cache": k_cache, "v_cache": v_cache, "cos": cos, "sin": sin,
             "lm_head": lm_head, "vocab_slice": (rank * vslice if vocab_parallel else 0, vslice),
             "tensors": {"argmax_in": argmax_in, "attn_out": attn_out}}
    if compile:
        # defer_connect: the caller exchanges the ranks' arena handles itself
        # (tensor_parallel.connect), e.g. after checking that every rank could build
        ypk.compile(dry_run=dry_run, defer_connect=defer_connect)
    return ypk, state


class PrefillDecodePair:
    """Two megakernels over one set of requests, K/V caches and meta tensors: `prefill` is
    built for `prefill_tokens` tokens per iteration (a request brings up to 64 new tokens,
    the LINEAR operators run on the tensor-core path), `decode` for at most 8 (flagged-word
    hand-off, GEMV path).  The reference runs prompts and decoding on one graph sized by
    max_num_batched_tokens (persistent_kernel.cuh:231-239); here the task kernels of the two
    regimes differ, so a run starts on `prefill`, which stops once the batcher forms a batch
    of at most 8 tokens, and `decode` takes the requests over from there.

    run() is the offline mode of the reference's launch_func: until every request has retired."""

    def __init__(self, prefill: PersistentKernel, decode: PersistentKernel, state: Dict,
                 decode_tokens: int):
        self.prefill, self.decode, self.state = prefill, decode, state
        self.decode_tokens = decode_tokens
        self.prefill.set_pause_below(decode_tokens)

    def reset(self):
        self.prefill.reset()
        self.decode.reset()

    def run(self, stream=None, max_iterations: int = 0):
        """Prompts on the wide graph, the rest on the narrow one.  Returns the iterations each
        ran.  `max_iterations` bounds the decode graph's launch (0: to the end)."""
        self.prefill(stream=stream)
        it_p = int(self.prefill.status().iterations)
        self.decode.adopt(self.prefill)
        self.decode(stream=stream, max_iterations=max_iterations)
        return it_p, int(self.decode.status().iterations)

    def finalize(self):
        self.prefill.finalize()
        self.decode.finalize()


def build_prefill_decode_pair(shape: LlamaShape, weights: Dict, *, tokens: torch.Tensor,
                              prompt_lengths: torch.Tensor, max_num_batched_requests: int,
                              max_num_pages: int, page_size: int, prefill_tokens: int = 64,
                              decode_tokens: int = 8, **kw) -> PrefillDecodePair:
    """build_decode_kernel twice over shared meta tensors and caches.  Under tensor
    parallelism every rank builds both graphs in this order (compile() exchanges the arena
    handles of each) and the ranks call run() together."""
    if not (decode_tokens <= 8 < prefill_tokens <= 64):
        raise ValueError("decode_tokens <= 8 < prefill_tokens <= 64")
    common = dict(tokens=tokens, prompt_lengths=prompt_lengths,
                  max_num_batched_requests=max_num_batched_requests,
                  max_num_pages=max_num_pages, page_size=page_size, **kw)
    pre, st = build_decode_kernel(shape, weights, max_num_batched_tokens=prefill_tokens, **common)
    dec, st2 = build_decode_kernel(shape, weights, max_num_batched_tokens=decode_tokens,
                                   meta=st["meta"], k_cache=st["k_cache"], v_cache=st["v_cache"],
                                   **common)
    st = dict(st, decode_tensors=st2["tensors"])
    return PrefillDecodePair(pre, dec, st, decode_tokens)
