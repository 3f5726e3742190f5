"""PersistentKernel: the Python front of the megakernel, same surface as the reference's
python/yirage/persistent_kernel.py:217-1347 (constructor, attach_input / new_tensor /
shuffle_tensors, the layer builders, compile, __call__, finalize).

What changed underneath: compile() does not generate and nvcc-compile a .cu per model; it
lowers the registered layers to a task table (lowering.py), hands tensors and tasks to the
prebuilt sm_100a library through the C ABI (include/ypk.h) and keeps the handle.
grid_dim / block_dim arguments of the builders are accepted as hints only.
"""
import ctypes as C
import os
import sys
from typing import Optional

import torch

from . import _native as N
from . import lowering
from .core import (CyKNGraph, CyTBGraph, DTensor, bfloat16, convert_torch_type_to_dtype, dtype,
                   int32, int64)
from .kernel import KNGraph
from .speculative import SpecDecodeConfig
from .threadblock import TBGraph

valid_persistent_kernel_modes = ("offline", "online", "onepass")

_META_KEYS = ("step", "tokens", "input_tokens", "output_tokens", "num_new_tokens",
              "prompt_lengths", "qo_indptr_buffer", "paged_kv_indptr_buffer",
              "paged_kv_indices_buffer", "paged_kv_last_page_len_buffer")


def _device_cc():
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(torch.cuda.current_device())
        return p.major * 10 + p.minor
    return 100  # graphs can be built and lowered without a GPU; they target sm_100a


class PersistentKernel:
    def __init__(
        self,
        mode: str,
        world_size: int,
        mpi_rank: int,
        num_workers: int,
        num_local_schedulers: int,
        num_remote_schedulers: int,
        max_seq_length: int,
        max_num_batched_requests: int,
        max_num_batched_tokens: int,
        max_num_pages: int,
        page_size: int,
        eos_token_id: int,
        meta_tensors: dict,
        profiler_tensor: Optional[torch.Tensor] = None,
        trace_name: str = "",
        spec_decode_config: Optional[SpecDecodeConfig] = None,
        use_cutlass_kernel: bool = True,
    ):
        self.__finalized__ = False
        self._is_compiled = False
        if mode not in valid_persistent_kernel_modes:
            raise ValueError(f"Invalid persistent kernel mode: {mode}")
        # "online" is the reference's one-request mode (MODE_ONLINE batcher,
        # persistent_kernel.cuh:325-352: step[0] advances by num_new_tokens[0] per iteration until
        # max_seq_length or EOS).  The on-device batcher here does the same for its one slot, so
        # online mode is the offline path with exactly one request; the caller may preset
        # step[0] after reset() to continue a sequence whose first tokens are already cached.
        self.online = mode == "online"
        if self.online:
            if max_num_batched_requests != 1 or meta_tensors["tokens"].shape[0] != 1:
                raise ValueError("online mode serves one request: max_num_batched_requests and "
                                 "tokens.shape[0] must be 1")
            mode = "offline"
        self.mode = mode
        self.world_size = world_size
        self.mpi_rank = mpi_rank
        self.num_workers = num_workers
        self.num_local_schedulers = num_local_schedulers
        self.num_remote_schedulers = num_remote_schedulers
        self.max_seq_length = max_seq_length
        self.max_num_batched_requests = max_num_batched_requests
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_num_pages = max_num_pages
        self.page_size = page_size
        self.eos_token_id = eos_token_id
        self.kn_graph = KNGraph(CyKNGraph(disable_fingerprint=True))
        self.kn_graph._task_graph_hook = self._generate_task_graph
        self.meta_tensors = meta_tensors
        self.profiler_tensor = profiler_tensor
        self.trace_name = trace_name
        self.use_nvshmem = world_size > 1
        self.spec_decode_config = spec_decode_config
        self.use_cutlass_kernel = use_cutlass_kernel
        self._spec_decode_handlers = {"promptlookup": self.prompt_lookup_spec_handler}
        self._spec_verify_handlers = {"promptlookup": self.prompt_lookup_verify_handler}
        # The reference's rmsnorm task hard-codes eps = 1e-6 (task_register.cc:1186); that
        # stays the default so unchanged callers see the same numbers.  Set this attribute
        # (or pass eps= to rmsnorm_layer) to use the model's own epsilon.
        self.rms_norm_eps = 1e-6
        self.target_cc = _device_cc()
        self._handle = None
        self._lowered = None
        self.init_func = self.launch_func = self.finalize_func = None
        if mode == "offline":
            self.total_num_requests = meta_tensors["tokens"].shape[0]
            assert self.max_seq_length == meta_tensors["tokens"].shape[1]
            assert meta_tensors["qo_indptr_buffer"].shape == (max_num_batched_requests + 1,)
            assert meta_tensors["paged_kv_indptr_buffer"].shape == (max_num_batched_requests + 1,)
            assert meta_tensors["paged_kv_indices_buffer"].shape == (max_num_pages,)
            assert meta_tensors["paged_kv_last_page_len_buffer"].shape == (max_num_batched_requests,)
        else:
            self.total_num_requests = 0

    # ------------------------------------------------------------------ tensors
    def attach_input(self, torch_tensor: torch.Tensor, name: str = None) -> DTensor:
        dims = tuple(d for d in torch_tensor.shape)
        strides = tuple(s for s in torch_tensor.stride())
        for d in range(len(dims) - 1):
            assert strides[d] == strides[d + 1] * dims[d + 1], "attach_input wants row-major"
        dt = convert_torch_type_to_dtype(torch_tensor.dtype)
        t = self.kn_graph.new_input(dims=dims, strides=strides, dtype=dt)
        assert name is not None
        self.kn_graph.attach_torch_tensor(t, torch_tensor, name)
        return t

    def new_tensor(self, dims: tuple, strides: tuple = None, dtype: dtype = bfloat16,
                   name: str = None, io_category: str = "cuda_tensor") -> DTensor:
        if strides is not None:
            for d in range(len(dims) - 1):
                assert strides[d] == strides[d + 1] * dims[d + 1]
        t = self.kn_graph.new_input(dims=dims, strides=strides, dtype=dtype)
        assert name is not None
        if io_category == "cuda_tensor":
            self.kn_graph.attach_cuda_tensor(t, name)
        elif io_category == "nvshmem_tensor":
            self.kn_graph.attach_nvshmem_tensor(t, name)
        else:
            raise RuntimeError(f"Invalid io_category: {io_category}")
        return t

    def fuse_tensors(self, inputs, fused_dim: int, num_groups: int, name: str = None):
        assert fused_dim == 0
        return self.kn_graph.fuse_tensors(inputs, fused_dim, num_groups, name)

    def shuffle_tensors(self, inputs, shuffled_dim: int, num_groups: int, name: str = None):
        assert shuffled_dim == 0
        return self.kn_graph.shuffle_tensors(inputs, shuffled_dim, num_groups, name)

    # ------------------------------------------------------------------ layer builders
    def _register(self, name, operands_maps, grid_dim, block_dim, params=None, **attrs):
        tb = TBGraph(CyTBGraph(grid_dim, block_dim, 1, 64))
        for t, imap, fdim in operands_maps:
            tb.new_input(t, imap, fdim, True)
        self.kn_graph.customized([t for t, _, _ in operands_maps], tb)
        self.kn_graph.register_task(tb, name, params, **attrs)

    def embed_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple,
                    block_dim: tuple, input_source: int = 0):
        self._register("embedding", [(input, (-1, 1, -1), -1), (weight, (1, -1, -1), -1),
                                     (output, (1, 0, -1), -1)], grid_dim, block_dim,
                       [input_source])

    def rmsnorm_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple,
                      block_dim: tuple, eps: float = None):
        assert input.num_dims == 2
        assert output.num_dims == 2
        self._register("rmsnorm_hopper" if self.target_cc >= 90 else "rmsnorm",
                       [(input, (0, -1, -1), 1), (weight, (-1, -1, -1), 0),
                        (output, (0, -1, -1), 1)], grid_dim, block_dim,
                       eps=self.rms_norm_eps if eps is None else eps)

    def rmsnorm_linear_layer(self, input: DTensor, weight_norm: DTensor, weight_linear: DTensor,
                             output: DTensor, grid_dim: tuple, block_dim: tuple, eps: float = None):
        """Fused form; recorded as the two layers it stands for so that the lowering fuses it
        the same way it fuses a separate rmsnorm_layer + linear_layer pair."""
        assert input.num_dims == 2 and weight_linear.num_dims == 2 and output.num_dims == 2
        tmp = self.new_tensor(dims=input.dims, dtype=input.dtype,
                              name=f"_rmsnorm_linear_tmp_{len(self.kn_graph.cygraph.tensors)}")
        self.rmsnorm_layer(input, weight_norm, tmp, (input.dims[0], 1, 1), block_dim, eps=eps)
        self.linear_layer(tmp, weight_linear, output, grid_dim, block_dim)

    def paged_attention_layer(self, input: DTensor, k_cache: DTensor, v_cache: DTensor,
                              q_norm: DTensor, k_norm: DTensor, cos_pos_embed: DTensor,
                              sin_pos_embed: DTensor, output: DTensor, grid_dim: tuple,
                              block_dim: tuple):
        assert input.num_dims == 2      # (num_tokens, fused_outdim / world_size)
        assert output.num_dims == 2     # (num_tokens, hidden_size / world_size)
        assert k_cache.num_dims == 4    # (num_pages, page_size, kv_heads, head_dim)
        assert v_cache.num_dims == 4
        assert k_cache.dim(0) == self.max_num_pages
        assert v_cache.dim(0) == self.max_num_pages
        assert k_cache.dim(1) == self.page_size
        assert v_cache.dim(1) == self.page_size
        head_dim = k_cache.dim(3)
        num_kv_heads = k_cache.dim(2)
        num_q_heads = output.dim(1) // head_dim
        rotary_embed = 0
        if cos_pos_embed is not None or sin_pos_embed is not None:
            assert cos_pos_embed.num_dims == 2 and sin_pos_embed.num_dims == 2
            assert cos_pos_embed.dim(1) == head_dim
            assert sin_pos_embed.dim(1) == head_dim
            rotary_embed = 1
        qk_norm = 0
        if q_norm is not None or k_norm is not None:
            assert q_norm.num_dims == 1 and k_norm.num_dims == 1
            assert q_norm.dim(0) == head_dim and k_norm.dim(0) == head_dim
            qk_norm = 1
        params = [num_q_heads, num_kv_heads, qk_norm, rotary_embed, self.max_seq_length,
                  self.page_size]
        assert grid_dim[0] == self.max_num_batched_requests
        assert grid_dim[1] == num_kv_heads
        name = {90: "paged_attention_hopper", 100: "paged_attention_sm100"}.get(
            self.target_cc, "paged_attention")
        attrs = {}
        if qk_norm:
            # the two weight vectors are packed into one runtime-owned [2, head_dim] tensor when
            # the graph is compiled (one pointer operand of the task)
            packed = self.kn_graph.cygraph.new_input((2, head_dim), None, q_norm.dtype)
            packed.kind, packed.name = "shuffled", f"{q_norm.name or 'q_norm'}+{k_norm.name or 'k_norm'}"
            packed.sources, packed.num_groups = [q_norm, k_norm], 1
            attrs = {"qk_norm_packed": packed, "eps": self.rms_norm_eps}
        self._register(name, [(input, (-1, 1, -1), -1), (k_cache, (-1, 2, -1), 1),
                              (v_cache, (-1, 2, -1), 1), (q_norm, (-1, -1, -1), -1),
                              (k_norm, (-1, -1, -1), -1), (cos_pos_embed, (-1, -1, -1), -1),
                              (sin_pos_embed, (-1, -1, -1), -1), (output, (-1, 1, -1), -1)],
                       grid_dim, block_dim, params, **attrs)

    def linear_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple,
                     block_dim: tuple):
        assert input.num_dims == 2 and weight.num_dims == 2 and output.num_dims == 2
        name = {100: "linear_sm100", 90: "linear_swapAB_hopper"}.get(self.target_cc, "linear")
        self._register(name, [(input, (-1, -1, -1), 1), (weight, (0, -1, -1), 1),
                              (output, (1, -1, -1), -1)], grid_dim, block_dim)

    def linear_with_residual_layer(self, input: DTensor, weight: DTensor, residual: DTensor,
                                   output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2 and weight.num_dims == 2
        assert residual.num_dims == 2 and output.num_dims == 2
        name = {100: "linear_with_residual_sm100",
                90: "linear_swapAB_with_residual_hopper"}.get(self.target_cc,
                                                              "linear_with_residual")
        self._register(name, [(input, (-1, -1, -1), 1), (weight, (0, -1, -1), 1),
                              (residual, (1, -1, -1), -1), (output, (1, -1, -1), -1)],
                       grid_dim, block_dim)

    def allreduce_layer(self, input: DTensor, buffer: DTensor, output: DTensor, grid_dim: tuple,
                        block_dim: tuple):
        assert input.num_dims == 2      # (batch_size, hidden_size)
        assert buffer.num_dims == 3     # (world_size, batch_size, hidden_size)
        assert output.num_dims == 2
        self._register("allreduce", [(input, (1, -1, -1), -1), (buffer, (2, -1, -1), -1),
                                     (output, (1, -1, -1), -1)], grid_dim, block_dim,
                       [self.world_size, self.mpi_rank])

    def silu_mul_layer(self, input: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2      # (batch_size, 2 * intermediate_size)
        assert output.num_dims == 2     # (batch_size, intermediate_size)
        self._register("silu_mul", [(input, (1, -1, -1), 1), (output, (1, -1, -1), 1)],
                       grid_dim, block_dim)

    def argmax_partial_layer(self, input: DTensor, output: tuple, grid_dim: tuple,
                             block_dim: tuple, valid_cols: int = None):
        """`valid_cols` (not in the reference): only logits columns [0, valid_cols) are real
        vocabulary; the zero-padded tail of the lm_head is never sampled."""
        assert input.num_dims == 2
        assert len(output) == 2
        output_value, output_index = output
        assert output_value.num_dims == 2 and output_index.num_dims == 2
        num_tasks = grid_dim[0]
        self.argmax_partial_output_size = input.dim(1) // num_tasks
        name = "argmax_partial_sm100" if self.target_cc in (90, 100) else "argmax_partial"
        self._register(name, [(input, (1, 0, -1), -1), (output_value, (1, 0, -1), -1),
                              (output_index, (1, 0, -1), -1)], grid_dim, block_dim, [num_tasks],
                       valid_cols=None if valid_cols is None else int(valid_cols))

    def argmax_reduce_layer(self, input: tuple, output: DTensor, grid_dim: tuple,
                            block_dim: tuple, vocab_offset: int = 0, exchange: bool = False):
        """`exchange=True` (not in the reference): the logits are this rank's slice of a
        vocabulary split over the tensor-parallel ranks, starting at row `vocab_offset`; the
        ranks exchange their winners and all write the same token."""
        assert len(input) == 2
        input_value, input_index = input
        assert input_value.num_dims == 2 and input_index.num_dims == 2
        assert output.num_dims == 2
        name = "argmax_reduce_sm100" if self.target_cc == 100 else "argmax_reduce"
        self._register(name, [(input_value, (1, 0, -1), -1), (input_index, (1, 0, -1), -1),
                              (output, (0, 1, -1), -1)], grid_dim, block_dim,
                       [getattr(self, "argmax_partial_output_size", 0)],
                       vocab_offset=int(vocab_offset), exchange=bool(exchange))

    # ------------------------------------------------------------------ speculative decoding
    # Prompt lookup (persistent_kernel.py:1013-1136 of the reference).  The reference serves one
    # request with it; here every request of the batch that is past its prompt brings its last
    # token plus `spec_length` draft slots per iteration when the token budget allows, the
    # draft ids take the place of the input ids in front of the embedding, and the batcher
    # advances each request by what the verification accepted.
    def find_ngram_partial_layer(self, input: DTensor, output: DTensor, grid_dim: tuple,
                                 block_dim: tuple, ngram_size: int = 3):
        assert input.num_dims == 2      # (requests, max_seq_length): the token matrix
        assert output.num_dims == 2     # (requests, tasks)
        self._register("find_ngram_partial", [(input, (-1, -1, -1), -1), (output, (1, -1, -1), -1)],
                       grid_dim, block_dim, [ngram_size])

    def find_ngram_global_layer(self, input: tuple, output: DTensor, grid_dim: tuple,
                                block_dim: tuple, ngram_size: int = 3, spec_length: int = 5):
        assert len(input) == 2
        partial_results, tokens = input
        assert partial_results.num_dims == 2 and tokens.num_dims == 2 and output.num_dims == 2
        self._register("find_ngram_global",
                       [(partial_results, (-1, -1, -1), -1), (tokens, (-1, -1, -1), -1),
                        (output, (-1, -1, -1), -1)], grid_dim, block_dim, [ngram_size, spec_length])

    def prompt_lookup_spec_handler(self, spec_decode_config, tokens: DTensor, grid_dim: tuple,
                                   block_dim: tuple):
        partial = self.new_tensor(dims=(max(tokens.dim(0), self.max_num_batched_requests), 96),
                                  dtype=int64, name="partial_ngram_output", io_category="cuda_tensor")
        self.find_ngram_partial_layer(input=tokens, output=partial, grid_dim=grid_dim,
                                      block_dim=block_dim, ngram_size=spec_decode_config.ngram_size)
        # one id per token slot of the iteration (the reference: one row of spec_length + 1)
        spec_tokens = self.new_tensor(dims=(self.max_num_batched_tokens, 1), dtype=int64,
                                      name="spec_tokens", io_category="cuda_tensor")
        self.find_ngram_global_layer(input=(partial, tokens), output=spec_tokens, grid_dim=(1, 1, 1),
                                     block_dim=(128, 1, 1), ngram_size=spec_decode_config.ngram_size,
                                     spec_length=spec_decode_config.spec_length)
        return spec_tokens

    def draft_forward_layer_dispatcher(self, spec_decode_config, tokens: DTensor, grid_dim: tuple,
                                       block_dim: tuple):
        handler = self._spec_decode_handlers.get(spec_decode_config.method)
        if handler is None:
            raise ValueError(f"Invalid spec decode method: {spec_decode_config.method}")
        return handler(spec_decode_config, tokens, grid_dim, block_dim)

    def target_verify_greedy_layer(self, input: tuple, output: DTensor, grid_dim: tuple,
                                   block_dim: tuple, spec_length: int = None):
        assert len(input) == 2
        spec_tokens, target_tokens = input
        assert spec_tokens.num_dims == 2 and target_tokens.num_dims == 2 and output.num_dims == 2
        self._register("target_verify_greedy",
                       [(spec_tokens, (-1, -1, -1), -1), (target_tokens, (-1, -1, -1), -1),
                        (output, (-1, -1, -1), -1)], grid_dim, block_dim, spec_length=spec_length)

    def prompt_lookup_verify_handler(self, spec_decode_config, spec_tokens: DTensor,
                                     target_output: DTensor, grid_dim: tuple, block_dim: tuple):
        verify_out = self.new_tensor(dims=(1, 1), dtype=int64, name="verify_out",
                                     io_category="cuda_tensor")
        self.target_verify_greedy_layer(input=(spec_tokens, target_output), output=verify_out,
                                        grid_dim=grid_dim, block_dim=block_dim,
                                        spec_length=spec_decode_config.spec_length)
        return verify_out

    def verify_layer_dispatcher(self, spec_decode_config, spec_tokens: DTensor,
                                target_output: DTensor, grid_dim: tuple = (1, 1, 1),
                                block_dim: tuple = (128, 1, 1)):
        handler = self._spec_verify_handlers.get(spec_decode_config.method)
        if handler is None:
            raise ValueError(f"Invalid spec decode method: {spec_decode_config.method}")
        return handler(spec_decode_config, spec_tokens, target_output, grid_dim, block_dim)

    def single_batch_extend_attention_layer(self, input: DTensor, k_cache: DTensor, v_cache: DTensor,
                                            q_norm: DTensor, k_norm: DTensor, cos_pos_embed: DTensor,
                                            sin_pos_embed: DTensor, output: DTensor, grid_dim: tuple,
                                            block_dim: tuple):
        """The reference's attention for the spec_length + 1 tokens of its one request
        (tasks/ampere/single_batch_extend.cuh); the paged attention task here takes several new
        tokens per request, so this is the same operator over all request slots."""
        self.paged_attention_layer(input, k_cache, v_cache, q_norm, k_norm, cos_pos_embed,
                                   sin_pos_embed, output,
                                   (self.max_num_batched_requests, k_cache.dim(2), 1), block_dim)

    # ------------------------------------------------------------------ mixture of experts
    # The reference's builders (persistent_kernel.py:612-800; graph demo/qwen3/demo_30B_A3B.py:
    # 564-645).  Expert work is laid out by active slot here (lowering.py), so the caller's
    # [tokens, experts per token, width] intermediates only fix the shapes; the runtime keeps
    # its own per-slot buffers.
    def moe_topk_softmax_routing_layer(self, input: DTensor, output: tuple, grid_dim: tuple,
                                       block_dim: tuple):
        assert input.num_dims == 2 and len(output) == 3     # (tokens, experts)
        weights, routing, mask = output
        assert weights.num_dims == 2 and routing.num_dims == 2 and mask.num_dims == 1
        self._register("moe_topk_softmax_sm100",
                       [(input, (0, -1, -1), -1), (weights, (0, -1, -1), -1),
                        (routing, (-1, -1, -1), -1), (mask, (-1, -1, -1), -1)], grid_dim, block_dim)

    def _moe_linear(self, name, input, weight, moe_routing_indices, moe_mask, output, grid_dim, block_dim):
        assert weight.num_dims == 3 and output.num_dims == 3
        assert moe_routing_indices.num_dims == 2 and moe_mask.num_dims == 1
        self._register(name, [(input, (-1, -1, -1), -1), (weight, (-1, 1, -1), 2),
                              (moe_routing_indices, (-1, -1, -1), -1), (moe_mask, (-1, -1, -1), -1),
                              (output, (-1, 2, -1), -1)], grid_dim, block_dim)

    def moe_w13_linear_layer(self, input: DTensor, weight: DTensor, moe_routing_indices: DTensor,
                             moe_mask: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2      # (tokens, hidden)
        self._moe_linear("moe_w13_linear_sm100", input, weight, moe_routing_indices, moe_mask,
                         output, grid_dim, block_dim)

    def moe_silu_mul_layer(self, input: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 3 and output.num_dims == 3
        self._register("moe_silu_mul", [(input, (0, 1, -1), -1), (output, (0, 1, -1), -1)],
                       grid_dim, block_dim)

    def moe_w2_linear_layer(self, input: DTensor, weight: DTensor, moe_routing_indices: DTensor,
                            moe_mask: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 3      # (tokens, experts per token, intermediate)
        self._moe_linear("moe_w2_linear_sm100", input, weight, moe_routing_indices, moe_mask,
                         output, grid_dim, block_dim)

    def moe_mul_sum_add_layer(self, input: DTensor, weight: DTensor, residual: DTensor,
                              output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 3 and weight.num_dims == 2
        assert residual.num_dims == 2 and output.num_dims == 2
        self._register("moe_mul_sum_add_sm100",
                       [(input, (0, 2, -1), -1), (weight, (0, -1, -1), -1),
                        (residual, (0, 1, -1), -1), (output, (0, 1, -1), -1)], grid_dim, block_dim)

    def splitk_linear_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple,
                            block_dim: tuple):
        """The reference's router projection split along K; the same product as linear_layer
        (the task cutter here decides about splits itself)."""
        self.linear_layer(input, weight, output, grid_dim, block_dim)

    def tensor_init_layer(self, *args, **kwargs):
        """The reference zeroes the split-K accumulation target with this task; nothing here
        accumulates into a graph tensor across tasks, so there is nothing to initialise."""
        return None

    # builders of the reference that are outside the decode hot path
    def _not_built(self, what):
        raise NotImplementedError(f"{what} is outside the decode hot path of this build")

    def attention_layer(self, *a, **k): self._not_built("attention_layer (contiguous KV)")
    def identity_layer(self, *a, **k): self._not_built("identity_layer")
    def silu_mul_linear_with_residual_layer(self, *a, **k): self._not_built("silu_mul_linear_with_residual_layer")
    def argmax_layer(self, *a, **k): self._not_built("single-task argmax_layer")

    # ------------------------------------------------------------------ lowering / compile
    def _scratch_tensor(self, dims, dt, name, symmetric=False):
        return self.new_tensor(dims=dims, dtype=dt, name=name,
                               io_category="nvshmem_tensor" if symmetric else "cuda_tensor")

    def _num_ctas(self):
        if torch.cuda.is_available():
            return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        return 148

    def lower(self, num_ctas: int = None) -> lowering.LoweredGraph:
        if self._lowered is None:
            self._lowered = lowering.lower(
                self.kn_graph.cygraph.tasks,
                num_workers=num_ctas or self._num_ctas(),
                max_tokens=self.max_num_batched_tokens,
                max_requests=self.max_num_batched_requests,
                max_seq_length=self.max_seq_length,
                page_size=self.page_size,
                world_size=self.world_size, rank=self.mpi_rank,
                default_eps=self.rms_norm_eps,
                new_tensor=self._scratch_tensor, serving=self.mode == "offline",
                handoff=getattr(self, "handoff", None) or os.environ.get("YPK_HANDOFF", "auto"))
        return self._lowered

    def _generate_task_graph(self, num_gpus: int, my_gpu_id: int):
        g = self.lower()
        note = ("// No per-model CUDA source is generated by this build: the task table in the\n"
                "// JSON file is executed by the prebuilt sm_100a megakernel (libypk.so).\n")
        return {"json_file": lowering.to_json(g), "cuda_code": note}

    def _config(self, device: int, num_ctas: int) -> N.Config:
        cfg = N.Config()
        cfg.device = device
        cfg.world_size, cfg.rank = self.world_size, self.mpi_rank
        cfg.num_workers = num_ctas
        cfg.mode = 1 if self.mode == "offline" else 0
        cfg.max_seq_length = self.max_seq_length
        cfg.max_num_batched_requests = self.max_num_batched_requests
        cfg.max_num_batched_tokens = self.max_num_batched_tokens
        cfg.max_num_pages = self.max_num_pages
        cfg.page_size = self.page_size
        cfg.total_num_requests = self.total_num_requests
        cfg.eos_token_id = int(self.eos_token_id) if self.eos_token_id is not None else -1
        cfg.wait_budget_ns = int(float(os.environ.get("YPK_WAIT_BUDGET_S", "2.0")) * 1e9)
        m = self.meta_tensors or {}
        expect = {"step": torch.int32, "tokens": torch.int64, "input_tokens": torch.int64,
                  "output_tokens": torch.int64, "num_new_tokens": torch.int32,
                  "prompt_lengths": torch.int32, "qo_indptr_buffer": torch.int32,
                  "paged_kv_indptr_buffer": torch.int32, "paged_kv_indices_buffer": torch.int32,
                  "paged_kv_last_page_len_buffer": torch.int32}
        fields = ("step", "tokens", "input_tokens", "output_tokens", "num_new_tokens",
                  "prompt_lengths", "qo_indptr", "paged_kv_indptr", "paged_kv_indices",
                  "paged_kv_last_page_len")
        for key, fld in zip(_META_KEYS, fields):
            t = m.get(key)
            if t is None:
                continue
            if t.dtype != expect[key]:
                raise TypeError(f"meta tensor '{key}' must be {expect[key]}, got {t.dtype}")
            if not t.is_contiguous():
                raise ValueError(f"meta tensor '{key}' must be contiguous")
            setattr(cfg, fld, t.data_ptr())
        if self.profiler_tensor is not None:
            cfg.profiler_buffer = self.profiler_tensor.data_ptr()
            cfg.profiler_bytes = self.profiler_tensor.numel() * self.profiler_tensor.element_size()
        return cfg

    def compile(self, **kwargs):
        """Lower the graph and load it into the native runtime.  `dry_run=True` validates
        the graph through a host-only handle (no GPU needed) and stops there."""
        assert not self._is_compiled
        dry = bool(kwargs.get("dry_run", False))
        output_dir = kwargs.get("output_dir", None)
        if not dry and not torch.cuda.is_available():
            raise RuntimeError("PersistentKernel.compile needs a CUDA device (sm_100a); "
                               "there is no CPU execution path")
        num_ctas = self._num_ctas()
        g = self.lower(num_ctas)
        if output_dir is not None:
            os.makedirs(output_dir, exist_ok=True)
            with open(os.path.join(output_dir, f"task_graph_rank{self.mpi_rank}.json"), "w") as f:
                f.write(lowering.to_json(g))
        device = -1 if dry else torch.cuda.current_device()
        h = N.Handle(self._config(device, num_ctas))
        # tensors: attached ones are bound, runtime-owned ones allocated, shuffles built
        used = {}
        for ts in g.tasks:
            for p in ts.ptr:
                if p is not None:
                    used[p[0].guid] = p[0]
        for sh in g.shuffles:
            for s in sh["sources"]:
                used[s.guid] = s
        shuffled = {id(sh["dst"]) for sh in g.shuffles}
        if self.world_size > 1:
            # peer-visible tensors come from one symmetric arena, allocated in guid order so
            # that every rank (same graph, same order) gets the same offsets
            sym = [t for _, t in sorted(used.items()) if t.kind == "nvshmem"]
            h.comm_init(sum((t.nbytes + 255) // 256 * 256 for t in sym) + 256)
        for guid, t in sorted(used.items()):
            name = t.name or f"tensor_{guid}"
            if t.kind == "torch":
                tt = t.torch_tensor
                if not dry and not tt.is_cuda:
                    raise ValueError(f"attached tensor '{name}' is not on the GPU")
                h.bind(guid, name, tt.data_ptr(), tt.numel() * tt.element_size())
            elif t.kind == "nvshmem" and self.world_size > 1:
                h.alloc_symmetric(guid, name, t.nbytes)
            elif t.kind in ("cuda", "nvshmem"):
                h.alloc(guid, name, t.nbytes)
            elif t.kind == "shuffled":
                if id(t) not in shuffled:
                    raise ValueError(f"shuffled tensor '{name}' is used by no linear layer")
            else:
                raise ValueError(f"tensor '{name}' has no storage (kind={t.kind})")
        for sh in g.shuffles:
            h.shuffle(sh["dst"].guid, sh["dst"].name or "shuffled",
                      [s.guid for s in sh["sources"]], sh["rows"], sh["gran"], sh["row_bytes"])
        tasks = []
        for ts in g.tasks:
            t = N.Task()
            t.type, t.flags, t.op_id = ts.type, ts.flags, ts.op_id
            t.dep_event, t.dep_count, t.trig_event = ts.dep_event, ts.dep_count, ts.trig_event
            for i, p in enumerate(ts.ptr):
                t.ptr[i] = N.ref(p[0].guid, p[1]) if p is not None else 0
            t.ptr_aux = N.ref(ts.ptr_aux[0].guid, ts.ptr_aux[1]) if ts.ptr_aux is not None else 0
            for i, v in enumerate(ts.iarg):
                t.iarg[i] = v
            for i, v in enumerate(ts.farg):
                t.farg[i] = v
            tasks.append(t)
        h.load_graph(tasks, g.num_events, g.queue, g.queue_off)
        if self.world_size > 1 and not kwargs.get("defer_connect", False):
            from . import tensor_parallel
            tensor_parallel.connect(h, self.world_size, self.mpi_rank)
        self._handle = h
        self._is_compiled = True
        self._dry = dry
        # the three callables the reference's generated launcher module exports
        self.init_func = lambda *a, **k: h.reset()
        self.launch_func = lambda *a, **k: self.__call__()
        self.finalize_func = lambda *a, **k: self.finalize()

    # ------------------------------------------------------------------ run
    def __call__(self, **kwargs):
        """Run the megakernel.  Offline mode: until every request has retired (or for
        `max_iterations` iterations, after which a later call resumes).  One-pass mode:
        the graph once for `batch` rows.  Synchronous, like the reference's launch_func."""
        if not self._is_compiled or self._dry:
            raise RuntimeError("PersistentKernel is not compiled for a device")
        stream = kwargs.get("stream", None)
        if stream is None:
            stream = torch.cuda.current_stream()
        sp = stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)
        self._handle.launch(sp, int(kwargs.get("max_iterations", 0)), int(kwargs.get("batch", 1)))
        if self.profiler_tensor is not None and self.trace_name:
            from .profiler_persistent import export_trace
            g = self.lower()
            export_trace(self.profiler_tensor, self.trace_name, self._handle.cfg.num_workers,
                         self.profile_stride(), g.tasks)

    def launch_async(self, **kwargs):
        """Enqueue the megakernel on the stream and return; `wait()` collects the outcome.
        (The reference's launch_func is synchronous; this is for callers that time the launch
        with events or overlap host work.)"""
        if not self._is_compiled or self._dry:
            raise RuntimeError("PersistentKernel is not compiled for a device")
        stream = kwargs.get("stream", None) or torch.cuda.current_stream()
        sp = stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)
        self._handle.launch_async(sp, int(kwargs.get("max_iterations", 0)), int(kwargs.get("batch", 1)))

    def wait(self):
        self._handle.wait()

    def profile_stride(self):
        """Records per worker in the profiler buffer (= the longest worker queue)."""
        g = self.lower()
        return max(b - a for a, b in zip(g.queue_off[:-1], g.queue_off[1:]))

    def profile_summary(self):
        """Per-operator timing of the last iteration (needs profiler_tensor)."""
        from .profiler_persistent import decode_records, summarize
        g = self.lower()
        recs = decode_records(self.profiler_tensor, self._handle.cfg.num_workers,
                              self.profile_stride())
        return summarize(recs, g.tasks, g.ops)

    def read_tensor(self, t: DTensor) -> torch.Tensor:
        """Copy of a tensor of the graph (attached or runtime-owned) as a torch tensor."""
        from .core import convert_dtype_to_torch_type
        out = torch.empty(t.dims, dtype=convert_dtype_to_torch_type(t.dtype), device="cuda")
        self._handle.read_tensor(t.guid, 0, out.data_ptr(), t.nbytes)
        return out

    def reset(self):
        """Back to the state right after compile(): step = 0, all pages free."""
        self._handle.reset()

    def status(self):
        return self._handle.status()

    # Two graphs over one set of requests (see ypk_adopt_batch): a graph built for many tokens
    # per iteration runs the prompts, one built for at most 8 tokens the decoding.
    def set_pause_below(self, tokens: int):
        """Launches return, with the batch left waiting, once the batcher forms a batch of at
        most `tokens` tokens (0: off)."""
        self._handle.set_pause_below(int(tokens))

    def adopt(self, other: "PersistentKernel"):
        """Take over the requests of `other` where it stopped.  Both kernels must have been
        built over the same meta tensors and K/V caches."""
        self._handle.adopt_batch(other._handle)

    def __del__(self):
        if sys is None or sys.is_finalizing():
            return
        try:
            if not self.__finalized__:
                self.finalize()
        except Exception:
            pass

    def finalize(self):
        assert not self.__finalized__
        if self._handle is not None:
            self._handle.close()
            self._handle = None
        self.__finalized__ = True
