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
