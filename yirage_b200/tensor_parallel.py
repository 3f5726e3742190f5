"""Tensor-parallel plumbing above the C ABI: moving the arena handles between the ranks.

The reference bootstraps NVSHMEM over MPI (persistent_kernel.cuh:1072-1085) and launches
one process per GPU with mpirun (demo/llama3/demo.py:61-81).  Here the ranks are
torch.distributed processes (torchrun); the only thing they exchange on the host is the
64-byte CUDA IPC handle of each rank's symmetric arena.  After that the data path is
device-side only: the ALLREDUCE tasks of the megakernel write into the peers' arenas over
NVLink and signal counters there.
"""
import torch.distributed as dist


def exchange_handles(own: bytes, world_size: int, rank: int, group=None):
    """All-gather of the per-rank IPC handles (any initialised process group will do:
    nccl on GPUs, gloo in the CPU tests)."""
    if not dist.is_initialized():
        raise RuntimeError("tensor parallelism needs torch.distributed to be initialised "
                           "(one process per GPU, e.g. under torchrun)")
    if dist.get_world_size(group) != world_size or dist.get_rank(group) != rank:
        raise RuntimeError("PersistentKernel world_size / mpi_rank do not match the process group")
    handles = [None] * world_size
    dist.all_gather_object(handles, own, group=group)
    return handles


def connect(handle, world_size: int, rank: int, group=None):
    """Export the own arena, import every peer's.  Collective: every rank calls it."""
    handles = exchange_handles(handle.comm_export(), world_size, rank, group)
    for peer, hb in enumerate(handles):
        if peer != rank:
            handle.comm_import(peer, hb)
    dist.barrier(group=group)
