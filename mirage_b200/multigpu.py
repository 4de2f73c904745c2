"""Tensor-parallel plumbing: exchange of the per-rank exchange-region handles.

Stands in for the reference's NVSHMEM bootstrap and team set-up
(python/mirage/mpk/multigpu.py:74-96, include/mirage/persistent_kernel/persistent_kernel.cuh:1225-1282):
one process per GPU, `torch.distributed` moves the 64-byte CUDA IPC handle of each rank's exchange
region (event counters + allreduce inboxes), every rank maps all peers, and from then on the
megakernel pushes partial sums and counter increments straight into peer memory over NVLink.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _native as N


def exchange_comm_handles(pk, group=None) -> None:
    """Collective: call on every rank after compile()."""
    if not dist.is_initialized():
        raise RuntimeError("world_size > 1 needs torch.distributed to be initialised (one process per GPU)")
    world = dist.get_world_size(group)
    if world != pk.world_size or dist.get_rank(group) != pk.mpi_rank:
        raise RuntimeError("PersistentKernel world_size/mpi_rank do not match the process group")
    buf = C.create_string_buffer(64)
    N.check(pk._h, N.lib.mpk_comm_export(pk._h, buf))
    mine = torch.tensor(list(buf.raw), dtype=torch.uint8)
    backend = dist.get_backend(group)
    dev = torch.device("cuda", pk.device) if backend == "nccl" else torch.device("cpu")
    gathered = [torch.empty(64, dtype=torch.uint8, device=dev) for _ in range(world)]
    dist.all_gather(gathered, mine.to(dev), group=group)
    for r, t in enumerate(gathered):
        if r == pk.mpi_rank:
            continue
        raw = bytes(t.cpu().tolist())
        N.check(pk._h, N.lib.mpk_comm_import(pk._h, r, C.create_string_buffer(raw, 64)))
    # from here on reset() is a collective of this group: nobody may push into a peer before that peer has finished
    # clearing its counters and inboxes
    pk._dist_linked, pk._dist_group = True, group
    pk.reset()


def rank_fence(pk, stream=None) -> None:
    """Every rank's work enqueued so far has finished on its device, and every rank knows it."""
    if not pk.dry_run:
        if hasattr(stream, "synchronize"):
            stream.synchronize()
        else:
            torch.cuda.synchronize(pk.device)
    dist.barrier(group=pk._dist_group)


def link_local(kernels) -> None:
    """Single-process variant (tests): `kernels[r]` is rank r's PersistentKernel on its own device."""
    for a in kernels:
        for r, b in enumerate(kernels):
            N.check(a._h, N.lib.mpk_comm_link_local(a._h, r, b._h))
    for k in kernels:
        k.reset()
