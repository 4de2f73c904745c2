"""Host side of the tensor-parallel set-up on CPU: two gloo ranks exchange their exchange-region handles
through mirage_b200.multigpu.exchange_comm_handles (dry-run handles: no CUDA call)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.qwen3_decoder import Qwen3Config
        from dry_util import dry_qwen3
        import json
        pk = dry_qwen3(Qwen3Config.qwen3_8b(2), world=world, rank=rank)
        g = json.loads(pk.dump_task_graph())
        # identical schedule on every rank: same task count, same event list
        sig = torch.tensor([g["num_tasks"], g["num_events"], g["weight_bytes"] % (1 << 31)], dtype=torch.int64)
        sigs = [torch.zeros_like(sig) for _ in range(world)]
        dist.all_gather(sigs, sig)
        assert all(torch.equal(s, sigs[0]) for s in sigs)
        # the handle exchange itself (all_gather of 64-byte handles, import of every peer)
        from mirage_b200.multigpu import exchange_comm_handles
        exchange_comm_handles(pk)
        # once linked, reset() is a collective: the early rank waits for the late one on both sides of the clearing
        # (a rank that launched before a peer had cleared its inbox would lose its first pushes)
        import time
        if rank == 1:
            time.sleep(1.0)
        t0 = time.perf_counter()
        pk.reset()
        waited = time.perf_counter() - t0
        assert rank != 0 or waited > 0.5, f"rank 0 left reset() after {waited:.2f} s without waiting for rank 1"
        # after an expired device wait, the next step() must clear counters and inboxes through the FENCED reset (the
        # library refuses to reset silently under tensor parallelism): the early rank waits for the late one again
        pk._timed_out = True                 # what status() records when it raises MpkTimeoutError
        if rank == 1:
            time.sleep(1.0)
        t0 = time.perf_counter()
        try:
            pk.step(1)                       # dry-run handles cannot launch: the reset comes first, then the refusal
        except Exception:
            pass
        waited = time.perf_counter() - t0
        assert not pk._timed_out
        assert rank != 0 or waited > 0.5, f"rank 0 re-launched after {waited:.2f} s without the collective reset"
        # a mismatch between the kernel's rank and the process group is refused
        pk.mpi_rank = (rank + 1) % world
        try:
            exchange_comm_handles(pk)
            q.put((rank, "no error"))
        except RuntimeError:
            q.put((rank, "ok"))
    finally:
        dist.destroy_process_group()


def test_handle_exchange_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    got = sorted(q.get(timeout=10) for _ in range(2))
    assert got == [(0, "ok"), (1, "ok")]
