"""A device-side wait that cannot be satisfied runs out and is reported; nothing hangs or traps.

Rank 0 of a two-rank tensor-parallel graph is launched ALONE: its allreduce consumer polls an inbox that the other
rank (compiled and linked in the same process, but never launched) does not fill.  Every device wait carries a
wall-clock budget (shortened here to 300 ms through MPK_SPIN_LIMIT_MS); when it expires the CTA records where it
gave up, raises the abort flag the other waits poll, the streaming warps drain their copies in flight, the launch
ends and the host reads MPK_ERR_TIMEOUT.  The context stays usable: a fresh single-rank kernel runs right after."""
import os

import pytest
import torch

from oracle import mpk_ops as ops
from gpu_util import make_test_kernel, rel_err

pytestmark = pytest.mark.gpu


def _tp_rank(mi, rank, x, w1, g, w2):
    pk = make_test_kernel(mi, x.shape[0], world_size=2, mpi_rank=rank)
    b, k = x.shape
    n = w1.shape[0]
    y = pk.new_tensor(dims=(b, n), dtype=mi.bfloat16, name="y", io_category="nvshmem_tensor")
    z = pk.new_tensor(dims=(b, n), dtype=mi.bfloat16, name="z", io_category="nvshmem_tensor")
    buf = pk.new_tensor(dims=(2, b, n), dtype=mi.bfloat16, name="ar_buf", io_category="nvshmem_tensor")
    out = torch.zeros(b, w2.shape[0], dtype=torch.bfloat16, device="cuda")
    pk.linear_layer(input=pk.attach_input(x.cuda(), "x"), weight=pk.attach_input(w1.cuda(), "w1"), output=y,
                    grid_dim=(8, 1, 1), block_dim=(128, 1, 1))
    pk.allreduce_layer(input=y, buffer=buf, output=z, grid_dim=(8, 1, 1), block_dim=(128, 1, 1))
    pk.rmsnorm_linear_layer(input=z, weight_norm=pk.attach_input(g.cuda(), "g"), weight_linear=pk.attach_input(w2.cuda(), "w2"),
                            output=pk.attach_input(out, "out"), grid_dim=(8, 1, 1), block_dim=(128, 1, 1))
    pk.compile(link_peers=False)
    return pk, out


def test_unsatisfied_peer_wait_times_out_and_is_reported(monkeypatch):
    import mirage_b200 as mi
    from mirage_b200.multigpu import link_local
    monkeypatch.setenv("MPK_SPIN_LIMIT_MS", "300")
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(2, 512, generator=gen).to(torch.bfloat16)
    w1 = (0.05 * torch.randn(1024, 512, generator=gen)).to(torch.bfloat16)
    g = (1 + 0.02 * torch.randn(1024, generator=gen)).to(torch.bfloat16)
    w2 = (0.05 * torch.randn(256, 1024, generator=gen)).to(torch.bfloat16)
    k0, _ = _tp_rank(mi, 0, x, w1, g, w2)
    k1, _ = _tp_rank(mi, 1, x, w1, g, w2)
    link_local([k0, k1])
    torch.cuda.synchronize()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    k0.step(1)                      # rank 1 is never launched: its partial sums never arrive
    t1.record()
    with pytest.raises(mi.MpkTimeoutError):
        k0.status()
    ms = t0.elapsed_time(t1)
    assert 250 <= ms <= 2000, ms    # gave up after the budget, not before, and did not linger
    monkeypatch.delenv("MPK_SPIN_LIMIT_MS")
    # the context is intact: an ordinary single-rank graph runs and is correct
    pk = make_test_kernel(mi, 2)
    out = torch.zeros(2, 1024, dtype=torch.bfloat16, device="cuda")
    pk.linear_layer(input=pk.attach_input(x.cuda(), "x"), weight=pk.attach_input(w1.cuda(), "w1"),
                    output=pk.attach_input(out, "out"), grid_dim=(8, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert rel_err(out.cpu(), ops.linear(x, w1)) <= 2e-2
