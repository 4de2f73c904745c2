"""Numerics of the multi-branch graphs of tests/graph_shapes.py on the GPU (one launch each, test mode) against the
CPU oracle; bf16 outputs within max relative error 2e-2.  Counterpart of the reference's test-mode suite
(tests/runtime_python/test_mode/test_{fork_point,join_point,diamond_fork_join,residual_stripping,grid_dim_sweep,
case2_case3_negative}_testmode.py); the two role combinations the reference refuses run here like any other graph."""
import pytest
import torch

from graph_shapes import KINDS, build
from gpu_util import make_test_kernel, rel_err

pytestmark = pytest.mark.gpu


def _run(kind, B, H):
    import mirage_b200 as mi
    pk = make_test_kernel(mi, B)
    _, outs, ref = build(pk, kind, B, H, "cuda")
    pk.compile()
    pk.run_test_mode()
    want = ref()
    for name, r in want.items():
        assert rel_err(outs[name].cpu(), r) <= 2e-2, (kind, name)
    first = {k: v.clone() for k, v in outs.items()}
    pk.run_test_mode()                      # a second launch leaves the same bits: no state is carried over
    for k, v in outs.items():
        assert torch.equal(first[k], v), (kind, k)


@pytest.mark.parametrize("kind", KINDS)
def test_graph_shape(kind):
    _run(kind, 8, 1024)


@pytest.mark.parametrize("B,H", [(4, 4096), (8, 4096), (16, 4096), (8, 2048)])
def test_fork_grid_sweep(B, H):
    _run("fork", B, H)


def test_diamond_with_sixteen_tokens_runs_on_the_tensor_path():
    _run("diamond", 16, 2048)
