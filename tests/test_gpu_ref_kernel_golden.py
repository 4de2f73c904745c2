"""Parity against outputs of the reference's own compiled sm100 kernels (tests/golden/ref_kernel_outputs.pt, made by
tests/golden/make_ref_kernel_golden.py on a B200 from the reference's unmodified sources): the FP8 expert GEMM at the
DeepSeek-V3 W13 shape and the 16-head absorbed-MLA decode.  The inputs are regenerated from their seeds; their byte
checksums are compared with the ones stored beside the outputs first, so a generator that changed shows up as a skip
with that reason and not as a kernel mismatch.  Bars: one bf16 step of the largest output magnitude."""
import os

import pytest
import torch

import bench
from gpu_util import input_checksums

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fixture(golden_dir):
    path = os.path.join(golden_dir, "ref_kernel_outputs.pt")
    if not os.path.exists(path):
        pytest.skip("tests/golden/ref_kernel_outputs.pt not generated")
    return torch.load(path, weights_only=False)


def _same_inputs(t, keys, want):
    got = input_checksums(t, keys)
    if got != want:
        pytest.skip(f"seeded inputs differ from the ones the fixture was made with ({got} vs {want}): regenerate the fixture")


def test_expert_gemm_matches_the_reference_kernel(fixture):
    import mirage_b200 as mi
    f = fixture["moe_w13"]
    dev = torch.device("cuda", 0)
    t = bench.moe_w13_inputs(dev)
    assert torch.equal(t["routing"].cpu(), f["routing"]) and torch.equal(t["mask"].cpu(), f["mask"])
    _same_inputs(t, ("w", "ws", "xq", "xs"), f["checksums"])
    pk, mine = bench.build_moe_w13_graph(mi, t)
    pk.run_test_mode()
    torch.cuda.synchronize()
    assert pk.status().error == 0
    got, ref = pk.tensor_as_torch(mine).float().cpu(), f["out"].float()
    routed = torch.zeros(t["B"], t["topk"], dtype=torch.bool)
    for b in range(t["B"]):
        slots = f["routing"][:, b]
        routed[b, (slots[slots > 0] - 1).long()] = True
    assert int(routed.sum()) == t["B"] * t["topk"]            # every (token, slot) pair is routed in this workload
    diff = (got - ref).abs()
    step = 2.0 ** (torch.floor(torch.log2(ref.abs().max())).item() - 7)      # one bf16 step at the largest magnitude
    assert float(diff.max()) <= step, f"max |difference| {float(diff.max())} > one bf16 step {step}"
    assert float((diff > 0).float().mean()) < 0.25           # most outputs are bit-identical


def test_mla_decode_matches_the_reference_kernel(fixture):
    import mirage_b200 as mi
    f = fixture["mla_dense"]
    dev = torch.device("cuda", 0)
    t = bench.mla_dense_inputs(dev)
    _same_inputs(t, ("q", "kv"), f["checksums"])
    pk, mine = bench.build_mla_dense_graph(mi, t)
    pk.run_test_mode()
    torch.cuda.synchronize()
    assert pk.status().error == 0
    got, ref = mine.float().cpu(), f["out"].float()
    step = 2.0 ** (torch.floor(torch.log2(ref.abs().max())).item() - 7)
    assert float((got - ref).abs().max()) <= step
