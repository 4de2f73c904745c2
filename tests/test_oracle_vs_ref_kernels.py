"""Pins the CPU oracle against outputs of the reference's own compiled sm100 kernels (tests/golden/ref_kernel_outputs.pt,
made on a B200 by tests/golden/make_ref_kernel_golden.py from the reference's unmodified sources): per-token x 128
quantisation to e4m3 with packed UE8M0 scales (bit-exact), grouped-sigmoid and softmax top-k routing (indices bit-exact,
active-expert list as a set -- the kernels fill it in arrival order --, weights to 1e-6).  The expert GEMM and MLA decode
outputs in the same fixture belong to inputs of several GB that are regenerated on the device: they are checked on the
GPU (tests/test_gpu_ref_kernel_golden.py)."""
import os

import pytest
import torch

from oracle import fp8_ops, moe_ops
from tests_golden import QUANTIZE_CASES, ROUTING_CASES, quantize_case_input, routing_case_input


@pytest.fixture(scope="module")
def fixture(golden_dir):
    return torch.load(os.path.join(golden_dir, "ref_kernel_outputs.pt"), weights_only=False)


@pytest.mark.parametrize("case", QUANTIZE_CASES)
def test_quantize_oracle_equals_the_reference_kernel(fixture, case):
    B, H, seed = case
    want = fixture["quantize_fp8"][case]
    q, exps, packed = fp8_ops.quantize_fp8_ue8m0(quantize_case_input(B, H, seed))
    assert torch.equal(q.view(torch.uint8), want["q"])
    # the kernel's scale tensor is [packed words, tokens]; the oracle's packed words are [tokens, packed words]
    got = (packed & 0xFFFFFFFF).t().contiguous()
    ref = want["scale_words"].to(torch.int64) & 0xFFFFFFFF
    assert torch.equal(got, ref)


@pytest.mark.parametrize("case", ROUTING_CASES)
def test_routing_oracles_equal_the_reference_kernels(fixture, case):
    B, seed = case
    logits, bias = routing_case_input(B, seed)
    for mode in ("sigmoid", "softmax"):
        w_ref, idx_ref, act_ref = fixture["routing"][case][mode]
        if mode == "sigmoid":
            w, idx, act = moe_ops.topk_sigmoid_routing(logits, bias, topk=8, num_groups=8, topk_group=4, scaling=2.5)[:3]
        else:
            w, idx, act = moe_ops.topk_softmax_routing(logits, topk=8)[:3]
        assert torch.equal(idx.to(torch.int32), idx_ref), mode
        n = int(act_ref[-1])
        assert int(act[-1]) == n and set(act[:n].tolist()) == set(act_ref[:n].tolist()), mode
        assert float((w - w_ref).abs().max()) <= 1e-6 * max(1.0, float(w_ref.abs().max())), mode
