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
from golden_inputs import QUANTIZE_CASES, ROUTING_CASES, quantize_case_input, routing_case_input


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


def test_attention_oracle_matches_the_reference_kernel(fixture):
    """oracle.mpk_ops.paged_attention_request against the reference's multitoken_paged_attention kernel: outputs and
    appended K rows to 1e-2 of the largest magnitude (bf16 kernel, fp32 oracle), appended V rows bit-exact."""
    from oracle import mpk_ops
    from golden_inputs import ATTENTION_CASES, attention_case_input
    if "paged_attention" not in fixture:
        pytest.skip("fixture has no paged_attention section")
    for case in ATTENTION_CASES:
        prefix, n_new, page, seed = case
        want = fixture["paged_attention"][case]
        t = attention_case_input(prefix, n_new, seed)
        kc, vc = t["k_cache"].clone().unsqueeze(2), t["v_cache"].clone().unsqueeze(2)
        out = mpk_ops.paged_attention_request(t["qkv"], kc, vc, [page], prefix + n_new, 4, 1, t["q_norm"], t["k_norm"],
                                              t["cos"], t["sin"], 1e-6)
        ref = want["out"].float()
        err = float((out.float().reshape(n_new * 4, 128) - ref).abs().max() / ref.abs().max())
        assert err <= 1e-2, (case, err)
        k_ref = want["k_rows"].float()
        assert float((kc[page, prefix:prefix + n_new, 0].float() - k_ref).abs().max() / k_ref.abs().max()) <= 1e-2, case
        assert torch.equal(vc[page, prefix:prefix + n_new, 0], want["v_rows"]), case

