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


def test_quantize_fp8_bit_exact_with_the_reference_kernel(fixture):
    """e4m3 bytes and packed UE8M0 scale words equal to the last bit (byte / integer work: no tolerance)."""
    import mirage_b200 as mi
    from gpu_util import make_test_kernel
    from golden_inputs import QUANTIZE_CASES, quantize_case_input
    if "quantize_fp8" not in fixture:
        pytest.skip("fixture has no quantize_fp8 section")
    for (B, H, seed) in QUANTIZE_CASES:
        want = fixture["quantize_fp8"][(B, H, seed)]
        pk = make_test_kernel(mi, B)
        q = pk.new_tensor(dims=(B, H), dtype=mi.float8_e4m3, name="q", io_category="cuda_tensor")
        packed = (H // 128 + 3) // 4
        sc = pk.new_tensor(dims=(packed, (B + 3) // 4 * 4), dtype=mi.uint32, name="s", io_category="cuda_tensor")
        pk.quantize_fp8_layer(input=pk.attach_input(quantize_case_input(B, H, seed).cuda(), "x"), output_fp8=q, output_scale=sc,
                              grid_dim=(B, 1, 1), block_dim=(128, 1, 1))
        pk.compile()
        pk.run_test_mode()
        torch.cuda.synchronize()
        assert pk.status().error == 0
        got_q = pk.tensor_as_torch(q).view(torch.uint8).cpu()
        got_s = pk.tensor_as_torch(sc).view(torch.int32).cpu()[:, :B]
        assert torch.equal(got_q, want["q"]), f"e4m3 bytes differ for {(B, H)}: {int((got_q != want['q']).sum())} of {got_q.numel()}"
        assert torch.equal(got_s, want["scale_words"]), f"scale words differ for {(B, H)}"


@pytest.mark.parametrize("mode", ["sigmoid", "softmax"])
def test_routing_matches_the_reference_kernel(fixture, mode):
    """Routing indices bit-exact, the active-expert list equal as a set with the same count, weights to 1e-5."""
    import mirage_b200 as mi
    from gpu_util import make_test_kernel
    from golden_inputs import ROUTING_CASES, routing_case_input
    if "routing" not in fixture:
        pytest.skip("fixture has no routing section")
    for (B, seed) in ROUTING_CASES:
        w_ref, idx_ref, act_ref = fixture["routing"][(B, seed)][mode]
        logits, bias = routing_case_input(B, seed)
        pk = make_test_kernel(mi, B)
        w = torch.zeros(B, 8, dtype=torch.float32, device="cuda")
        idx = torch.zeros(256, B, dtype=torch.int32, device="cuda")
        act = torch.zeros(257, dtype=torch.int32, device="cuda")
        outs = (pk.attach_input(w, "w"), pk.attach_input(idx, "idx"), pk.attach_input(act, "mask"))
        if mode == "sigmoid":
            pk.moe_topk_sigmoid_routing_layer(input=pk.attach_input(logits.cuda(), "logits"), bias=pk.attach_input(bias.cuda(), "bias"),
                                              output=outs, grid_dim=(1, 1, 1), block_dim=(256, 1, 1))
        else:
            pk.moe_topk_softmax_routing_layer(input=pk.attach_input(logits.cuda(), "logits"), output=outs, grid_dim=(1, 1, 1),
                                              block_dim=(256, 1, 1))
        pk.compile()
        pk.run_test_mode()
        torch.cuda.synchronize()
        assert pk.status().error == 0
        assert torch.equal(idx.cpu(), idx_ref), f"routing indices differ ({mode}, {B} tokens)"
        n = int(act_ref[-1])
        assert int(act[-1]) == n and set(act[:n].cpu().tolist()) == set(act_ref[:n].tolist())
        assert float((w.cpu() - w_ref).abs().max()) <= 1e-5 * max(1.0, float(w_ref.abs().max()))


def test_paged_attention_matches_the_reference_kernel(fixture):
    """Fused q/k RMSNorm + RoPE + append + causal attention of one request against the reference's
    multitoken_paged_attention kernel (4 query heads, 1 kv head, pages of 4096 rows): output rows to 1e-2 of the largest
    magnitude, the appended K rows likewise, the appended V rows bit-exact."""
    import mirage_b200 as mi
    from gpu_util import make_test_kernel, rel_err
    from golden_inputs import ATTENTION_CASES, attention_case_input
    if "paged_attention" not in fixture:
        pytest.skip("fixture has no paged_attention section")
    for token_budget in (0, 16):                 # the batch-1 instantiation and the one that serves many requests
        for case in ATTENTION_CASES:
            prefix, n_new, page, seed = case
            want = fixture["paged_attention"][case]
            t = attention_case_input(prefix, n_new, seed)
            dev = "cuda"
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
            meta = {"qo_indptr_buffer": i32([0, n_new]), "paged_kv_indptr_buffer": i32([0, 1]),
                    "paged_kv_indices_buffer": i32([page, 1 - page]), "paged_kv_last_page_len_buffer": i32([prefix + n_new])}
            pk = make_test_kernel(mi, max(n_new, token_budget), max_num_batched_requests=1, max_num_pages=2, page_size=4096,
                                  max_seq_length=512, meta_tensors=meta)
            kc, vc = t["k_cache"].unsqueeze(2).cuda(), t["v_cache"].unsqueeze(2).cuda()
            out = torch.zeros(n_new, 4 * 128, dtype=torch.bfloat16, device=dev)
            pk.paged_attention_layer(
                input=pk.attach_input(t["qkv"].cuda(), "qkv"), k_cache=pk.attach_input(kc, "kc"), v_cache=pk.attach_input(vc, "vc"),
                q_norm=pk.attach_input(t["q_norm"].cuda(), "qn"), k_norm=pk.attach_input(t["k_norm"].cuda(), "kn"),
                cos_pos_embed=pk.attach_input(t["cos"].cuda(), "cos"), sin_pos_embed=pk.attach_input(t["sin"].cuda(), "sin"),
                output=pk.attach_input(out, "out"), grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
            pk.compile()
            pk.run_test_mode()
            torch.cuda.synchronize()
            assert pk.status().error == 0
            assert rel_err(out.cpu().reshape(n_new * 4, 128), want["out"]) <= 1e-2, (case, token_budget)
            assert rel_err(kc[page, prefix:prefix + n_new, 0].cpu(), want["k_rows"]) <= 1e-2, (case, token_budget)
            assert torch.equal(vc[page, prefix:prefix + n_new, 0].cpu(), want["v_rows"]), (case, token_budget)

