"""The CPU oracle against the fixtures produced from the reference's own test oracles
and from HuggingFace's Qwen3 (tests/golden/make_golden.py)."""
import os

import numpy as np
import torch

from oracle import mpk_ops as ops
from oracle.qwen3_decoder import Qwen3Config, make_weights, greedy_generate


def _load(golden_dir, name):
    return torch.load(os.path.join(golden_dir, name), weights_only=False)


def test_rmsnorm_matches_reference_oracle(golden_dir):
    f = _load(golden_dir, "ref_rmsnorm.pt")
    out = ops.rmsnorm(f["x"], f["w"], f["eps"])
    # the reference function rounds x*rsqrt to bf16 before the weight multiply; ours rounds once
    torch.testing.assert_close(out.float(), f["out"].float(), rtol=1e-2, atol=1e-2)


def test_rmsnorm_linear_matches_reference_oracle(golden_dir):
    f = _load(golden_dir, "ref_norm_linear.pt")
    out = ops.rmsnorm_linear(f["x"], f["g"].reshape(-1), f["w"], f["eps"])
    ref = f["out_f32"]
    rel = (out.float() - ref).abs().max() / ref.abs().max()
    assert rel < 2e-2, rel


def test_paged_attention_matches_reference_oracle(golden_dir):
    f = _load(golden_dir, "ref_paged_attention.pt")
    kc = f["k_cache"].clone().unsqueeze(2)   # [pages, page, 1 kv head, D]
    vc = f["v_cache"].clone().unsqueeze(2)
    d = 128
    qkv = f["qkv"]
    n = qkv.shape[0]
    out = ops.paged_attention_request(
        qkv, kc, vc, [int(f["page_ids"][0])], int(f["seq_len"]), 4, 1,
        f["q_norm"].reshape(-1), f["k_norm"].reshape(-1), f["cos"], f["sin"], 1e-6)
    ref = f["out"].reshape(n, 4 * d)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    # the appended (normalised + rotated) keys must match what the reference wrote back
    torch.testing.assert_close(kc[:, :, 0, :].float(), f["k_cache_after"].float(), rtol=1e-2, atol=1e-2)


def test_mlp_matches_reference_oracle(golden_dir):
    f = _load(golden_dir, "ref_mlp.pt")
    ng = 4
    w_gu = ops.shuffle_rows([f["w_gate"], f["w_up"]], ng)
    mid = ops.linear(f["x"], w_gu)
    act = ops.silu_mul(mid, ng)
    out = ops.linear(act, f["w_down"], f["residual"])
    torch.testing.assert_close(out.float(), f["out"].float(), rtol=2e-2, atol=2e-2)


def test_allreduce_matches_reference_oracle(golden_dir):
    f = _load(golden_dir, "ref_allreduce.pt")
    out = ops.allreduce(f["parts"])
    torch.testing.assert_close(out.float(), f["out_f32"], rtol=1e-2, atol=1e-2)


def test_shuffle_rows_layout():
    a = torch.arange(8).reshape(4, 2)
    b = 100 + torch.arange(8).reshape(4, 2)
    s = ops.shuffle_rows([a, b], 2)
    assert s[:, 0].tolist() == [0, 2, 100, 102, 4, 6, 104, 106]


def test_embedding_negative_ids_give_zero_rows():
    tab = torch.arange(12, dtype=torch.float32).reshape(4, 3)
    out = ops.embedding(torch.tensor([2, -1]), tab)
    assert out[0].tolist() == [6, 7, 8] and out[1].abs().sum() == 0


def test_argmax_lowest_index_wins():
    assert ops.argmax(torch.tensor([[1.0, 3.0, 3.0, 2.0]])).item() == 1


def test_qwen3_decoder_matches_huggingface(golden_dir):
    """Token-by-token paged decode of the oracle == HF causal prefill logits."""
    f = _load(golden_dir, "qwen3_tiny_hf.pt")
    cfg = Qwen3Config.tiny()
    w = make_weights(cfg, seed=int(f["seed"]))
    ids = f["ids"].tolist()
    st, orc, logits = greedy_generate(
        cfg, w, [ids], max_seq_length=64, max_num_batched_requests=1, max_num_batched_tokens=1,
        max_num_pages=4, page_size=16, max_iterations=len(ids), keep_logits=True)
    got = torch.cat(logits, 0).float()
    ref = f["logits"]
    assert got.shape == ref.shape
    assert (got - ref).abs().max() < 5e-2, (got - ref).abs().max()
    # chunked prefill (4 tokens per iteration) gives the same logits
    st2, _, logits2 = greedy_generate(
        cfg, w, [ids], max_seq_length=64, max_num_batched_requests=1, max_num_batched_tokens=4,
        max_num_pages=4, page_size=16, max_iterations=len(ids) // 4, keep_logits=True)
    got2 = torch.cat(logits2, 0).float()
    assert (got2 - ref).abs().max() < 5e-2


def test_qwen3_decoder_tp_emulation_close_to_tp1():
    cfg = Qwen3Config.tiny()
    w = make_weights(cfg, seed=5)
    kw = dict(max_seq_length=32, max_num_batched_requests=2, max_num_batched_tokens=2,
              max_num_pages=8, page_size=16, max_iterations=6, keep_logits=True)
    _, _, l1 = greedy_generate(cfg, w, [[1, 2, 3], [7, 8]], **kw)
    _, _, l2 = greedy_generate(cfg, w, [[1, 2, 3], [7, 8]], world_size=2, **kw)
    for a, b in zip(l1, l2):
        assert (a.float() - b.float()).abs().max() < 5e-2


def test_fp8_quantize_and_linear_match_reference_helpers(golden_dir):
    from oracle import fp8_ops as f8
    f = _load(golden_dir, "ref_fp8.pt")
    q, exps, packed = f8.quantize_fp8_ue8m0(f["x"])
    assert torch.equal(packed, f["xs"])                                   # scales: exact
    assert torch.equal(q.view(torch.uint8), f["xq"])                     # codes: exact on the CPU
    assert torch.equal(f8.unpack_ue8m0(f["xs"], 4), exps)
    assert torch.equal(f8.dequant(q, f8.decode_ue8m0(exps)), f["x_deq"])
    wq, wexps, wpacked = f8.quantize_fp8_ue8m0(f["w"])
    assert torch.equal(wpacked, f["ws"]) and torch.equal(wq.view(torch.uint8), f["wq"])
    out = f8.linear_fp8(q, exps, wq, wexps, f["residual"])
    torch.testing.assert_close(out.float(), f["out"].float(), rtol=1e-2, atol=1e-2)
    # float32-scale variant: dequantised values stay within one e4m3 step of the input
    q2, s2 = f8.quantize_fp8_f32scale(f["x"])
    err = (f8.dequant(q2, s2) - f["x"].float()).abs()
    assert (err <= f["x"].float().abs() * 0.0626 + s2.repeat_interleave(128, 1) * 2 ** -9 + 1e-6).all()


def test_moe_routing_matches_reference_oracle(golden_dir):
    """oracle/moe_ops.topk_sigmoid_routing against reference_sigmoid_routing
    (tests/runtime_python/blackwell/sm100_moe_sigmoid/test_gate_topk_sigmoid.py:27-76): routing indices and
    the set of active experts bit-exact, weights to fp32 rounding."""
    from oracle import moe_ops as M
    f = torch.load(os.path.join(golden_dir, "ref_moe.pt"), weights_only=False)
    c = f["route_consts"]
    w, routing, active, chosen = M.topk_sigmoid_routing(f["logits"], f["bias"], topk=c["NUM_EXPERTS_PER_TOK"],
                                                        num_groups=c["NUM_GROUPS"], topk_group=c["TOPK_GROUP"],
                                                        scaling=c["ROUTED_SCALING_FACTOR"])
    assert torch.equal(routing, f["routing"])
    n = int(active[-1])
    mask = torch.zeros(c["NUM_EXPERTS"], dtype=torch.int32)
    mask[active[:n].long()] = 1
    assert torch.equal(mask, f["expert_active"])
    assert active[:n].tolist() == sorted(active[:n].tolist())
    torch.testing.assert_close(w, f["weights"], rtol=1e-6, atol=1e-7)
    # ties (which torch.topk leaves unspecified) resolve to the lower group / expert index, as in the kernel
    # (topk_sigmoid_sm100.cuh:252-258, 282-303)
    lg = f["logits"].clone()
    lg[:, 8:16] = lg[:, 0:8]
    b = f["bias"].clone()
    b[8:16] = b[0:8]
    _, _, _, ch = M.topk_sigmoid_routing(lg, b, topk=4, num_groups=8, topk_group=3, scaling=2.5)
    for row in ch.tolist():
        for e in row:
            if 8 <= e < 16:
                assert (e - 8) in row      # the twin with the lower index was taken first


def test_moe_fp8_grouped_gemm_matches_reference_oracle(golden_dir):
    """oracle/moe_ops.moe_gemm_fp8 against reference_moe_w13 / reference_moe_w2
    (tests/runtime_python/blackwell/sm100_fp8_moe/test_fp8_moe_gemm.py:121-190).  The reference rounds the
    de-quantised operands to bf16 before its matmul; the kernels (and this oracle) accumulate the exact e4m3
    products in fp32, so the comparison carries the reference test's own tolerance."""
    from oracle import moe_ops as M
    f = torch.load(os.path.join(golden_dir, "ref_moe.pt"), weights_only=False)
    e4 = torch.float8_e4m3fn
    q, s = M.quantize_fp8_f32(f["x13"])
    assert torch.equal(q.view(torch.uint8), f["x13q"]) and torch.equal(s, f["x13s"])
    out13 = M.moe_gemm_fp8(f["x13q"].view(e4), f["x13s"], f["w13q"].view(e4), f["w13s"], f["g_routing"], topk=2,
                           per_slot_input=False)
    out2 = M.moe_gemm_fp8(f["x2q"].view(e4), f["x2s"], f["w2q"].view(e4), f["w2s"], f["g_routing"], topk=2,
                          per_slot_input=True)
    for got, ref in ((out13, f["out13"]), (out2, f["out2"])):
        err = (got.float() - ref.float()).abs().max() / ref.float().abs().max()
        assert err <= 2e-2
        assert torch.equal(got.float() == 0, ref.float() == 0) or err <= 2e-2


def test_mla_decode_matches_reference_oracle(golden_dir):
    """oracle/mla_ops.mla_decode_request (paged cache, appended rows, causal limits of the new tokens) against
    pytorch_mla_ref (tests/runtime_python/blackwell/sm100_mla/test_mla_mtp.py:44-69)."""
    from oracle import mla_ops as A
    f = torch.load(os.path.join(golden_dir, "ref_mla.pt"), weights_only=False)
    for case in f.values():
        Q, KV, L = case["Q"], case["KV"], case["kv_len"]
        n = Q.shape[1]
        page = 16
        npages = (L + page - 1) // page
        perm = torch.randperm(npages + 3, generator=torch.Generator().manual_seed(L)).tolist()[:npages]
        cache = torch.zeros(npages + 3, page, 576, dtype=torch.bfloat16)
        for p in range(L - n):                         # the old rows are in the cache, the new ones get appended
            cache[perm[p // page], p % page] = KV[0, p]
        A.mla_append(cache, KV[0, L - n:, :512], KV[0, L - n:, 512:], perm, L)
        assert torch.equal(A.gather_rows(cache, perm, L), KV[0])
        out = A.mla_decode_request(Q[0], cache, perm, L, case["scale"])
        assert (out.float() - case["out"][0].float()).abs().max() <= 1e-3


def test_softmax_routing_oracle_equals_the_reference_test_expression():
    """oracle.moe_ops.topk_softmax_routing against the expression the reference's own test checks its kernel with
    (tests/runtime_python/blackwell/sm100_moe/test_gate_topk.py:34-52): softmax, torch.topk, renormalise, 1-based slots."""
    import torch
    from oracle import moe_ops as M
    g = torch.Generator().manual_seed(1234)
    for e in (128, 256):
        logits = torch.randn(5, e, generator=g)      # fp32: no equal values, whose order torch.topk leaves unspecified
        f = logits.float()
        sm = torch.softmax(f - f.amax(dim=1, keepdim=True), dim=1, dtype=torch.float)
        vals, ids = torch.topk(sm, 8, dim=1)
        want_w = vals / vals.sum(dim=-1, keepdim=True)
        want_r = torch.zeros(e, 5, dtype=torch.int32)
        for t in range(5):
            for k in range(8):
                want_r[ids[t, k], t] = k + 1
        w, r, active, chosen = M.topk_softmax_routing(logits, topk=8)
        assert torch.equal(chosen, ids) and torch.equal(r, want_r)
        assert torch.allclose(w, want_w, rtol=1e-6, atol=0)
        assert int(active[e]) == int((want_r != 0).any(1).sum())
