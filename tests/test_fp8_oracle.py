"""CPU checks of the FP8 decoder oracle and of the host weight preparation the builder uses."""
import torch

from fp8_util import fp8_checkpoint
from oracle import fp8_ops as F
from oracle.qwen3_decoder import Qwen3Config, Qwen3Fp8Oracle, make_weights


def test_host_requantisation_equals_the_oracle_quantiser():
    """mirage_b200.builders.fp8_prep (product code: de-quantise with the block scales, power-of-two scale per row and
    128 columns rounded up, quantise again, pack four exponents per word) against oracle.fp8_ops, which is pinned to the
    reference's helper module: bytes, exponents and packed words identical."""
    from mirage_b200.builders import fp8_prep as P
    g = torch.Generator().manual_seed(1)
    wq, scale = P.synthetic_block_scaled_weight(300, 1024, g)
    q, packed, exps = P.requantize_for_ue8m0(wq, scale)
    q2, e2, p2 = F.quantize_fp8_ue8m0(P.dequantize_block_scaled(wq, scale))
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8))
    assert torch.equal(exps, e2)
    assert torch.equal(packed.view(torch.int32).to(torch.int64) & 0xFFFFFFFF, p2)
    assert packed.stride() == (1, 300)           # words of one packed column are contiguous over the rows
    assert torch.equal(P.packed_rows_contiguous(packed).view(torch.int32), packed.view(torch.int32))


def test_power_of_two_requantisation_gap_is_small():
    """The kernels implement the reference's host re-quantisation (power-of-two scales); against the checkpoint's
    exact float32 block scales the logits move by a bounded amount, measured here on the CPU oracle alone (the gap is
    reported; the bound only guards against a broken re-quantiser)."""
    cfg = Qwen3Config(num_layers=2, hidden_size=512, num_q_heads=4, num_kv_heads=2, head_dim=128, intermediate_size=512,
                      vocab_size=512, max_position=64)
    w = make_weights(cfg, seed=5)
    fp8 = fp8_checkpoint(cfg, w, seed=6)
    ids = torch.tensor([3, 17, 400])
    reqs = [((0, 3), [0], 3)]
    a = Qwen3Fp8Oracle(cfg, w, fp8, max_num_pages=2, page_size=16).forward_tokens(ids, reqs).float()
    b = Qwen3Fp8Oracle(cfg, w, fp8, exact_scales=True, max_num_pages=2, page_size=16).forward_tokens(ids, reqs).float()
    gap = float((a - b).abs().max())
    print(f"max |logit| difference, power-of-two vs exact float32 block scales: {gap:.4f}")
    assert gap < 0.25


def test_fp8_decoder_noise_floor():
    """How far one-ulp bf16 differences upstream move the logits of the FP8 decoder used by the GPU end-to-end test
    (tests/test_gpu_qwen3_fp8.py), compared with the bf16 decoder of the same weights: the measurement behind that
    test's tolerance."""
    from mirage_b200.builders import fp8_prep as P
    from oracle.qwen3_decoder import Qwen3Oracle
    cfg = Qwen3Config(num_layers=2, hidden_size=2048, num_q_heads=16, num_kv_heads=4, head_dim=128, intermediate_size=2048,
                      vocab_size=1024, max_position=256)
    w = make_weights(cfg, seed=1010)
    fp8 = fp8_checkpoint(cfg, w, seed=77)
    ids = torch.randint(0, 1024, (16,), generator=torch.Generator().manual_seed(3))
    reqs = [((b, b + 1), [b], 1) for b in range(16)]
    emb = w["model.embed_tokens.weight"].clone()
    flip = torch.rand(emb.shape, generator=torch.Generator().manual_seed(9)) < 0.02
    bits = emb.view(torch.int16)
    bits[flip] += 1
    w2 = dict(w)
    w2["model.embed_tokens.weight"] = bits.view(torch.bfloat16)
    kw = dict(max_num_pages=32, page_size=16)
    d_fp8 = float((Qwen3Fp8Oracle(cfg, w, fp8, **kw).forward_tokens(ids, reqs).float() -
                   Qwen3Fp8Oracle(cfg, w2, fp8, **kw).forward_tokens(ids, reqs).float()).abs().max())
    wd = dict(w)
    for k, (q, s) in fp8.items():
        wd[k] = P.dequantize_block_scaled(q, s).to(torch.bfloat16)
    wd2 = dict(wd)
    wd2["model.embed_tokens.weight"] = w2["model.embed_tokens.weight"]
    d_bf16 = float((Qwen3Oracle(cfg, wd, **kw).forward_tokens(ids, reqs).float() -
                    Qwen3Oracle(cfg, wd2, **kw).forward_tokens(ids, reqs).float()).abs().max())
    print(f"one-ulp perturbation of 2% of the embedding: FP8 decoder logits move by {d_fp8:.3f}, bf16 decoder by {d_bf16:.3f}")
    assert d_bf16 < 5e-2 < d_fp8 < 0.35


def test_fp8_oracle_tensor_parallel_emulation_is_close_to_one_rank():
    """Row-parallel projections cut over 2 ranks with bf16 partials: the same function up to rounding noise."""
    cfg = Qwen3Config(num_layers=2, hidden_size=512, num_q_heads=4, num_kv_heads=2, head_dim=128, intermediate_size=512,
                      vocab_size=512, max_position=64)
    w = make_weights(cfg, seed=5)
    fp8 = fp8_checkpoint(cfg, w, seed=6)
    ids = torch.tensor([3, 17, 400])
    reqs = [((0, 3), [0], 3)]
    a = Qwen3Fp8Oracle(cfg, w, fp8, max_num_pages=2, page_size=16).forward_tokens(ids, reqs).float()
    b = Qwen3Fp8Oracle(cfg, w, fp8, max_num_pages=2, page_size=16, world_size=2).forward_tokens(ids, reqs).float()
    assert float((a - b).abs().max()) < 0.2 and not torch.equal(a, b)
