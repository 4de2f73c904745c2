"""The rounding noise floor of the 2-rank tensor-parallel decoder at the shape tests/test_gpu_tp_single_device.py uses,
measured on the CPU oracle alone: the measurement behind that test's logit bar."""
import torch

from oracle.qwen3_decoder import Qwen3Config, Qwen3Oracle, make_weights


def test_one_ulp_upstream_moves_tp_logits_by_two_bf16_steps():
    cfg = Qwen3Config(num_layers=2, vocab_size=8192, max_position=256)
    w = make_weights(cfg, seed=1007)
    ids = torch.randint(0, 8192, (16,), generator=torch.Generator().manual_seed(3))
    reqs = [((b, b + 1), [b], 1) for b in range(16)]
    emb = w["model.embed_tokens.weight"].clone()
    flip = torch.rand(emb.shape, generator=torch.Generator().manual_seed(9)) < 0.02   # one bf16 step on 2% of the entries
    bits = emb.view(torch.int16)
    bits[flip] += 1
    w2 = dict(w)
    w2["model.embed_tokens.weight"] = bits.view(torch.bfloat16)
    kw = dict(max_num_pages=32, page_size=16, world_size=2, residual_after_sum=True)
    a = Qwen3Oracle(cfg, w, **kw).forward_tokens(ids, reqs).float()
    b = Qwen3Oracle(cfg, w2, **kw).forward_tokens(ids, reqs).float()
    d = (a - b).abs()
    beyond = int((d > 5e-2).sum())
    print(f"one-ulp perturbation of 2% of the embedding: TP=2 logits (max |x| {float(a.abs().max()):.2f}) move by "
          f"{float(d.max()):.4f}; {beyond} of {d.numel()} entries beyond 5e-2")
    assert 0.03 < float(d.max()) <= 0.1
    assert beyond <= d.numel() // 2000
