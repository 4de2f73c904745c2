"""The composed DeepSeek-V3 oracle (oracle/deepseek_v3.py) checked against itself on the CPU: the absorbed latent-space
attention against plain multi-head attention with materialised K / V, and the tensor- / expert-parallel emulation
against the single-rank graph."""
import torch

from oracle import fp8_ops as F
from oracle import mla_ops as A
from oracle import mpk_ops as ops
from oracle.deepseek_v3 import DeepSeekConfig, DeepSeekOracle, make_checkpoint, plain_attention_reference


def _setup(world=1, **kw):
    cfg = DeepSeekConfig.tiny()
    ckpt = make_checkpoint(cfg, seed=1005)
    return cfg, ckpt, DeepSeekOracle(cfg, ckpt, max_num_pages=8, page_size=16, world_size=world, **kw)


def test_absorbed_attention_equals_plain_attention():
    """q_b with W_UK absorbed, the [latent | rope] cache and o_proj with W_UV folded in compute what un-absorbed
    multi-head attention followed by o_proj computes (bf16 rounding of the absorbed weights aside)."""
    cfg, ckpt, orc = _setup()
    n = 6
    g = torch.Generator().manual_seed(3)
    xn = torch.randn(n, cfg.hidden_size, generator=g).to(torch.bfloat16)
    x = torch.zeros(n, cfg.hidden_size, dtype=torch.bfloat16)
    got = orc._attention(0, xn, x, [((0, n), [0], n)]).float()
    a = "model.layers.0.self_attn."
    w = orc.L[0]
    q_a = ops.rmsnorm(w["q_a"](xn), ckpt[a + "q_a_layernorm.weight"], cfg.rms_eps)
    xq, xe, _ = F.quantize_fp8_ue8m0(xn)
    lat = ops.rmsnorm(F.linear_fp8(xq, xe, *w["kv_lat"]), ckpt[a + "kv_a_layernorm.weight"], cfg.rms_eps)
    k_pe = F.linear_fp8(xq, xe, *w["kv_rope"])
    heads_out = plain_attention_reference(cfg, ckpt, 0, q_a, lat, k_pe)
    ref = heads_out @ ckpt[a + "o_proj.weight"].float().T
    err = float((got - ref).abs().max() / ref.abs().max())
    assert err < 3e-2, err


def test_parallel_emulation_matches_single_rank():
    """Heads, MLP columns and experts split over 2 or 4 ranks with bf16 partials: same function, rounding noise only."""
    cfg, ckpt, one = _setup()
    ids = torch.tensor([5, 77, 901, 12])
    reqs = [((0, 2), [0], 2), ((2, 4), [1], 2)]
    ref = one.forward_tokens(ids, reqs).float()
    for world in (2, 4):
        _, _, orc = _setup(world)
        got = orc.forward_tokens(ids, reqs).float()
        assert float((got - ref).abs().max()) < 0.1, world
        assert torch.equal(orc.last_routing, one.last_routing) or float((got - ref).abs().max()) < 0.1


def test_rope_switch_changes_the_result_and_runs():
    cfg, ckpt, plain = _setup()
    _, _, roped = _setup(rope=True)
    ids = torch.tensor([5, 77, 901])
    reqs = [((0, 3), [0], 3)]
    a, b = plain.forward_tokens(ids, reqs).float(), roped.forward_tokens(ids, reqs).float()
    assert torch.isfinite(b).all() and not torch.equal(a, b)
