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


def test_unquantised_oracle_matches_huggingface_deepseek_v3():
    """Composition check against an independent implementation: HuggingFace's DeepseekV3ForCausalLM (fp32, plain
    multi-head latent attention, its own router and experts) loaded with the block-dequantised weights of the synthetic
    checkpoint, against this oracle with every FP8 step switched off (`quantize=False`) -- the absorbed q_b / fused
    o_proj attention over the latent cache, rotary embedding in the builder's table convention, grouped sigmoid
    routing, routed + shared experts, dense MLP.  With the same softmax scale (HF uses 1 / sqrt(192) without a YaRN
    configuration) the logits of a 12-token prefill agree to bf16 rounding noise (measured 5.5e-3 of the largest logit;
    bar 2e-2); the same graph without the rotary embedding or with the reference's hard-coded scale is off by 5e-2 and
    1.7e-1, so the bar does separate them.  Also run as two tensor- / expert-parallel ranks."""
    import numpy as np
    from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
    from oracle.batching import BatchState
    from oracle.deepseek_v3 import DeepSeekConfig, DeepSeekOracle, _deq_block, make_checkpoint
    cfg = DeepSeekConfig.tiny()
    ck = make_checkpoint(cfg, 1005)
    hf_cfg = DeepseekV3Config(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
        moe_intermediate_size=cfg.moe_intermediate_size, num_hidden_layers=cfg.num_layers, num_attention_heads=cfg.num_heads,
        num_key_value_heads=cfg.num_heads, n_shared_experts=1, n_routed_experts=cfg.num_experts,
        routed_scaling_factor=cfg.routed_scaling_factor, kv_lora_rank=cfg.kv_lora_rank, q_lora_rank=cfg.q_lora_rank,
        qk_rope_head_dim=cfg.qk_rope_head_dim, v_head_dim=cfg.v_head_dim, qk_nope_head_dim=cfg.qk_nope_head_dim,
        n_group=cfg.n_group, topk_group=cfg.topk_group, num_experts_per_tok=cfg.num_experts_per_tok,
        first_k_dense_replace=cfg.first_moe_layer, norm_topk_prob=True, rms_norm_eps=cfg.rms_eps, rope_interleave=False,
        max_position_embeddings=512, rope_parameters={"rope_type": "default", "rope_theta": 10000.0}, attention_bias=False,
        tie_word_embeddings=False)
    model = DeepseekV3ForCausalLM(hf_cfg).eval()
    sd = {}
    for k, v in ck.items():
        if k.endswith("_scale_inv"):
            continue
        w = _deq_block(v, ck[k + "_scale_inv"]) if (k + "_scale_inv") in ck else v.float()
        sd[k.replace("experts.w13.weight", "experts.gate_up_proj").replace("experts.w2.weight", "experts.down_proj")] = w
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not missing and not unexpected
    prompt = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(7))
    with torch.no_grad():
        hf = model(prompt[None]).logits[0].float()

    def oracle_logits(**kw):
        page, pages = 16, 4
        orc = DeepSeekOracle(cfg, ck, max_num_pages=pages, page_size=page, quantize=False, **kw)
        tokens = np.zeros((1, 64), np.int64)
        tokens[0, :12] = prompt.numpy()
        st = BatchState(tokens, np.array([12], np.int32), max_num_batched_requests=1, max_num_batched_tokens=16,
                        max_num_pages=pages, page_size=page)
        assert orc.run_iteration(st)
        return orc.last_logits.float()

    err = lambda o: float((o - hf).abs().max() / hf.abs().max())
    plain_scale = 192 ** -0.5
    good = oracle_logits(rope=True, softmax_scale=plain_scale)
    assert err(good) <= 2e-2 and torch.equal(good.argmax(-1), hf.argmax(-1))
    assert err(oracle_logits(rope=True, softmax_scale=plain_scale, world_size=2)) <= 2e-2
    assert err(oracle_logits(rope=False, softmax_scale=plain_scale)) > 3e-2            # the check sees a missing rotary embedding
    assert err(oracle_logits(rope=True)) > 3e-2                                        # ... and a different softmax scale
