"""Checkpoint reader: a rank's shard read straight from *.safetensors equals the shard cut from the whole state dict
(the cut demo/qwen3/demo.py:13-29 describes), for bf16 and for FP8 projections with 128 x 128 block scales, with and
without an index file."""
import json

import pytest
import torch
from safetensors.torch import save_file

from mirage_b200.builders.checkpoint import checkpoint_index, load_sharded_state_dict, shape_from_config
from mirage_b200.builders.qwen3 import shard_fp8_state_dict, shard_state_dict


def _state(layers=2, hidden=256, heads=4, kv=2, hd=64, inter=512, vocab=1024, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16)
    sd = {"model.embed_tokens.weight": r(vocab, hidden), "model.norm.weight": r(hidden), "lm_head.weight": r(vocab, hidden)}
    for i in range(layers):
        p = f"model.layers.{i}."
        sd.update({p + "input_layernorm.weight": r(hidden), p + "post_attention_layernorm.weight": r(hidden),
                   p + "self_attn.q_norm.weight": r(hd), p + "self_attn.k_norm.weight": r(hd),
                   p + "self_attn.q_proj.weight": r(heads * hd, hidden), p + "self_attn.k_proj.weight": r(kv * hd, hidden),
                   p + "self_attn.v_proj.weight": r(kv * hd, hidden), p + "self_attn.o_proj.weight": r(hidden, heads * hd),
                   p + "mlp.gate_proj.weight": r(inter, hidden), p + "mlp.up_proj.weight": r(inter, hidden),
                   p + "mlp.down_proj.weight": r(hidden, inter)})
    return sd


@pytest.mark.parametrize("world,shard_lm_head,indexed", [(1, False, False), (2, False, True), (2, True, False), (4, True, True)])
def test_bf16_shards_read_from_disk(tmp_path, world, shard_lm_head, indexed):
    sd = _state()
    keys = sorted(sd)
    if indexed:                                   # two files + an index, as large checkpoints are stored
        half = len(keys) // 2
        parts = {"model-00001-of-00002.safetensors": keys[:half], "model-00002-of-00002.safetensors": keys[half:]}
        for fn, ks in parts.items():
            save_file({k: sd[k] for k in ks}, str(tmp_path / fn))
        (tmp_path / "model.safetensors.index.json").write_text(
            json.dumps({"weight_map": {k: fn for fn, ks in parts.items() for k in ks}}))
    else:
        save_file(sd, str(tmp_path / "model.safetensors"))
    assert set(checkpoint_index(str(tmp_path))) == set(keys)
    for rank in range(world):
        got, fp8 = load_sharded_state_dict(str(tmp_path), world, rank, shard_lm_head=shard_lm_head)
        want = shard_state_dict(sd, world, rank, 4, 2, 64, shard_lm_head=shard_lm_head)
        assert not fp8 and set(got) == set(want)
        for k in want:
            assert got[k].dtype == want[k].dtype and torch.equal(got[k], want[k]), k


def test_fp8_projections_and_scales(tmp_path):
    sd = _state(layers=1, kv=4)               # every shard a multiple of the 128 x 128 scale block
    g = torch.Generator().manual_seed(5)
    stored, fp8_full = {}, {}
    for k, v in sd.items():
        if k.endswith("_proj.weight"):
            q = v.float().clamp(-1, 1).to(torch.float8_e4m3fn)
            sc = torch.rand(v.shape[0] // 128, v.shape[1] // 128, generator=g) * 0.1 + 1e-3
            stored[k], stored[k + "_scale_inv"] = q, sc
            fp8_full[k] = (q, sc)
        else:
            stored[k] = v
    save_file(stored, str(tmp_path / "model.safetensors"))
    for rank in range(2):
        plain, fp8 = load_sharded_state_dict(str(tmp_path), 2, rank)
        want = shard_fp8_state_dict(fp8_full, 2, rank)
        assert set(fp8) == set(want) and not any(k.endswith("_proj.weight") for k in plain)
        for k, (q, sc) in want.items():
            assert torch.equal(fp8[k][0].view(torch.uint8), q.view(torch.uint8)) and torch.equal(fp8[k][1], sc), k
        assert torch.equal(plain["lm_head.weight"], sd["lm_head.weight"])


def test_errors_and_config(tmp_path):
    sd = _state(layers=1)
    save_file(sd, str(tmp_path / "model.safetensors"))
    with pytest.raises(KeyError):
        load_sharded_state_dict(str(tmp_path), names=["model.layers.7.mlp.up_proj.weight"])
    with pytest.raises(ValueError):
        load_sharded_state_dict(str(tmp_path), 3, 0)                  # 256 rows do not split over 3 ranks
    only, _ = load_sharded_state_dict(str(tmp_path), names=["model.norm.weight"], dtype=torch.float32)
    assert list(only) == ["model.norm.weight"] and only["model.norm.weight"].dtype == torch.float32
    with pytest.raises(FileNotFoundError):
        checkpoint_index(str(tmp_path / "nothing"))
    (tmp_path / "config.json").write_text(json.dumps({
        "num_hidden_layers": 1, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
        "intermediate_size": 512, "vocab_size": 1024, "rope_theta": 1e6, "max_position_embeddings": 2048}))
    s = shape_from_config(str(tmp_path))
    assert (s.num_layers, s.num_q_heads, s.head_dim, s.max_position, s.rope_theta) == (1, 4, 64, 2048, 1e6)
