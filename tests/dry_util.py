"""Dry-run (no CUDA call) construction of Qwen3 graphs: shapes come from meta tensors."""
import torch

import mirage_b200 as mi
from mirage_b200.builders.qwen3 import Qwen3Builder, Qwen3ModelConfig


def meta_state_dict(cfg, world=1, shard_lm_head=False):
    h, d = cfg.hidden_size, cfg.head_dim
    mk = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device="meta")
    w = {"model.embed_tokens.weight": mk(cfg.vocab_size, h), "model.norm.weight": mk(h),
         "lm_head.weight": mk(cfg.vocab_size // (world if shard_lm_head else 1), h)}
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = mk(h)
        w[p + "post_attention_layernorm.weight"] = mk(h)
        w[p + "self_attn.q_proj.weight"] = mk(cfg.num_q_heads * d // world, h)
        w[p + "self_attn.k_proj.weight"] = mk(cfg.num_kv_heads * d // world, h)
        w[p + "self_attn.v_proj.weight"] = mk(cfg.num_kv_heads * d // world, h)
        w[p + "self_attn.q_norm.weight"] = mk(d)
        w[p + "self_attn.k_norm.weight"] = mk(d)
        w[p + "self_attn.o_proj.weight"] = mk(h, cfg.num_q_heads * d // world)
        w[p + "mlp.gate_proj.weight"] = mk(cfg.intermediate_size // world, h)
        w[p + "mlp.up_proj.weight"] = mk(cfg.intermediate_size // world, h)
        w[p + "mlp.down_proj.weight"] = mk(h, cfg.intermediate_size // world)
    return w


def dry_qwen3(cfg, *, mbt=1, mbr=1, world=1, rank=0, pages=32, page=64, max_seq=2048, num_workers=0,
              shard_lm_head=False):
    i32 = lambda *s: torch.empty(*s, dtype=torch.int32, device="meta")
    i64 = lambda *s: torch.empty(*s, dtype=torch.int64, device="meta")
    meta = dict(step=i32(mbr), tokens=i64(mbr, max_seq), input_tokens=i64(mbt, 1), output_tokens=i64(mbt, 1),
                num_new_tokens=i32(mbr), prompt_lengths=i32(mbr), qo_indptr_buffer=i32(mbr + 1),
                paged_kv_indptr_buffer=i32(mbr + 1), paged_kv_indices_buffer=i32(pages),
                paged_kv_last_page_len_buffer=i32(mbr))
    pk = mi.PersistentKernel(mode="offline", world_size=world, mpi_rank=rank, num_workers=num_workers,
                             max_seq_length=max_seq, max_num_batched_requests=mbr, max_num_batched_tokens=mbt,
                             max_num_pages=pages, page_size=page, meta_tensors=meta, dry_run=True)
    kc = torch.empty(cfg.num_layers, pages, page, cfg.num_kv_heads // world, cfg.head_dim, dtype=torch.bfloat16,
                     device="meta")
    rope = torch.empty(4096, cfg.head_dim, dtype=torch.bfloat16, device="meta")
    mc = Qwen3ModelConfig(cfg.hidden_size, cfg.intermediate_size // world, cfg.vocab_size, cfg.num_q_heads // world,
                          cfg.num_kv_heads // world, cfg.head_dim, cfg.num_layers, kc, kc, (rope, rope),
                          meta_state_dict(cfg, world, shard_lm_head))
    Qwen3Builder(pk).build_from_config(mc)
    pk.compile()
    return pk
