"""Layer sequence of a Qwen3-architecture decoder on a `PersistentKernel`.

Emits the same graph as the reference's Qwen3Builder
(python/mirage/mpk/models/qwen3/builder.py:252-646): embed, then per layer
rmsnorm -> qkv linear (weights interleaved per kv head as [q x G | k | v]) ->
paged attention with QK-norm and RoPE -> o_proj + residual [-> allreduce] -> rmsnorm ->
gate_up linear (gate/up interleaved in groups) -> silu_mul -> down_proj + residual
[-> allreduce], then final rmsnorm -> lm_head -> argmax partial/reduce.

Differences, all on the host side: the lm_head is not padded to 153600 rows (the library cuts a
linear into row panels of any size), and with tensor parallelism the row-parallel projections are
registered as linear_with_residual_layer + allreduce_layer so that the residual is added exactly
once (the reference's B200 split-K variant accumulates it on every rank before the allreduce,
builder.py:379-408).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from ..mpk import register_model_builder
from ..persistent_kernel import DTensor, PersistentKernel, bfloat16, int64


def grid_for_rmsnorm_linear_layer(size: int) -> int:
    """Task-count heuristic of python/mirage/mpk/models/utils.py:3-16; here it only fixes the number of
    gate/up interleave groups so that weight layouts match the reference's."""
    if size / 96 > 400:
        assert size % 256 == 0
        return size // 256
    if size % 96 == 0:
        return 96
    if size % 64 == 0:
        return 64
    raise ValueError(f"unsupported fused width {size}")


@dataclass
class Qwen3ModelConfig:
    """What MirageModelConfig carries in the reference (python/mirage/mpk/models/graph_builder.py)."""
    hidden_size: int
    intermediate_size: int          # local (already divided by world_size)
    vocab_size: int
    local_num_q_heads: int
    local_num_kv_heads: int
    head_dim: int
    num_layers: int
    k_cache: torch.Tensor           # [layers, max_num_pages, page_size, local_kv_heads, head_dim]
    v_cache: torch.Tensor
    position_embeddings: Tuple[torch.Tensor, torch.Tensor]   # cos, sin: [positions, head_dim] bf16
    state_dict: Dict[str, torch.Tensor]                       # this rank's shard, HF names
    with_lm_head: bool = True
    sampling_seed: Optional[int] = None   # None: greedy argmax; an int: Gumbel-max sampling (demo/qwen3/demo_sampling.py)


def shard_state_dict(sd: Dict[str, torch.Tensor], world_size: int, rank: int, num_q_heads: int,
                     num_kv_heads: int, head_dim: int) -> Dict[str, torch.Tensor]:
    """Tensor-parallel shard of a full HF-named Qwen3 state dict, as demo/qwen3/demo.py:13-29 lays it out:
    q/k/v and gate/up by output rows, o_proj/down_proj by input columns, everything else replicated."""
    if world_size == 1:
        return sd
    out = {}
    for k, v in sd.items():
        if k.endswith(("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate_proj.weight", "up_proj.weight")):
            n = v.shape[0] // world_size
            out[k] = v[rank * n:(rank + 1) * n].contiguous()
        elif k.endswith(("o_proj.weight", "down_proj.weight")):
            n = v.shape[1] // world_size
            out[k] = v[:, rank * n:(rank + 1) * n].contiguous()
        else:
            out[k] = v
    return out


@register_model_builder("qwen3", "Qwen3")
class Qwen3Builder:
    def __init__(self, mpk: PersistentKernel):
        self.mpk = mpk
        self.world_size, self.rank = mpk.world_size, mpk.mpi_rank
        self.input_tokens = mpk.meta_tensors.get("input_tokens")
        self.output_tokens = mpk.meta_tensors.get("output_tokens")
        self.logits: Optional[DTensor] = None

    def build_from_config(self, c: Qwen3ModelConfig):
        mpk, sd = self.mpk, c.state_dict
        mbt = mpk.max_num_batched_tokens
        tp = self.world_size > 1
        sym = "nvshmem_tensor" if tp else "cuda_tensor"
        qkv_width = (c.local_num_q_heads + 2 * c.local_num_kv_heads) * c.head_dim
        new = lambda name, w, cat="cuda_tensor": mpk.new_tensor(dims=(mbt, w), dtype=bfloat16, name=name, io_category=cat)

        x_in = mpk.attach_input(self.input_tokens, name="input_token")
        cos = mpk.attach_input(c.position_embeddings[0], name="cos_position_embedding")
        sin = mpk.attach_input(c.position_embeddings[1], name="sin_position_embedding")
        x = new("embed_out", c.hidden_size)
        rmsnorm_out = new("rmsnorm_out", c.hidden_size)
        attn_in = new("attn_in", qkv_width)
        attn_out = new("attn_out", c.local_num_q_heads * c.head_dim)
        attn_proj_out = new("attn_proj_out", c.hidden_size, sym)
        allreduce_buf = mpk.new_tensor(dims=(self.world_size, mbt, c.hidden_size), dtype=bfloat16,
                                       name="all_reduce_buf", io_category=sym) if tp else None
        attn_allreduce_out = new("attn_allreduce_out", c.hidden_size, sym) if tp else None
        mlp_mid = new("mlp_mid", 2 * c.intermediate_size)
        silu_mul_out = new("silu_mul_out", c.intermediate_size)
        mlp_out = new("mlp_out", c.hidden_size, sym)
        mlp_final = new("mlp_final", c.hidden_size, sym) if tp else None

        embed_w = mpk.attach_input(sd["model.embed_tokens.weight"], name="embed_tokens")
        mpk.embed_layer(input=x_in, weight=embed_w, output=x, grid_dim=(1, 1, 1), block_dim=(128, 1, 1),
                        input_source=1)

        gu_tasks = grid_for_rmsnorm_linear_layer(2 * c.intermediate_size)
        for i in range(c.num_layers):
            p = f"model.layers.{i}."
            att = lambda key, nm: mpk.attach_input(sd[p + key], name=f"layer_{i}_{nm}")
            w_norm = att("input_layernorm.weight", "input_layernorm")
            w_qkv = mpk.shuffle_tensors(
                inputs=[att("self_attn.q_proj.weight", "q_proj"), att("self_attn.k_proj.weight", "k_proj"),
                        att("self_attn.v_proj.weight", "v_proj")],
                shuffled_dim=0, num_groups=c.local_num_kv_heads, name=f"layer_{i}_qkv_proj")
            mpk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
            mpk.linear_layer(input=rmsnorm_out, weight=w_qkv, output=attn_in,
                             grid_dim=(grid_for_rmsnorm_linear_layer(w_qkv.dim(0)), 1, 1), block_dim=(128, 1, 1))
            mpk.paged_attention_layer(
                input=attn_in, k_cache=mpk.attach_input(c.k_cache[i], name=f"layer_{i}_k_cache"),
                v_cache=mpk.attach_input(c.v_cache[i], name=f"layer_{i}_v_cache"),
                q_norm=att("self_attn.q_norm.weight", "q_norm"), k_norm=att("self_attn.k_norm.weight", "k_norm"),
                cos_pos_embed=cos, sin_pos_embed=sin, output=attn_out,
                grid_dim=(mpk.max_num_batched_requests, c.local_num_kv_heads, 1), block_dim=(128, 1, 1))
            w_o = att("self_attn.o_proj.weight", "o_proj")
            mpk.linear_with_residual_layer(input=attn_out, weight=w_o, residual=x, output=attn_proj_out,
                                           grid_dim=(c.hidden_size // 64, 1, 1), block_dim=(128, 1, 1))
            x_prev, x = x, attn_proj_out
            if tp:
                mpk.allreduce_layer(input=attn_proj_out, buffer=allreduce_buf, output=attn_allreduce_out,
                                    grid_dim=(c.hidden_size // 64, 1, 1), block_dim=(128, 1, 1))
                x = attn_allreduce_out
            w_norm = att("post_attention_layernorm.weight", "post_attn_layernorm")
            w_gu = mpk.shuffle_tensors(
                inputs=[att("mlp.gate_proj.weight", "gate_proj"), att("mlp.up_proj.weight", "up_proj")],
                shuffled_dim=0, num_groups=gu_tasks // 2, name=f"layer_{i}_gatedup_proj")
            mpk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
            mpk.linear_layer(input=rmsnorm_out, weight=w_gu, output=mlp_mid, grid_dim=(gu_tasks, 1, 1),
                             block_dim=(128, 1, 1))
            mpk.silu_mul_layer(input=mlp_mid, output=silu_mul_out, grid_dim=(gu_tasks // 2, 1, 1),
                               block_dim=(128, 1, 1))
            w_d = att("mlp.down_proj.weight", "down_proj")
            # ping-pong the residual stream between two buffers so that no layer writes the tensor it adds
            out_buf = mlp_out if x is not mlp_out else x_prev
            mpk.linear_with_residual_layer(input=silu_mul_out, weight=w_d, residual=x, output=out_buf,
                                           grid_dim=(c.hidden_size // 64, 1, 1), block_dim=(128, 1, 1))
            x = out_buf
            if tp:
                mpk.allreduce_layer(input=out_buf, buffer=allreduce_buf, output=mlp_final,
                                    grid_dim=(c.hidden_size // 64, 1, 1), block_dim=(128, 1, 1))
                x = mlp_final
        self.hidden = x
        w_norm = mpk.attach_input(sd["model.norm.weight"], name="model_norm_weight")
        mpk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
        if not c.with_lm_head:
            return
        lm_head = mpk.attach_input(sd["lm_head.weight"], name="lm_head")
        self.logits = new("argmax_in", c.vocab_size)
        if c.sampling_seed is not None:
            argmax_out = mpk.attach_input(self.output_tokens, name="output_token")
            mpk.linear_layer(input=rmsnorm_out, weight=lm_head, output=self.logits,
                             grid_dim=(96, 1, 1), block_dim=(128, 1, 1))
            mpk.sampling_sm100_layer(logits=self.logits, output=argmax_out, grid_dim=(mbt, 1, 1),
                                     block_dim=(256, 1, 1), seed=c.sampling_seed)
            return
        n_part = mpk.num_workers
        part_v = mpk.new_tensor(dims=(mbt, n_part), dtype=bfloat16, name="argmax_part_value")
        part_i = mpk.new_tensor(dims=(mbt, n_part), dtype=int64, name="argmax_part_index")
        argmax_out = mpk.attach_input(self.output_tokens, name="output_token")
        mpk.linear_layer(input=rmsnorm_out, weight=lm_head, output=self.logits,
                         grid_dim=(96, 1, 1), block_dim=(128, 1, 1))
        mpk.argmax_partial_layer(input=self.logits, output=(part_v, part_i), grid_dim=(n_part, 1, 1),
                                 block_dim=(128, 1, 1))
        mpk.argmax_reduce_layer(input=(part_v, part_i), output=argmax_out, grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
