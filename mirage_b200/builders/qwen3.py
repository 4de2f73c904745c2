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
from ..persistent_kernel import DTensor, PersistentKernel, bfloat16, float8_e4m3, int64, uint32
from . import fp8_prep


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
    # FP8 decoder layers: HF name of a projection weight -> (e4m3 [N, K], float32 128 x 128 block scales), this rank's
    # shard.  When given, the seven projections of every layer run as quantize_fp8 + linear_fp8 tasks on these
    # weights (re-quantised to power-of-two scales at build time); embedding, norms and lm_head stay bf16.
    fp8_state_dict: Optional[Dict[str, Tuple[torch.Tensor, torch.Tensor]]] = None


def shard_state_dict(sd: Dict[str, torch.Tensor], world_size: int, rank: int, num_q_heads: int,
                     num_kv_heads: int, head_dim: int, shard_lm_head: bool = True) -> Dict[str, torch.Tensor]:
    """Tensor-parallel shard of a full HF-named Qwen3 state dict, as demo/qwen3/demo.py:13-29 lays it out:
    q/k/v and gate/up by output rows, o_proj/down_proj by input columns, everything else replicated -- except, with
    `shard_lm_head`, the lm_head, which the reference keeps whole on every rank: here rank r gets vocabulary rows
    [r V / world, (r + 1) V / world) and the builder merges the ranks' argmax results (`argmax_exchange_layer`)."""
    if world_size == 1:
        return sd
    out = {}
    for k, v in sd.items():
        if k == "lm_head.weight" and shard_lm_head and v.shape[0] % world_size == 0:
            n = v.shape[0] // world_size
            out[k] = v[rank * n:(rank + 1) * n].contiguous()
            continue
        if k.endswith(("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate_proj.weight", "up_proj.weight")):
            n = v.shape[0] // world_size
            out[k] = v[rank * n:(rank + 1) * n].contiguous()
        elif k.endswith(("o_proj.weight", "down_proj.weight")):
            n = v.shape[1] // world_size
            out[k] = v[:, rank * n:(rank + 1) * n].contiguous()
        else:
            out[k] = v
    return out


def shard_fp8_state_dict(fp8: Dict[str, Tuple[torch.Tensor, torch.Tensor]], world_size: int, rank: int):
    """Tensor-parallel shard of FP8 projections given as (e4m3 [N, K], float32 128 x 128 block scales): q/k/v and gate/up
    by output rows, o_proj/down_proj by input columns; the block scales are cut along with their 128-row / 128-column
    blocks (the shard sizes must be multiples of 128)."""
    if world_size == 1:
        return fp8
    out = {}
    for k, (q, sc) in fp8.items():
        if k.endswith(("o_proj.weight", "down_proj.weight")):
            n = q.shape[1] // world_size
            assert n % 128 == 0, k
            out[k] = (q[:, rank * n:(rank + 1) * n].contiguous(), sc[:, rank * n // 128:(rank + 1) * n // 128].contiguous())
        else:
            n = q.shape[0] // world_size
            assert n % 128 == 0, k
            out[k] = (q[rank * n:(rank + 1) * n].contiguous(), sc[rank * n // 128:(rank + 1) * n // 128].contiguous())
    return out


@register_model_builder("qwen3", "Qwen3")
class Qwen3Builder:
    def _build_layers_fp8(self, c, x, rmsnorm_out, attn_in, attn_out, attn_proj_out, mlp_mid, silu_mul_out, mlp_out,
                          cos, sin, gu_tasks):
        """Decoder layers with e4m3 projections: every projection is `quantize_fp8_layer` on its bf16 input followed by
        `linear_fp8[_with_residual]_layer`, the chain the reference's builders emit for FP8 checkpoints
        (python/mirage/mpk/models/deepseek_v3/builder.py:118-207); q/k/v and gate/up weights -- and their scale rows --
        are interleaved exactly as the bf16 path interleaves them."""
        mpk, sd = self.mpk, c.state_dict
        mbt = mpk.max_num_batched_tokens
        self._keep = []

        def act_buffers(width, tag):
            q = mpk.new_tensor(dims=(mbt, width), dtype=float8_e4m3, name=f"fp8_act_{tag}", io_category="cuda_tensor")
            sc = mpk.new_tensor(dims=((width // 128 + 3) // 4, (mbt + 3) // 4 * 4), dtype=uint32, name=f"fp8_act_scale_{tag}",
                                io_category="cuda_tensor")
            return q, sc

        def prepared(name):
            wq, scale_inv = c.fp8_state_dict[name]
            q, packed, _ = fp8_prep.requantize_for_ue8m0(wq, scale_inv)
            rows = fp8_prep.packed_rows_contiguous(packed)
            self._keep += [q, rows]
            return q, rows

        tp = self.world_size > 1
        if tp:
            ar_buf = mpk.new_tensor(dims=(self.world_size, mbt, c.hidden_size), dtype=bfloat16, name="fp8_all_reduce_buf",
                                    io_category="nvshmem_tensor")

        def row_parallel(q_in, s_in, w, ws, residual, tag):
            """Tensor-parallel o_proj / down_proj: this rank's partial product, summed over the ranks by an allreduce
            (the FP8 linear has no push epilogue: the library puts a push stage in front), residual added once."""
            part = mpk.new_tensor(dims=(mbt, c.hidden_size), dtype=bfloat16, name=tag + "_partial", io_category="nvshmem_tensor")
            mpk.linear_fp8_layer(input_fp8=q_in, input_scale=s_in, weight_fp8=w, weight_scale=ws, output=part,
                                 grid_dim=(c.hidden_size // 64, 1, 1), block_dim=(128, 1, 1))
            summed = mpk.new_tensor(dims=(mbt, c.hidden_size), dtype=bfloat16, name=tag + "_summed", io_category="nvshmem_tensor")
            mpk.allreduce_layer(input=part, buffer=ar_buf, output=summed, grid_dim=(c.hidden_size // 64, 1, 1),
                                block_dim=(128, 1, 1))
            out = mpk.new_tensor(dims=(mbt, c.hidden_size), dtype=bfloat16, name=tag + "_out", io_category="cuda_tensor")
            mpk.elementwise_add_layer(input_a=residual, input_b=summed, output=out, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
            return out

        h_q, h_s = act_buffers(c.hidden_size, "hidden")
        a_q, a_s = act_buffers(c.local_num_q_heads * c.head_dim, "attn")
        m_q, m_s = act_buffers(c.intermediate_size, "mlp")
        for i in range(c.num_layers):
            p = f"model.layers.{i}."
            att = lambda key, nm: mpk.attach_input(sd[p + key], name=f"layer_{i}_{nm}")

            def fp8_pair(keys, nm, groups=None):
                prep = [prepared(p + k) for k in keys]
                if len(prep) == 1:
                    return mpk.attach_input(prep[0][0], name=f"layer_{i}_{nm}"), mpk.attach_input(prep[0][1], name=f"layer_{i}_{nm}_scale")
                wq = mpk.shuffle_tensors(inputs=[mpk.attach_input(q, name=f"layer_{i}_{nm}_{j}") for j, (q, _) in enumerate(prep)],
                                         shuffled_dim=0, num_groups=groups, name=f"layer_{i}_{nm}")
                ws = mpk.shuffle_tensors(inputs=[mpk.attach_input(r, name=f"layer_{i}_{nm}_scale_{j}") for j, (_, r) in enumerate(prep)],
                                         shuffled_dim=0, num_groups=groups, name=f"layer_{i}_{nm}_scale")
                return wq, ws

            def quantize(src, q, sc):
                mpk.quantize_fp8_layer(input=src, output_fp8=q, output_scale=sc, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))

            w_qkv, s_qkv = fp8_pair(["self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight"], "qkv_proj",
                                    c.local_num_kv_heads)
            mpk.rmsnorm_layer(input=x, weight=att("input_layernorm.weight", "input_layernorm"), output=rmsnorm_out,
                              grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
            quantize(rmsnorm_out, h_q, h_s)
            mpk.linear_fp8_layer(input_fp8=h_q, input_scale=h_s, weight_fp8=w_qkv, weight_scale=s_qkv, output=attn_in,
                                 grid_dim=(96, 1, 1), block_dim=(128, 1, 1))
            mpk.paged_attention_layer(
                input=attn_in, k_cache=mpk.attach_input(c.k_cache[i], name=f"layer_{i}_k_cache"),
                v_cache=mpk.attach_input(c.v_cache[i], name=f"layer_{i}_v_cache"),
                q_norm=att("self_attn.q_norm.weight", "q_norm"), k_norm=att("self_attn.k_norm.weight", "k_norm"),
                cos_pos_embed=cos, sin_pos_embed=sin, output=attn_out,
                grid_dim=(mpk.max_num_batched_requests, c.local_num_kv_heads, 1), block_dim=(128, 1, 1))
            w_o, s_o = fp8_pair(["self_attn.o_proj.weight"], "o_proj")
            quantize(attn_out, a_q, a_s)
            if tp:
                x = row_parallel(a_q, a_s, w_o, s_o, x, f"layer_{i}_attn")
                x_prev = x
            else:
                mpk.linear_fp8_with_residual_layer(input_fp8=a_q, input_scale=a_s, weight_fp8=w_o, weight_scale=s_o, residual=x,
                                                   output=attn_proj_out, grid_dim=(c.hidden_size // 64, 1, 1), block_dim=(128, 1, 1))
                x_prev, x = x, attn_proj_out
            w_gu, s_gu = fp8_pair(["mlp.gate_proj.weight", "mlp.up_proj.weight"], "gatedup_proj", gu_tasks // 2)
            mpk.rmsnorm_layer(input=x, weight=att("post_attention_layernorm.weight", "post_attn_layernorm"), output=rmsnorm_out,
                              grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
            quantize(rmsnorm_out, h_q, h_s)
            mpk.linear_fp8_layer(input_fp8=h_q, input_scale=h_s, weight_fp8=w_gu, weight_scale=s_gu, output=mlp_mid,
                                 grid_dim=(gu_tasks, 1, 1), block_dim=(128, 1, 1))
            mpk.silu_mul_layer(input=mlp_mid, output=silu_mul_out, grid_dim=(gu_tasks // 2, 1, 1), block_dim=(128, 1, 1))
            w_d, s_d = fp8_pair(["mlp.down_proj.weight"], "down_proj")
            quantize(silu_mul_out, m_q, m_s)
            if tp:
                x = row_parallel(m_q, m_s, w_d, s_d, x, f"layer_{i}_mlp")
                continue
            out_buf = mlp_out if x is not mlp_out else x_prev
            mpk.linear_fp8_with_residual_layer(input_fp8=m_q, input_scale=m_s, weight_fp8=w_d, weight_scale=s_d, residual=x,
                                               output=out_buf, grid_dim=(c.hidden_size // 64, 1, 1), block_dim=(128, 1, 1))
            x = out_buf
        return x

    def __init__(self, mpk: PersistentKernel):
        self.mpk = mpk
        self.world_size, self.rank = mpk.world_size, mpk.mpi_rank
        self.input_tokens = mpk.meta_tensors.get("input_tokens")
        self.output_tokens = mpk.meta_tensors.get("output_tokens")
        self.logits: Optional[DTensor] = None
        self.rmsnorm_out: Optional[DTensor] = None

    @property
    def returned_hidden_state(self) -> torch.Tensor:
        """[max_num_batched_tokens, hidden] bf16 view of the buffer that holds the final-norm output after a run: what
        `MPK.__call__` hands back in online_notoken mode without an lm_head (python/mirage/mpk/mpk.py:424-426,
        models/qwen3/builder.py:124-126)."""
        return self.mpk.tensor_as_torch(self.rmsnorm_out)

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
        if c.fp8_state_dict is not None:
            x = self._build_layers_fp8(c, x, rmsnorm_out, attn_in, attn_out, attn_proj_out, mlp_mid, silu_mul_out, mlp_out,
                                       cos, sin, gu_tasks)
        for i in range(c.num_layers if c.fp8_state_dict is None else 0):
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
        self.rmsnorm_out = rmsnorm_out     # after the final norm below: the last hidden state a caller without lm_head gets back
        w_norm = mpk.attach_input(sd["model.norm.weight"], name="model_norm_weight")
        mpk.rmsnorm_layer(input=x, weight=w_norm, output=rmsnorm_out, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
        if not c.with_lm_head:
            return
        lm_head = mpk.attach_input(sd["lm_head.weight"], name="lm_head")
        # a vocabulary-sharded lm_head (fewer rows than the vocabulary): this rank owns columns [first, first + rows)
        v_local = int(sd["lm_head.weight"].shape[0])
        self.vocab_first = mpk.mpi_rank * v_local if v_local != c.vocab_size else 0
        self.logits = new("argmax_in", v_local)
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
        if v_local != c.vocab_size:
            assert c.sampling_seed is None and v_local * mpk.world_size == c.vocab_size
            mpk.argmax_exchange_layer(input=(part_v, part_i), output=argmax_out, first_column=self.vocab_first)
        else:
            mpk.argmax_reduce_layer(input=(part_v, part_i), output=argmax_out, grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
