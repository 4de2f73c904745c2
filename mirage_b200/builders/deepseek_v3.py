"""Layer sequence of a DeepSeek-V3-architecture decoder slice on a `PersistentKernel`, with its host weight preparation.

Emits the graph of the reference's builder (python/mirage/mpk/models/deepseek_v3/builder.py:563-1154, 2040-2119):
embed, then per layer

    rmsnorm -> q_a (FP8) -> rmsnorm -> q_b with W_UK absorbed (bf16) ┐
            -> kv_a latent (FP8) -> rmsnorm ; kv_a rope (FP8)        ├-> mla_kv_gather -> mla_mtp_decode -> mla_mtp_reduce
                                                                     ┘   -> o_proj with W_UV folded in (bf16) + residual
    rmsnorm -> dense:  gate_up (FP8) -> silu_mul -> down (FP8) + residual
            -> MoE:    router linear -> sigmoid top-k routing -> quantize -> experts w13 (FP8) -> silu_mul -> quantize ->
                       experts w2 (FP8);  shared expert gate_up -> silu_mul -> down;  weighted sum + shared -> + residual

then final rmsnorm -> lm_head -> argmax.  FP8 projections are `quantize_fp8_layer` + `linear_fp8[_with_residual]_layer`
pairs on weights re-quantised to power-of-two scales (fp8_prep.requantize_for_ue8m0); the routed experts keep float32
scales expanded per row (builder.py:924-931).  As in the reference snapshot, no task applies RoPE to q_pe / k_pe.

Parallel form (world_size > 1), one process per GPU: attention heads, the dense MLP and the shared expert are tensor
parallel; the routed experts are EXPERT parallel -- rank r holds experts [E r / world, E (r + 1) / world) and every rank
computes the same routing (`local_experts` of the routing layer, `first_expert` of the expert projections).  Row-parallel
outputs are combined by `allreduce_layer`: after o_proj, after the dense MLP, and once per MoE block over (routed
partial + shared-expert partial).  The reference snapshot shards every expert's intermediate dimension instead and has an
allreduce only after the MoE block (demo/deepseek_v3/demo.py:741-748, builder.py:2083-2105).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Sequence

import torch

from ..persistent_kernel import PersistentKernel, bfloat16, float8_e4m3, float32, int32, int64, uint32
from . import fp8_prep
from .qwen3 import grid_for_rmsnorm_linear_layer

D_LATENT, D_ROPE = 512, 64
D_K = D_LATENT + D_ROPE


@dataclass
class DeepSeekV3Shape:
    num_layers: int = 4
    first_moe_layer: int = 1
    hidden_size: int = 7168
    q_lora_rank: int = 1536
    kv_lora_rank: int = 512
    num_heads: int = 128
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    num_experts: int = 256
    num_experts_per_tok: int = 8
    n_group: int = 8
    topk_group: int = 4
    routed_scaling_factor: float = 2.5
    moe_intermediate_size: int = 2048
    intermediate_size: int = 18432
    vocab_size: int = 129280


def _deq(wq: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    return fp8_prep.dequantize_block_scaled(wq, scale_inv)


def prepare_state(ckpt: Dict[str, torch.Tensor], s: DeepSeekV3Shape, world_size: int = 1, rank: int = 0) -> Dict[str, torch.Tensor]:
    """Checkpoint (HF names; FP8 tensors with `.weight_scale_inv` 128 x 128 block scales, the rest bf16) -> this rank's
    tensors in the forms the graph consumes.  Follows demo/deepseek_v3/demo.py:548-645 and models/convert.py:150-230:

      q_b_absorbed  [Hl * 576, q_lora] bf16   per head [k_nope^T q_nope (512 rows) | q_rope (64 rows)], fp32 then bf16
      o_fused       [hidden, Hl * 512] bf16   o_proj[:, head] @ W_UV[head], fp32 product of the bf16 factors
      kv_a latent / rope                      split, rope rows padded to 128, each re-quantised on its own
      dense / shared-expert MLP               gate and up rows, down columns split by rank
      experts w13 / w2                        this rank's experts, float32 scales expanded per row

    Tensors stay on the device of the checkpoint."""
    nh, dn, dr, dv, r = s.num_heads, s.qk_nope_head_dim, s.qk_rope_head_dim, s.v_head_dim, s.kv_lora_rank
    assert r == D_LATENT and dr == D_ROPE and nh % world_size == 0
    hl = nh // world_size
    out: Dict[str, torch.Tensor] = {}
    for k in ("model.embed_tokens.weight", "model.norm.weight", "lm_head.weight"):
        out[k] = ckpt[k]

    def fp8(dst, wq, sc):
        q, packed, _ = fp8_prep.requantize_for_ue8m0(wq.contiguous(), sc.contiguous())
        out[dst + ".weight"], out[dst + ".scale"] = q, fp8_prep.packed_rows_contiguous(packed)

    def rows(t, n_per):      # block-scale rows that go with weight rows [rank * n_per, (rank + 1) * n_per)
        assert n_per % 128 == 0
        return t[rank * n_per // 128:(rank + 1) * n_per // 128]

    for i in range(s.num_layers):
        p = f"model.layers.{i}."
        a = p + "self_attn."
        for k in ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_a_layernorm.weight",
                  "self_attn.kv_a_layernorm.weight"):
            out[p + k] = ckpt[p + k]
        fp8(a + "q_a_proj", ckpt[a + "q_a_proj.weight"], ckpt[a + "q_a_proj.weight_scale_inv"])
        qb = ckpt[a + "q_b_proj.weight"].float().reshape(nh, dn + dr, -1)[rank * hl:(rank + 1) * hl]
        kvb = ckpt[a + "kv_b_proj.weight"].float().reshape(nh, dn + dv, r)[rank * hl:(rank + 1) * hl]
        absorbed = torch.einsum("hdr,hdq->hrq", kvb[:, :dn], qb[:, :dn])
        out[a + "q_b_absorbed.weight"] = torch.cat((absorbed, qb[:, dn:]), dim=1).to(torch.bfloat16).reshape(hl * D_K, -1).contiguous()
        o = ckpt[a + "o_proj.weight"].reshape(s.hidden_size, nh, dv)[:, rank * hl:(rank + 1) * hl]
        w_uv = kvb.to(torch.bfloat16)[:, dn:]
        out[a + "o_fused.weight"] = torch.einsum("dhn,hnk->dhk", o.float(), w_uv.float()).to(torch.bfloat16) \
            .reshape(s.hidden_size, hl * D_LATENT).contiguous()
        full = _deq(ckpt[a + "kv_a_proj_with_mqa.weight"], ckpt[a + "kv_a_proj_with_mqa.weight_scale_inv"])
        for name, part in (("kv_a_latent", full[:r]), ("kv_a_rope", torch.cat((full[r:], torch.zeros(128 - dr, full.shape[1],
                                                                                        device=full.device))))):
            q, packed, _ = fp8_prep.quantize_ue8m0(part)
            out[a + name + ".weight"], out[a + name + ".scale"] = q, fp8_prep.packed_rows_contiguous(packed)
        m = p + "mlp."
        if i < s.first_moe_layer:
            blocks = [("", s.intermediate_size)]
        else:
            blocks = [("shared_experts.", s.moe_intermediate_size)]
            out[m + "gate.weight"] = ckpt[m + "gate.weight"]
            out[m + "gate.e_score_correction_bias"] = ckpt[m + "gate.e_score_correction_bias"]
            per = s.num_experts // world_size
            assert s.num_experts % world_size == 0
            for nm in ("w13", "w2"):
                w = ckpt[m + f"experts.{nm}.weight"][rank * per:(rank + 1) * per].contiguous()
                sc = ckpt[m + f"experts.{nm}.weight_scale_inv"][rank * per:(rank + 1) * per].float().clamp(min=1e-30)
                out[m + f"experts.{nm}.weight"] = w
                out[m + f"experts.{nm}.scale"] = sc.repeat_interleave(128, dim=1)[:, :w.shape[1]].contiguous()
        for sub, width in blocks:
            loc = width // world_size
            for nm in ("gate_proj", "up_proj"):
                key = m + sub + nm
                fp8(key, ckpt[key + ".weight"][rank * loc:(rank + 1) * loc], rows(ckpt[key + ".weight_scale_inv"], loc))
            key = m + sub + "down_proj"
            assert loc % 128 == 0
            fp8(key, ckpt[key + ".weight"][:, rank * loc:(rank + 1) * loc],
                ckpt[key + ".weight_scale_inv"][:, rank * loc // 128:(rank + 1) * loc // 128])
    return out


class DeepSeekV3Builder:
    """Builds the slice on `mpk` from a state prepared by `prepare_state` (this rank's shard)."""

    def __init__(self, mpk: PersistentKernel, shape: DeepSeekV3Shape):
        self.mpk, self.s = mpk, shape
        self.world_size, self.rank = mpk.world_size, mpk.mpi_rank
        self.input_tokens = mpk.meta_tensors.get("input_tokens")
        self.output_tokens = mpk.meta_tensors.get("output_tokens")
        self._keep = []
        self.moe_masks = []          # per MoE layer: the [E + 1] tensor whose last entry is the number of active local experts

    # ---- helpers --------------------------------------------------------------------------------------------------
    def _new(self, name, width, dtype=bfloat16):
        mbt = self.mpk.max_num_batched_tokens
        return self.mpk.new_tensor(dims=(mbt, width), dtype=dtype, name=name, io_category="cuda_tensor")

    def _act_fp8(self, width, tag):
        mbt = self.mpk.max_num_batched_tokens
        q = self.mpk.new_tensor(dims=(mbt, width), dtype=float8_e4m3, name=f"fp8_act_{tag}", io_category="cuda_tensor")
        sc = self.mpk.new_tensor(dims=((width // 128 + 3) // 4, (mbt + 3) // 4 * 4), dtype=uint32, name=f"fp8_act_scale_{tag}",
                                 io_category="cuda_tensor")
        return q, sc

    def _fp8_linear(self, src, key, out, name, *, residual=None, quantized=None):
        """quantize_fp8 (unless `quantized` = (q, scale) of the same input is handed in) + linear_fp8."""
        mpk, mbt = self.mpk, self.mpk.max_num_batched_tokens
        w = mpk.attach_input(self.sd[key + ".weight"], name=name)
        ws = mpk.attach_input(self.sd[key + ".scale"], name=name + "_scale")
        if quantized is None:
            quantized = self._act_fp8(w.dim(1), name)
            mpk.quantize_fp8_layer(input=src, output_fp8=quantized[0], output_scale=quantized[1], grid_dim=(mbt, 1, 1),
                                   block_dim=(128, 1, 1))
        kw = dict(input_fp8=quantized[0], input_scale=quantized[1], weight_fp8=w, weight_scale=ws, output=out,
                  grid_dim=(max(1, w.dim(0) // 128), 1, 1), block_dim=(128, 1, 1))
        if residual is None:
            mpk.linear_fp8_layer(**kw)
        else:
            mpk.linear_fp8_with_residual_layer(residual=residual, **kw)
        return quantized

    def _allreduce(self, x, name):
        """x (this rank's partial) -> the sum over the ranks; identity on one rank."""
        if self.world_size == 1:
            return x
        out = self.mpk.new_tensor(dims=(self.mpk.max_num_batched_tokens, self.s.hidden_size), dtype=bfloat16, name=name,
                                  io_category="nvshmem_tensor")
        self.mpk.allreduce_layer(input=x, buffer=self.allreduce_buf, output=out, grid_dim=(self.s.hidden_size // 128, 1, 1),
                                 block_dim=(128, 1, 1))
        return out

    def _swiglu(self, prefix, xn, width_local, out, name, *, residual=None, quantized=None):
        """gate / up interleaved in groups (as the reference fuses them, demo.py:611-640) -> silu_mul -> down."""
        mpk, sd, mbt = self.mpk, self.sd, self.mpk.max_num_batched_tokens
        groups = grid_for_rmsnorm_linear_layer(2 * width_local) // 2
        while width_local % groups != 0:
            groups -= 1
        parts = []
        for nm in ("gate_proj", "up_proj"):
            parts.append((mpk.attach_input(sd[prefix + nm + ".weight"], name=f"{name}_{nm}"),
                          mpk.attach_input(sd[prefix + nm + ".scale"], name=f"{name}_{nm}_scale")))
        w = mpk.shuffle_tensors(inputs=[q for q, _ in parts], shuffled_dim=0, num_groups=groups, name=f"{name}_gate_up")
        ws = mpk.shuffle_tensors(inputs=[r for _, r in parts], shuffled_dim=0, num_groups=groups, name=f"{name}_gate_up_scale")
        if quantized is None:
            quantized = self._act_fp8(self.s.hidden_size, name + "_in")
            mpk.quantize_fp8_layer(input=xn, output_fp8=quantized[0], output_scale=quantized[1], grid_dim=(mbt, 1, 1),
                                   block_dim=(128, 1, 1))
        mid = self._new(name + "_mid", 2 * width_local)
        mpk.linear_fp8_layer(input_fp8=quantized[0], input_scale=quantized[1], weight_fp8=w, weight_scale=ws, output=mid,
                             grid_dim=(2 * groups, 1, 1), block_dim=(128, 1, 1))
        act = self._new(name + "_act", width_local)
        mpk.silu_mul_layer(input=mid, output=act, grid_dim=(groups, 1, 1), block_dim=(128, 1, 1))
        self._fp8_linear(act, prefix + "down_proj", out, name + "_down", residual=residual)
        return quantized

    # ---- layers ---------------------------------------------------------------------------------------------------
    def _attention(self, i, x, xn, caches):
        mpk, s, sd, mbt = self.mpk, self.s, self.sd, self.mpk.max_num_batched_tokens
        a = f"model.layers.{i}.self_attn."
        hl = s.num_heads // self.world_size
        q_a = self._new(f"layer_{i}_q_a", s.q_lora_rank)
        hidden_q = self._fp8_linear(xn, a + "q_a_proj", q_a, f"layer_{i}_q_a_proj")
        q_a_n = self._new(f"layer_{i}_q_a_normed", s.q_lora_rank)
        mpk.rmsnorm_layer(input=q_a, weight=mpk.attach_input(sd[a + "q_a_layernorm.weight"], name=f"layer_{i}_q_a_layernorm"),
                          output=q_a_n, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
        q = self._new(f"layer_{i}_q_nope_pe", hl * D_K)
        w_qb = mpk.attach_input(sd[a + "q_b_absorbed.weight"], name=f"layer_{i}_q_b_absorbed")
        mpk.linear_layer(input=q_a_n, weight=w_qb, output=q, grid_dim=(grid_for_rmsnorm_linear_layer(hl * D_K), 1, 1),
                         block_dim=(128, 1, 1))
        lat = self._new(f"layer_{i}_c_latent", D_LATENT)
        self._fp8_linear(xn, a + "kv_a_latent", lat, f"layer_{i}_kv_a_latent", quantized=hidden_q)
        k_pe = self._new(f"layer_{i}_k_pe", 128)
        self._fp8_linear(xn, a + "kv_a_rope", k_pe, f"layer_{i}_kv_a_rope", quantized=hidden_q)
        lat_n = self._new(f"layer_{i}_c_latent_normed", D_LATENT)
        mpk.rmsnorm_layer(input=lat, weight=mpk.attach_input(sd[a + "kv_a_layernorm.weight"], name=f"layer_{i}_kv_a_layernorm"),
                          output=lat_n, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
        cache = mpk.attach_input(caches[i], name=f"layer_{i}_kv_cache")
        mpk.mla_kv_gather_layer(c_latent_new=lat_n, k_pe_new=k_pe, paged_cache=cache, contiguous_kv=self.contiguous_kv,
                                mla_params=(D_K, D_LATENT, mpk.page_size), grid_dim=(mpk.max_num_batched_requests, 1, 1),
                                block_dim=(128, 1, 1))
        splits = (mpk.max_seq_length + 127) // 128
        po = mpk.new_tensor(dims=(mbt * hl * splits, D_LATENT), dtype=bfloat16, name=f"layer_{i}_mla_partial_o")
        lse = mpk.new_tensor(dims=(mbt * hl * splits,), dtype=float32, name=f"layer_{i}_mla_partial_lse")
        attn = self._new(f"layer_{i}_attn_out", hl * D_LATENT)
        mpk.mla_mtp_decode_layer(q, self.contiguous_kv, po, lse, mbt, mpk.max_seq_length)
        mpk.mla_mtp_reduce_layer(po, lse, attn, mbt, mpk.max_seq_length)
        out = mpk.new_tensor(dims=(mbt, s.hidden_size), dtype=bfloat16, name=f"layer_{i}_attn_proj",
                             io_category="nvshmem_tensor" if self.world_size > 1 else "cuda_tensor")
        mpk.linear_with_residual_layer(input=attn, weight=mpk.attach_input(sd[a + "o_fused.weight"], name=f"layer_{i}_o_fused"),
                                       residual=x, output=out, grid_dim=(s.hidden_size // 64, 1, 1), block_dim=(128, 1, 1))
        return self._allreduce(out, f"layer_{i}_attn_allreduce")

    def _moe(self, i, x, xn):
        mpk, s, sd, mbt = self.mpk, self.s, self.sd, self.mpk.max_num_batched_tokens
        m = f"model.layers.{i}.mlp."
        E, topk, I, H = s.num_experts, s.num_experts_per_tok, s.moe_intermediate_size, s.hidden_size
        per = E // self.world_size
        first = self.rank * per
        logits = self._new(f"layer_{i}_router_logits", E)
        mpk.linear_layer(input=xn, weight=mpk.attach_input(sd[m + "gate.weight"], name=f"layer_{i}_moe_gate"), output=logits,
                         grid_dim=(max(1, E // 8), 1, 1), block_dim=(128, 1, 1))
        t_w = mpk.new_tensor(dims=(mbt, topk), dtype=float32, name=f"layer_{i}_moe_topk_weights")
        t_idx = mpk.new_tensor(dims=(E, mbt), dtype=int32, name=f"layer_{i}_moe_routing_indices")
        t_mask = mpk.new_tensor(dims=(E + 1,), dtype=int32, name=f"layer_{i}_moe_mask")
        self.moe_masks.append(t_mask)
        mpk.moe_topk_sigmoid_routing_layer(
            input=logits, bias=mpk.attach_input(sd[m + "gate.e_score_correction_bias"], name=f"layer_{i}_moe_gate_bias"),
            output=(t_w, t_idx, t_mask), grid_dim=(1, 1, 1), block_dim=(256, 1, 1), num_groups=s.n_group,
            topk_group=s.topk_group, routed_scaling_factor=s.routed_scaling_factor,
            local_experts=(first, first + per) if self.world_size > 1 else None)
        xq = mpk.new_tensor(dims=(mbt, H), dtype=float8_e4m3, name=f"layer_{i}_moe_input_fp8")
        xs = mpk.new_tensor(dims=(mbt, H // 128), dtype=float32, name=f"layer_{i}_moe_input_scale")
        mpk.quantize_fp8_layer(input=xn, output_fp8=xq, output_scale=xs, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1),
                               scale_ue8m0=False)
        mid = mpk.new_tensor(dims=(mbt, topk, 2 * I), dtype=bfloat16, name=f"layer_{i}_moe_mid")
        att = lambda k, nm: mpk.attach_input(sd[m + k], name=f"layer_{i}_{nm}")
        mpk.moe_w13_fp8_layer(input_fp8=xq, input_scale=xs, weight_fp8=att("experts.w13.weight", "experts_w13"),
                              weight_scale=att("experts.w13.scale", "experts_w13_scale"), moe_routing_indices=t_idx,
                              moe_mask=t_mask, output=mid, grid_dim=(E, 2, 1), block_dim=(128, 1, 1), first_expert=first)
        act = mpk.new_tensor(dims=(mbt, topk, I), dtype=bfloat16, name=f"layer_{i}_moe_silu")
        mpk.moe_silu_mul_layer(input=mid, output=act, grid_dim=(mbt, topk, 1), block_dim=(128, 1, 1))
        aq = mpk.new_tensor(dims=(mbt, topk, I), dtype=float8_e4m3, name=f"layer_{i}_moe_silu_fp8")
        asc = mpk.new_tensor(dims=(mbt, topk, I // 128), dtype=float32, name=f"layer_{i}_moe_silu_scale")
        mpk.quantize_fp8_layer(input=act, output_fp8=aq, output_scale=asc, grid_dim=(mbt * topk, 1, 1), block_dim=(128, 1, 1),
                               scale_ue8m0=False)
        down = mpk.new_tensor(dims=(mbt, topk, H), dtype=bfloat16, name=f"layer_{i}_moe_down")
        mpk.moe_w2_fp8_layer(input_fp8=aq, input_scale=asc, weight_fp8=att("experts.w2.weight", "experts_w2"),
                             weight_scale=att("experts.w2.scale", "experts_w2_scale"), moe_routing_indices=t_idx,
                             moe_mask=t_mask, output=down, grid_dim=(E, 2, 1), block_dim=(128, 1, 1), first_expert=first)
        shared = self._new(f"layer_{i}_shared_residual", H)
        self._swiglu(m + "shared_experts.", xn, I // self.world_size, shared, f"layer_{i}_shared")
        moe_out = mpk.new_tensor(dims=(mbt, H), dtype=bfloat16, name=f"layer_{i}_moe_output",
                                 io_category="nvshmem_tensor" if self.world_size > 1 else "cuda_tensor")
        mpk.moe_mul_sum_add_layer(input=down, weight=t_w, residual=shared, output=moe_out, grid_dim=(mbt, 1, 1),
                                  block_dim=(128, 1, 1))
        summed = self._allreduce(moe_out, f"layer_{i}_moe_allreduce")
        out = self._new(f"layer_{i}_moe_residual", H)
        mpk.elementwise_add_layer(input_a=x, input_b=summed, output=out, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
        return out

    def build(self, state: Dict[str, torch.Tensor], caches: Sequence[torch.Tensor]):
        """`state`: prepare_state(...) of this rank; `caches[i]`: [max_num_pages, page_size, 576] bf16 per layer."""
        mpk, s = self.mpk, self.s
        self.sd = sd = state
        mbt = mpk.max_num_batched_tokens
        H = s.hidden_size
        if self.world_size > 1:
            self.allreduce_buf = mpk.new_tensor(dims=(self.world_size, mbt, H), dtype=bfloat16, name="all_reduce_buf",
                                                io_category="nvshmem_tensor")
        self.contiguous_kv = mpk.new_tensor(dims=(8, D_K), dtype=bfloat16, name="contiguous_kv")   # (never filled: see mla_kv_gather_layer)
        x = self._new("embed_out", H)
        mpk.embed_layer(input=mpk.attach_input(self.input_tokens, name="input_token"),
                        weight=mpk.attach_input(sd["model.embed_tokens.weight"], name="embed_tokens"), output=x,
                        grid_dim=(1, 1, 1), block_dim=(128, 1, 1), input_source=1)
        for i in range(s.num_layers):
            p = f"model.layers.{i}."
            xn = self._new(f"layer_{i}_input_normed", H)
            mpk.rmsnorm_layer(input=x, weight=mpk.attach_input(sd[p + "input_layernorm.weight"], name=f"layer_{i}_input_layernorm"),
                              output=xn, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
            x = self._attention(i, x, xn, caches)
            xn = self._new(f"layer_{i}_post_normed", H)
            mpk.rmsnorm_layer(input=x, weight=mpk.attach_input(sd[p + "post_attention_layernorm.weight"],
                                                               name=f"layer_{i}_post_attn_layernorm"),
                              output=xn, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
            if i < s.first_moe_layer:
                out = mpk.new_tensor(dims=(mbt, H), dtype=bfloat16, name=f"layer_{i}_mlp_out",
                                     io_category="nvshmem_tensor" if self.world_size > 1 else "cuda_tensor")
                if self.world_size == 1:
                    self._swiglu(p + "mlp.", xn, s.intermediate_size, out, f"layer_{i}_mlp", residual=x)
                    x = out
                else:   # partial sums first, the residual once on the reduced sum
                    self._swiglu(p + "mlp.", xn, s.intermediate_size // self.world_size, out, f"layer_{i}_mlp")
                    summed = self._allreduce(out, f"layer_{i}_mlp_allreduce")
                    nxt = self._new(f"layer_{i}_mlp_residual", H)
                    mpk.elementwise_add_layer(input_a=x, input_b=summed, output=nxt, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
                    x = nxt
            else:
                x = self._moe(i, x, xn)
        self.hidden = x
        xn = self._new("final_normed", H)
        mpk.rmsnorm_layer(input=x, weight=mpk.attach_input(sd["model.norm.weight"], name="model_norm_weight"), output=xn,
                          grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
        self.logits = self._new("argmax_in", s.vocab_size)
        mpk.linear_layer(input=xn, weight=mpk.attach_input(sd["lm_head.weight"], name="lm_head"), output=self.logits,
                         grid_dim=(96, 1, 1), block_dim=(128, 1, 1))
        n_part = mpk.num_workers
        part_v = mpk.new_tensor(dims=(mbt, n_part), dtype=bfloat16, name="argmax_part_value")
        part_i = mpk.new_tensor(dims=(mbt, n_part), dtype=int64, name="argmax_part_index")
        mpk.argmax_partial_layer(input=self.logits, output=(part_v, part_i), grid_dim=(n_part, 1, 1), block_dim=(128, 1, 1))
        mpk.argmax_reduce_layer(input=(part_v, part_i), output=mpk.attach_input(self.output_tokens, name="output_token"),
                                grid_dim=(1, 1, 1), block_dim=(128, 1, 1))


class DeepSeekV3Runner:
    """Owns the device state of one rank (meta tensors, latent caches, prepared weights) and the compiled megakernel."""

    def __init__(self, shape: DeepSeekV3Shape, ckpt: Optional[Dict[str, torch.Tensor]] = None, *, total_num_requests: int,
                 max_seq_length: int, max_num_batched_requests: int, max_num_batched_tokens: int, max_num_pages: int,
                 page_size: int, eos_token_id: int = -1, world_size: int = 1, rank: int = 0, device: Optional[int] = None,
                 num_workers: int = 0, link_peers: bool = True, prepared: Optional[Dict[str, torch.Tensor]] = None):
        dev = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.device, self.shape = dev, shape
        mbr, mbt = max_num_batched_requests, max_num_batched_tokens
        i32, i64 = dict(dtype=torch.int32, device=dev), dict(dtype=torch.int64, device=dev)
        self.meta = {
            "step": torch.zeros(total_num_requests, **i32), "tokens": torch.zeros(total_num_requests, max_seq_length, **i64),
            "input_tokens": torch.zeros(mbt, 1, **i64), "output_tokens": torch.zeros(mbt, 1, **i64),
            "num_new_tokens": torch.ones(total_num_requests, **i32), "prompt_lengths": torch.zeros(total_num_requests, **i32),
            "qo_indptr_buffer": torch.zeros(mbr + 1, **i32), "paged_kv_indptr_buffer": torch.zeros(mbr + 1, **i32),
            "paged_kv_indices_buffer": torch.zeros(max_num_pages, **i32), "paged_kv_last_page_len_buffer": torch.zeros(mbr, **i32),
        }
        self.caches = [torch.zeros(max_num_pages, page_size, D_K, dtype=torch.bfloat16, device=dev) for _ in range(shape.num_layers)]
        if prepared is None:
            prepared = prepare_state({k: v.to(dev) for k, v in ckpt.items()}, shape, world_size, rank)
        self.state = prepared
        self.mpk = PersistentKernel(
            mode="offline", world_size=world_size, mpi_rank=rank, num_workers=num_workers, max_seq_length=max_seq_length,
            max_num_batched_requests=mbr, max_num_batched_tokens=mbt, max_num_pages=max_num_pages, page_size=page_size,
            meta_tensors=self.meta, eos_token_id=eos_token_id, device=dev.index)
        self.builder = DeepSeekV3Builder(self.mpk, shape)
        self.builder.build(self.state, self.caches)
        self.mpk.compile(link_peers=link_peers)
        self.logits = self.mpk.tensor_as_torch(self.builder.logits)
        self.vocab_first = 0

    def load_prompts(self, prompts):
        tok = torch.zeros_like(self.meta["tokens"], device="cpu")
        plen = torch.zeros_like(self.meta["prompt_lengths"], device="cpu")
        for i, p in enumerate(prompts):
            tok[i, :len(p)] = torch.tensor(list(p), dtype=torch.int64)
            plen[i] = len(p)
        self.meta["tokens"].copy_(tok)
        self.meta["prompt_lengths"].copy_(plen)
        self.mpk.reset()

    def step(self, n: int = 1):
        self.mpk.step(n)
