"""CPU oracle for a DeepSeek-V3-architecture decoder slice as the MPK builder lays it out.

TEST INFRASTRUCTURE ONLY (see oracle/mpk_ops.py for the rules).

Composition of the pinned op oracles (oracle/mpk_ops.py, fp8_ops.py, moe_ops.py, mla_ops.py) in the order of the
reference's graph builder, python/mirage/mpk/models/deepseek_v3/builder.py:
  * decoder layer, :2040-2119: input norm -> MLA attention (:563-792) -> post-attention norm -> dense MLP (:794-830)
    or mixture-of-experts MLP with a shared expert (:832-1154) -> residual;
  * MLA attention: q_a (FP8) -> q_a norm -> q_b with W_UK absorbed (bf16, [heads * 576, q_lora], per head
    [latent 512 | rope 64] rows) -> kv_a split into latent (FP8, 512 rows) and rope (FP8, 64 rows padded to 128)
    -> kv_a norm on the latent -> append [latent | rope] to the paged cache -> absorbed decode over the cache ->
    o_proj with W_UV folded in (bf16, [hidden, heads * 512]) + residual;
  * host weight preparation, demo/deepseek_v3/demo.py:548-645 and models/convert.py:150-230: absorption and the
    o_proj fusion are computed in fp32 and rounded to bf16 once; dense FP8 weights are re-quantised to power-of-two
    scales per row and 128 columns (builder.py:475-542); expert scales are expanded per row and FLOORED to powers of
    two inside the grouped GEMM (fp8_group_gemm_sm100.cuh:1378).

Positions taken where the reference snapshot is incomplete (each switchable):
  * `rope=False` (default) reproduces the snapshot: its builder precomputes RoPE tables (:208-225) but no task applies
    them to q_pe / k_pe.  `rope=True` applies the builder's own table convention (theta 10000) and is the
    mathematically complete graph; the megakernel implements the snapshot's graph.
  * `w_uv_from_k_rows=False` (default) folds the V rows of kv_b_proj into o_proj, which is what the absorption means;
    the snapshot slices the FIRST v_head_dim rows of each head's kv_b block (demo.py:584, the k_nope rows).  Both give a
    random matrix for random-init weights; the switch reproduces the snapshot's slice.
  * tensor / expert parallelism (`world_size` > 1): heads, dense-MLP and shared-expert columns split by rank, routed
    experts [E r / world, E (r + 1) / world) on rank r; partial outputs are rounded to bf16 per rank and summed in
    fp32 in rank order -- after o_proj (residual added once to the sum), after the dense MLP (the same), and once per
    MoE block over (routed partial + shared-expert partial).  The snapshot has an allreduce only after the MoE block.

Parity status: composition of pinned ops; the composition itself is cross-checked in tests/test_deepseek_oracle.py
(absorbed attention against plain multi-head attention with materialised K / V in fp32; the parallel emulation
against world_size = 1).  The reference has no end-to-end test of this graph.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List

import numpy as np
import torch

from . import fp8_ops as F
from . import mla_ops as A
from . import moe_ops as M
from . import mpk_ops as ops
from .batching import BatchState

BF16 = torch.bfloat16


@dataclass
class DeepSeekConfig:
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
    rms_eps: float = 1e-6

    @staticmethod
    def tiny(**kw):
        base = dict(num_layers=2, first_moe_layer=1, hidden_size=1024, q_lora_rank=512, num_heads=32, num_experts=16,
                    num_experts_per_tok=4, n_group=4, topk_group=2, moe_intermediate_size=512, intermediate_size=1024,
                    vocab_size=1024)
        base.update(kw)
        return DeepSeekConfig(**base)


FP8_LINEARS = ("self_attn.q_a_proj", "self_attn.kv_a_proj_with_mqa", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj",
               "mlp.shared_experts.gate_proj", "mlp.shared_experts.up_proj", "mlp.shared_experts.down_proj")


def _block_quantize(w: torch.Tensor, g: torch.Generator):
    """bf16 weight -> (e4m3 values, float32 128 x 128 block scales drawn log-uniformly from [1e-3, 1e-1]); value x scale
    reproduces the weight to e4m3 precision (the form BASELINE's FP8 configurations describe)."""
    lead, (n, k) = w.shape[:-2], w.shape[-2:]
    lo, hi = math.log(1e-3), math.log(1e-1)
    scale = torch.exp(lo + torch.rand(*lead, (n + 127) // 128, (k + 127) // 128, generator=g) * (hi - lo)).float()
    per = scale.repeat_interleave(128, -2)[..., :n, :].repeat_interleave(128, -1)[..., :k]
    return (w.float() / per).clamp(-448, 448).to(torch.float8_e4m3fn), scale


def make_checkpoint(cfg: DeepSeekConfig, seed: int) -> Dict[str, torch.Tensor]:
    """Random-init checkpoint in the form the reference's demo reads: N(0, 0.02) linears, 1 + N(0, 0.02) norms, router
    bias N(0, 0.1) fp32; the linears listed in FP8_LINEARS and the routed experts as e4m3 + `_scale_inv` block scales,
    q_b / kv_b / o_proj / router / embedding / lm_head in bf16."""
    g = torch.Generator().manual_seed(seed)
    lin = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(BF16)
    norm = lambda n: (1 + torch.randn(n, generator=g) * 0.02).to(BF16)
    h, nh = cfg.hidden_size, cfg.num_heads
    sd = {"model.embed_tokens.weight": lin(cfg.vocab_size, h), "model.norm.weight": norm(h), "lm_head.weight": lin(cfg.vocab_size, h)}
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = norm(h)
        sd[p + "post_attention_layernorm.weight"] = norm(h)
        a = p + "self_attn."
        sd[a + "q_a_proj.weight"] = lin(cfg.q_lora_rank, h)
        sd[a + "q_a_layernorm.weight"] = norm(cfg.q_lora_rank)
        sd[a + "q_b_proj.weight"] = lin(nh * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim), cfg.q_lora_rank)
        sd[a + "kv_a_proj_with_mqa.weight"] = lin(cfg.kv_lora_rank + cfg.qk_rope_head_dim, h)
        sd[a + "kv_a_layernorm.weight"] = norm(cfg.kv_lora_rank)
        sd[a + "kv_b_proj.weight"] = lin(nh * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank)
        sd[a + "o_proj.weight"] = lin(h, nh * cfg.v_head_dim)
        m = p + "mlp."
        if i < cfg.first_moe_layer:
            sd[m + "gate_proj.weight"] = lin(cfg.intermediate_size, h)
            sd[m + "up_proj.weight"] = lin(cfg.intermediate_size, h)
            sd[m + "down_proj.weight"] = lin(h, cfg.intermediate_size)
        else:
            e, im = cfg.num_experts, cfg.moe_intermediate_size
            sd[m + "gate.weight"] = lin(e, h)
            sd[m + "gate.e_score_correction_bias"] = (torch.randn(e, generator=g) * 0.1).float()
            sd[m + "experts.w13.weight"] = lin(e, 2 * im, h)          # per expert [gate rows | up rows]
            sd[m + "experts.w2.weight"] = lin(e, h, im)
            for nme, shape in (("gate_proj", (im, h)), ("up_proj", (im, h)), ("down_proj", (h, im))):
                sd[m + f"shared_experts.{nme}.weight"] = lin(*shape)
    for k in list(sd):
        stem = k[:-len(".weight")] if k.endswith(".weight") else None
        if stem and (any(stem.endswith(n) for n in FP8_LINEARS) or stem.endswith(("experts.w13", "experts.w2"))):
            sd[k], sd[k + "_scale_inv"] = _block_quantize(sd[k], g)
    return sd


def _deq_block(wq: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    n, k = wq.shape[-2:]
    return wq.float() * scale_inv.float().repeat_interleave(128, -2)[..., :n, :].repeat_interleave(128, -1)[..., :k]


class _Fp8Weight:
    """A dense FP8 weight after the reference's host re-quantisation: e4m3 values + UE8M0 exponents per (row, 128 columns)."""

    def __init__(self, wq, scale_inv):
        self.q, self.exps, _ = F.quantize_fp8_ue8m0(_deq_block(wq, scale_inv))

    def __call__(self, x, residual=None):
        xq, xe, _ = F.quantize_fp8_ue8m0(x)
        return F.linear_fp8(xq, xe, self.q, self.exps, residual)


class _PlainWeight:
    """The same weight without any FP8 step: the checkpoint's block-dequantised values, fp32 (composition checks)."""

    def __init__(self, wq, scale_inv):
        self.w = _deq_block(wq, scale_inv)

    def __call__(self, x, residual=None):
        return ops.linear(x, self.w, residual)


class DeepSeekOracle:
    def __init__(self, cfg: DeepSeekConfig, ckpt: Dict[str, torch.Tensor], *, max_num_pages: int, page_size: int,
                 world_size: int = 1, rope: bool = False, w_uv_from_k_rows: bool = False, quantize: bool = True,
                 softmax_scale: float = None):
        """`quantize=False` replaces every FP8 step (activation quantisation, re-quantised weights, expert GEMM scales)
        by the block-dequantised checkpoint weights in fp32 and leaves the graph otherwise unchanged: the form that an
        independent bf16 / fp32 implementation of the model can be compared with.  `softmax_scale` overrides the
        constant the reference's call sites hard-code (mla_ops.DEEPSEEK_SCALE)."""
        self.cfg, self.ws, self.rope = cfg, world_size, rope
        self.quant = quantize
        self.weight_cls = _Fp8Weight if quantize else _PlainWeight
        self.sm_scale = A.DEEPSEEK_SCALE if softmax_scale is None else float(softmax_scale)
        self.sd = ckpt
        self.cache = [torch.zeros(max_num_pages, page_size, A.D_K, dtype=BF16) for _ in range(cfg.num_layers)]
        assert cfg.kv_lora_rank == A.D_V and cfg.kv_lora_rank + cfg.qk_rope_head_dim == A.D_K
        nh, dn, dr, dv, r = cfg.num_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        self.L = []
        for i in range(cfg.num_layers):
            p = f"model.layers.{i}."
            a = p + "self_attn."
            w = {}
            # absorption (convert.py:150-230): per head [k_nope^T q_nope (512 rows) | q_rope (64 rows)], fp32 then bf16
            qb = ckpt[a + "q_b_proj.weight"].float().reshape(nh, dn + dr, -1)
            kvb = ckpt[a + "kv_b_proj.weight"].float().reshape(nh, dn + dv, r)
            absorbed = torch.einsum("hdr,hdq->hrq", kvb[:, :dn], qb[:, :dn])
            w["q_b"] = torch.cat((absorbed, qb[:, dn:]), dim=1).to(BF16)                   # [heads, 576, q_lora]
            # o_proj with W_UV folded in (demo.py:575-603): fp32 product of the bf16 factors, rounded once
            w_uv = kvb.to(BF16)[:, :dv] if w_uv_from_k_rows else kvb.to(BF16)[:, dn:]
            o = ckpt[a + "o_proj.weight"].reshape(cfg.hidden_size, nh, dv)
            w["o"] = torch.einsum("dhn,hnk->dhk", o.float(), w_uv.float()).to(BF16)        # [hidden, heads, 512]
            w["q_a"] = self.weight_cls(ckpt[a + "q_a_proj.weight"], ckpt[a + "q_a_proj.weight_scale_inv"])
            kva, kvs = ckpt[a + "kv_a_proj_with_mqa.weight"], ckpt[a + "kv_a_proj_with_mqa.weight_scale_inv"]
            full = _deq_block(kva, kvs)
            # (builder.py:621-659: the latent rows and the rope rows are re-quantised separately; the rope rows are
            # padded to 128 with zeros first, which does not change their per-row scales)
            lat_q, lat_e, _ = F.quantize_fp8_ue8m0(full[:r])
            rope_q, rope_e, _ = F.quantize_fp8_ue8m0(full[r:])
            w["kv_lat"], w["kv_rope"] = (lat_q, lat_e), (rope_q, rope_e)
            w["kv_plain"] = full
            self.L.append(w)
        if rope:
            inv = 1.0 / (10000.0 ** (torch.arange(0, dr, 2, dtype=torch.float32) / dr))
            fr = torch.outer(torch.arange(8192, dtype=torch.float32), inv)
            self.cos, self.sin = torch.cat((fr.cos(), fr.cos()), -1).to(BF16), torch.cat((-fr.sin(), fr.sin()), -1).to(BF16)

    # ---- pieces ---------------------------------------------------------------------------------------------------
    @staticmethod
    def _rope(x, cos, sin):
        """x cos + swap_halves(x) sin with the builder's tables cos = [c, c], sin = [-s, s] (builder.py:208-225)."""
        half = x.shape[-1] // 2
        swapped = torch.cat((x[..., half:], x[..., :half]), dim=-1)
        return (x.float() * cos.float() + swapped.float() * sin.float()).to(BF16)

    def _fp8(self, key: str):
        return self.weight_cls(self.sd[key + ".weight"], self.sd[key + ".weight_scale_inv"])

    @staticmethod
    def _rank_sum(parts: List[torch.Tensor], residual=None) -> torch.Tensor:
        """bf16 partial outputs of the ranks summed in fp32 in rank order (+ residual once), one bf16 rounding."""
        acc = torch.zeros_like(parts[0], dtype=torch.float32)
        for prt in parts:
            acc = acc + prt.float()
        if residual is not None:
            acc = acc + residual.float()
        return acc.to(BF16)

    def _fp8_row_parallel(self, key: str, x_in: torch.Tensor, residual) -> torch.Tensor:
        """y = x W^T (+ residual) with W's columns split over the ranks (down projections)."""
        wq, sc = self.sd[key + ".weight"], self.sd[key + ".weight_scale_inv"]
        if self.ws == 1:
            return self.weight_cls(wq, sc)(x_in, residual)
        kk = wq.shape[1] // self.ws
        assert kk % 128 == 0
        parts = [self.weight_cls(wq[:, r * kk:(r + 1) * kk], sc[:, r * kk // 128:(r + 1) * kk // 128])(x_in[:, r * kk:(r + 1) * kk])
                 for r in range(self.ws)]
        return self._rank_sum(parts, residual)

    def _attention(self, li: int, xn: torch.Tensor, x: torch.Tensor, reqs) -> torch.Tensor:
        cfg, w = self.cfg, self.L[li]
        a = f"model.layers.{li}.self_attn."
        nh = cfg.num_heads
        q_a = ops.rmsnorm(w["q_a"](xn), self.sd[a + "q_a_layernorm.weight"], cfg.rms_eps)
        q = ops.linear(q_a, w["q_b"].reshape(nh * A.D_K, -1)).reshape(-1, nh, A.D_K)
        if self.quant:
            xq, xe, _ = F.quantize_fp8_ue8m0(xn)
            lat = ops.rmsnorm(F.linear_fp8(xq, xe, *w["kv_lat"]), self.sd[a + "kv_a_layernorm.weight"], cfg.rms_eps)
            k_pe = F.linear_fp8(xq, xe, *w["kv_rope"])
        else:
            r = cfg.kv_lora_rank
            lat = ops.rmsnorm(ops.linear(xn, w["kv_plain"][:r]), self.sd[a + "kv_a_layernorm.weight"], cfg.rms_eps)
            k_pe = ops.linear(xn, w["kv_plain"][r:])
        out = torch.zeros(xn.shape[0], nh, A.D_V, dtype=BF16)
        for (q0, q1), pages, seq_len in reqs:
            qr, kp = q[q0:q1].clone(), k_pe[q0:q1].clone()
            if self.rope:
                pos = torch.arange(seq_len - (q1 - q0), seq_len)
                cos, sin = self.cos[pos], self.sin[pos]
                kp = self._rope(kp, cos, sin)
                qr[..., A.D_V:] = self._rope(qr[..., A.D_V:], cos[:, None], sin[:, None])
            A.mla_append(self.cache[li], lat[q0:q1], kp, pages, seq_len)
            out[q0:q1] = A.mla_decode_request(qr, self.cache[li], pages, seq_len, self.sm_scale)
        o = w["o"]
        if self.ws == 1:
            return ops.linear(out.reshape(-1, nh * A.D_V), o.reshape(cfg.hidden_size, nh * A.D_V), x)
        hl = nh // self.ws
        parts = [ops.linear(out[:, r * hl:(r + 1) * hl].reshape(-1, hl * A.D_V),
                            o[:, r * hl:(r + 1) * hl].reshape(cfg.hidden_size, hl * A.D_V)) for r in range(self.ws)]
        return self._rank_sum(parts, x)

    def _swiglu(self, prefix: str, xn: torch.Tensor, residual) -> torch.Tensor:
        """gate / up (FP8, column parallel) -> silu(gate) * up -> down (FP8, row parallel)."""
        gate, up = self._fp8(prefix + "gate_proj")(xn), self._fp8(prefix + "up_proj")(xn)
        act = ops.silu_mul(torch.cat((gate, up), dim=1), 1)
        return self._fp8_row_parallel(prefix + "down_proj", act, residual)

    def _swiglu_partials(self, prefix: str, xn: torch.Tensor) -> List[torch.Tensor]:
        gate, up = self._fp8(prefix + "gate_proj")(xn), self._fp8(prefix + "up_proj")(xn)
        act = ops.silu_mul(torch.cat((gate, up), dim=1), 1)
        wq, sc = self.sd[prefix + "down_proj.weight"], self.sd[prefix + "down_proj.weight_scale_inv"]
        kk = wq.shape[1] // self.ws
        return [self.weight_cls(wq[:, r * kk:(r + 1) * kk], sc[:, r * kk // 128:(r + 1) * kk // 128])(act[:, r * kk:(r + 1) * kk])
                for r in range(self.ws)]

    def _moe(self, li: int, xn: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        m = f"model.layers.{li}.mlp."
        logits = ops.linear(xn, self.sd[m + "gate.weight"])
        weights, routing, _, chosen = M.topk_sigmoid_routing(
            logits, self.sd[m + "gate.e_score_correction_bias"], topk=cfg.num_experts_per_tok, num_groups=cfg.n_group,
            topk_group=cfg.topk_group, scaling=cfg.routed_scaling_factor)
        self.last_routing = chosen
        topk = cfg.num_experts_per_tok
        # expert scales: block scales expanded per row (builder.py:924-931); the grouped GEMM floors them
        w13, s13 = self.sd[m + "experts.w13.weight"], self.sd[m + "experts.w13.weight_scale_inv"].repeat_interleave(128, 1)
        w2, s2 = self.sd[m + "experts.w2.weight"], self.sd[m + "experts.w2.weight_scale_inv"].repeat_interleave(128, 1)
        if self.quant:
            xq, xs = F.quantize_fp8_f32scale(xn)
            mid = M.moe_gemm_fp8(xq, xs, w13, s13[:, :w13.shape[1]], routing, topk=topk, per_slot_input=False)
            act = M.moe_silu_mul(mid)
            aq, asc = F.quantize_fp8_f32scale(act.reshape(-1, act.shape[-1]))
            down = M.moe_gemm_fp8(aq.reshape(act.shape), asc.reshape(act.shape[0], topk, -1), w2, s2[:, :w2.shape[1]], routing,
                                  topk=topk, per_slot_input=True)
        else:
            mid = M.moe_gemm_bf16(xn, _deq_block(w13, self.sd[m + "experts.w13.weight_scale_inv"]), routing, topk=topk,
                                  per_slot_input=False)
            act = M.moe_silu_mul(mid)
            down = M.moe_gemm_bf16(act, _deq_block(w2, self.sd[m + "experts.w2.weight_scale_inv"]), routing, topk=topk,
                                   per_slot_input=True)
        shared_parts = self._swiglu_partials(m + "shared_experts.", xn)
        if self.ws == 1:
            moe_out = M.moe_mul_sum_add(down, weights, shared_parts[0])
        else:
            per = cfg.num_experts // self.ws
            parts = []
            for r in range(self.ws):
                local = (chosen >= r * per) & (chosen < (r + 1) * per)
                parts.append(M.moe_mul_sum_add(down, torch.where(local, weights, torch.zeros_like(weights)), shared_parts[r]))
            moe_out = self._rank_sum(parts)
        return (x.float() + moe_out.float()).to(BF16)          # elementwise_add_layer (builder.py:2099-2117)

    def forward_tokens(self, token_ids: torch.Tensor, reqs) -> torch.Tensor:
        cfg = self.cfg
        x = ops.embedding(token_ids, self.sd["model.embed_tokens.weight"])
        for li in range(cfg.num_layers):
            p = f"model.layers.{li}."
            xn = ops.rmsnorm(x, self.sd[p + "input_layernorm.weight"], cfg.rms_eps)
            x = self._attention(li, xn, x, reqs)
            xn = ops.rmsnorm(x, self.sd[p + "post_attention_layernorm.weight"], cfg.rms_eps)
            if li < cfg.first_moe_layer:
                x = self._swiglu(p + "mlp.", xn, x)
            else:
                x = self._moe(li, xn, x)
        self.last_hidden = x
        xn = ops.rmsnorm(x, self.sd["model.norm.weight"], cfg.rms_eps)
        self.last_logits = ops.linear(xn, self.sd["lm_head.weight"])
        return self.last_logits

    def run_iteration(self, st: BatchState) -> bool:
        """prepare_next_batch + one forward; writes st.output_tokens.  False when done."""
        if not st.prepare_next_batch():
            return False
        n = st.num_active_tokens
        reqs = []
        for slot in range(st.mbr):
            if st.request_ids[slot] == -1:
                continue
            _, qr, pages, seq_len = st.request_view(slot)
            reqs.append((qr, pages, seq_len))
        logits = self.forward_tokens(torch.from_numpy(st.input_tokens[:n].copy()), reqs)
        st.output_tokens[:n] = ops.argmax(logits).cpu().numpy()
        return True


def plain_attention_reference(cfg: DeepSeekConfig, ckpt, li: int, q_a_normed: torch.Tensor, kv_latent_normed: torch.Tensor,
                              k_pe: torch.Tensor) -> torch.Tensor:
    """Multi-head attention with K and V materialised from the latent (the un-absorbed form, fp32 throughout) for ONE
    sequence whose tokens are all given: row i attends to rows <= i.  -> what o_proj receives, [n, heads * v_head_dim].
    Used to check that the absorbed weights + latent-space decode compute the same function."""
    a = f"model.layers.{li}.self_attn."
    nh, dn, dr, dv = cfg.num_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
    q = (q_a_normed.float() @ ckpt[a + "q_b_proj.weight"].float().T).reshape(-1, nh, dn + dr)
    kv = (kv_latent_normed.float() @ ckpt[a + "kv_b_proj.weight"].float().T).reshape(-1, nh, dn + dv)
    k = torch.cat((kv[..., :dn], k_pe.float()[:, None, :].expand(-1, nh, -1)), dim=-1)
    v = kv[..., dn:]
    n = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * A.DEEPSEEK_SCALE
    s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), v).reshape(n, nh * dv)
