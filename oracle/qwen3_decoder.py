"""CPU oracle for a Qwen3-architecture decoder driven by the MPK batching state.

TEST INFRASTRUCTURE ONLY (see oracle/mpk_ops.py for the rules).  Also the
timed CPU baseline of the benchmark (reported, never a target).

Restates the reference's PyTorch forward of the graph its Qwen3 builder emits:
demo/qwen3/models/modeling_qwen3.py -- Qwen3Attention.forward :261-335 (q/k norm
per head -> RoPE -> cache write -> GQA attention -> o_proj [-> all_reduce]),
Qwen3MLP.forward :155-166, Qwen3DecoderLayer.forward :357-396, decode loop
demo/qwen3/demo.py:763-782 -- using the op order and rounding points of
python/mirage/mpk/models/qwen3/builder.py:252-522 (embed, per layer
rmsnorm -> qkv linear -> paged attention -> o_proj + residual [-> allreduce] ->
rmsnorm -> gate_up linear -> silu_mul -> down + residual [-> allreduce], final
rmsnorm -> lm_head -> argmax).  RMSNorm uses eps = 1e-6 in fp32 as the kernels do
(the demo's torch module drops eps and runs in bf16; that difference is far
inside the 2e-2 tolerance).

Parity status: PINNED against HuggingFace transformers' Qwen3ForCausalLM on a
small configuration (fixture tests/golden/qwen3_tiny_hf.pt, made by
tests/golden/make_golden.py) and, op by op, against the reference's own test
oracles through oracle/mpk_ops.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from . import mpk_ops as ops
from .batching import BatchState

BF16 = torch.bfloat16


@dataclass
class Qwen3Config:
    num_layers: int = 36
    hidden_size: int = 4096
    num_q_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 12288
    vocab_size: int = 151936
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    max_position: int = 4096

    @staticmethod
    def qwen3_8b(num_layers: int = 36) -> "Qwen3Config":
        return Qwen3Config(num_layers=num_layers)

    @staticmethod
    def tiny() -> "Qwen3Config":
        return Qwen3Config(num_layers=2, hidden_size=256, num_q_heads=4, num_kv_heads=2,
                           head_dim=128, intermediate_size=512, vocab_size=1024,
                           max_position=512)


def make_weights(cfg: Qwen3Config, seed: int, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Random-init weights with HuggingFace parameter names.

    Linears ~ N(0, 0.02), norm weights 1 + N(0, 0.02); drawn in fp32 on the CPU
    generator (so CPU oracle and GPU runs share bit-identical values), cast to bf16.
    """
    g = torch.Generator(device="cpu").manual_seed(seed)

    def lin(n, k):
        return (torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02).to(BF16).to(device)

    def norm(n):
        return (1.0 + torch.randn(n, generator=g, dtype=torch.float32) * 0.02).to(BF16).to(device)

    h, d = cfg.hidden_size, cfg.head_dim
    w = {"model.embed_tokens.weight": lin(cfg.vocab_size, h)}
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = norm(h)
        w[p + "self_attn.q_proj.weight"] = lin(cfg.num_q_heads * d, h)
        w[p + "self_attn.k_proj.weight"] = lin(cfg.num_kv_heads * d, h)
        w[p + "self_attn.v_proj.weight"] = lin(cfg.num_kv_heads * d, h)
        w[p + "self_attn.q_norm.weight"] = norm(d)
        w[p + "self_attn.k_norm.weight"] = norm(d)
        w[p + "self_attn.o_proj.weight"] = lin(h, cfg.num_q_heads * d)
        w[p + "post_attention_layernorm.weight"] = norm(h)
        w[p + "mlp.gate_proj.weight"] = lin(cfg.intermediate_size, h)
        w[p + "mlp.up_proj.weight"] = lin(cfg.intermediate_size, h)
        w[p + "mlp.down_proj.weight"] = lin(h, cfg.intermediate_size)
    w["model.norm.weight"] = norm(h)
    w["lm_head.weight"] = lin(cfg.vocab_size, h)
    return w


class Qwen3Oracle:
    """Runs decoder iterations on the batches a BatchState describes.

    world_size > 1 emulates tensor parallelism the way the reference shards it
    (demo/qwen3/demo.py:13-29): q/kv heads and gate/up rows split by rank,
    o_proj/down_proj split along K, bf16 partial outputs summed in fp32
    (oracle.mpk_ops.allreduce), residual added once.
    """

    def __init__(self, cfg: Qwen3Config, weights: Dict[str, torch.Tensor], *,
                 max_num_pages: int, page_size: int, world_size: int = 1,
                 device: str = "cpu", residual_after_sum: bool = False):
        self.cfg, self.w, self.ws, self.device = cfg, weights, world_size, device
        # Where the residual enters a row-parallel projection under tensor parallelism.  False: rank 0 adds it to
        # its partial before the allreduce, i.e. it is rounded to bf16 together with that partial (the reference's
        # linear_with_residual_layer on rank 0 only, python/mirage/mpk/persistent_kernel.py:1783-1787).  True: the
        # bf16 partials are summed in fp32, the residual is added to that sum, one rounding -- what the fused
        # allreduce of mirage_b200 computes.  Both add the residual once; they differ by one bf16 rounding of a
        # residual-sized value per projection.
        self.residual_after_sum = residual_after_sum
        self.page_size = page_size
        hkv = cfg.num_kv_heads
        self.k_cache = [torch.zeros(max_num_pages, page_size, hkv, cfg.head_dim, dtype=BF16, device=device)
                        for _ in range(cfg.num_layers)]
        self.v_cache = [torch.zeros_like(k) for k in self.k_cache]
        cos, sin = ops.rope_tables(cfg.head_dim, cfg.max_position, cfg.rope_theta)
        self.cos, self.sin = cos.to(device), sin.to(device)
        self.last_logits: Optional[torch.Tensor] = None
        self.last_hidden: Optional[torch.Tensor] = None

    # ---- one transformer layer on the active tokens ---------------------
    def _attention(self, li: int, x_norm: torch.Tensor, reqs) -> torch.Tensor:
        cfg, p = self.cfg, f"model.layers.{li}."
        d, hq, hkv = cfg.head_dim, cfg.num_q_heads, cfg.num_kv_heads
        g = hq // hkv
        q = self._proj(p + "self_attn.q_proj.weight", x_norm).view(-1, hkv, g, d)
        k = self._proj(p + "self_attn.k_proj.weight", x_norm).view(-1, hkv, 1, d)
        v = self._proj(p + "self_attn.v_proj.weight", x_norm).view(-1, hkv, 1, d)
        qkv = torch.cat((q, k, v), dim=2).reshape(x_norm.shape[0], -1)  # packed per kv head
        out = torch.empty(x_norm.shape[0], hq * d, dtype=BF16, device=x_norm.device)
        for (q0, q1), pages, seq_len in reqs:
            if q1 == q0:
                continue
            out[q0:q1] = ops.paged_attention_request(
                qkv[q0:q1], self.k_cache[li], self.v_cache[li], pages, seq_len, hq, hkv,
                self.w[p + "self_attn.q_norm.weight"], self.w[p + "self_attn.k_norm.weight"],
                self.cos, self.sin, cfg.rms_eps)
        return out

    def _proj(self, key: str, x_in: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One projection of a decoder layer (bf16 here; the FP8 oracle overrides it)."""
        return ops.linear(x_in, self.w[key], residual)

    def _row_parallel(self, x_in: torch.Tensor, key: str, residual: torch.Tensor) -> torch.Tensor:
        if self.ws == 1:
            return self._proj(key, x_in, residual)
        w = self.w[key]
        kk = w.shape[1] // self.ws
        if self.residual_after_sum:
            parts = [ops.linear(x_in[:, r * kk:(r + 1) * kk], w[:, r * kk:(r + 1) * kk]) for r in range(self.ws)]
            acc = residual.float()
            for part in parts:
                acc = acc + part.float()
            return acc.to(BF16)
        parts = [ops.linear(x_in[:, r * kk:(r + 1) * kk], w[:, r * kk:(r + 1) * kk],
                            residual if r == 0 else None) for r in range(self.ws)]
        return ops.allreduce(parts)

    def forward_tokens(self, token_ids: torch.Tensor, reqs) -> torch.Tensor:
        """token_ids [T]; reqs = [((q0,q1), page_ids, seq_len), ...] -> logits [T, vocab] (bf16)."""
        cfg = self.cfg
        x = ops.embedding(token_ids.to(self.device), self.w["model.embed_tokens.weight"])
        for li in range(cfg.num_layers):
            p = f"model.layers.{li}."
            xn = ops.rmsnorm(x, self.w[p + "input_layernorm.weight"], cfg.rms_eps)
            attn = self._attention(li, xn, reqs)
            x = self._row_parallel(attn, p + "self_attn.o_proj.weight", x)
            xn = ops.rmsnorm(x, self.w[p + "post_attention_layernorm.weight"], cfg.rms_eps)
            gate = self._proj(p + "mlp.gate_proj.weight", xn)
            up = self._proj(p + "mlp.up_proj.weight", xn)
            act = ops.silu_mul(torch.cat((gate, up), dim=1), 1)
            x = self._row_parallel(act, p + "mlp.down_proj.weight", x)
        self.last_hidden = x
        xn = ops.rmsnorm(x, self.w["model.norm.weight"], cfg.rms_eps)
        logits = ops.linear(xn, self.w["lm_head.weight"])
        self.last_logits = logits
        return logits

    # ---- driven by the batching state ----------------------------------
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
        ids = torch.from_numpy(st.input_tokens[:n].copy())
        logits = self.forward_tokens(ids, reqs)
        st.output_tokens[:n] = ops.argmax(logits).cpu().numpy()
        return True


class Qwen3Fp8Oracle(Qwen3Oracle):
    """The same decoder with FP8 (e4m3) projections inside the layers, as BASELINE configuration 4 words it: weights
    given as e4m3 values + float32 128 x 128 block scales, re-quantised on the host to power-of-two scales per row and
    128 columns (python/mirage/mpk/models/deepseek_v3/builder.py:475-542, restated in oracle.fp8_ops terms), bf16
    activations quantised per token and 128 columns right before every projection
    (per_token_group_quantize_fp8.cuh:33-160), block-scaled product accumulated in fp32 and rounded once
    (test_linear_1d2d_fp8.py:67-74).  Embedding, norms, attention and the lm_head stay bf16.

    `fp8_weights[name] = (e4m3 [N, K], float32 block scales)`.  `exact_scales=True` skips the re-quantisation of the
    weights and multiplies by the checkpoint's float32 block scales instead: the result the power-of-two rounding is
    measured against (tests report the gap; the kernels implement the re-quantised form).
    """

    def __init__(self, cfg, weights, fp8_weights, *, exact_scales: bool = False, **kw):
        super().__init__(cfg, weights, **kw)
        from . import fp8_ops as F
        self.F, self.exact = F, exact_scales
        self.q = {}
        for name, (wq, scale_inv) in fp8_weights.items():
            n, k = wq.shape
            wf = wq.float() * scale_inv.float().repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :k]
            if exact_scales:
                self.q[name] = wf
            else:
                q, exps, _ = F.quantize_fp8_ue8m0(wf)      # the reference's host re-quantisation is this quantiser
                self.q[name] = (q, exps)

    def _proj(self, key, x_in, residual=None):
        F = self.F
        xq, xe, _ = F.quantize_fp8_ue8m0(x_in)
        if self.exact:
            y = F.dequant(xq, F.decode_ue8m0(xe)) @ self.q[key].T
            if residual is not None:
                y = y + residual.float()
            return y.to(BF16)
        wq, we = self.q[key]
        return F.linear_fp8(xq, xe, wq, we, residual)

    def _row_parallel(self, x_in, key, residual):
        """o_proj / down_proj with the input columns split over the ranks: every rank quantises its slice of the
        activations (the 128-column groups do not straddle ranks), multiplies with its columns of the weight and rounds
        its partial to bf16; the partials are summed in fp32 in rank order and the residual is added once to the sum."""
        if self.ws == 1:
            return self._proj(key, x_in, residual)
        assert not self.exact
        F = self.F
        wq, we = self.q[key]
        kk = wq.shape[1] // self.ws
        assert kk % 128 == 0
        acc = residual.float()
        for r in range(self.ws):
            xq, xe, _ = F.quantize_fp8_ue8m0(x_in[:, r * kk:(r + 1) * kk].contiguous())
            part = F.linear_fp8(xq, xe, wq[:, r * kk:(r + 1) * kk], we[:, r * kk // 128:(r + 1) * kk // 128])
            acc = acc + part.float()
        return acc.to(BF16)


def greedy_generate(cfg: Qwen3Config, weights, prompts: List[List[int]], max_seq_length: int, *,
                    max_num_batched_requests: int, max_num_batched_tokens: int,
                    max_num_pages: int, page_size: int, eos_token_id: int = -1,
                    max_iterations: int = 1 << 30, world_size: int = 1,
                    keep_logits: bool = False, fp8_weights=None):
    """Offline-mode generation exactly as the megakernel's scheduler batches it."""
    tokens = np.zeros((len(prompts), max_seq_length), np.int64)
    plen = np.zeros(len(prompts), np.int32)
    for i, p in enumerate(prompts):
        tokens[i, :len(p)] = p
        plen[i] = len(p)
    st = BatchState(tokens, plen, max_num_batched_requests=max_num_batched_requests,
                    max_num_batched_tokens=max_num_batched_tokens, max_num_pages=max_num_pages,
                    page_size=page_size, eos_token_id=eos_token_id)
    if fp8_weights is not None:
        orc = Qwen3Fp8Oracle(cfg, weights, fp8_weights, max_num_pages=max_num_pages, page_size=page_size)
    else:
        orc = Qwen3Oracle(cfg, weights, max_num_pages=max_num_pages, page_size=page_size, world_size=world_size)
    logits_log = []
    it = 0
    while it < max_iterations and orc.run_iteration(st):
        if keep_logits:
            logits_log.append(orc.last_logits.clone())
        it += 1
    return st, orc, logits_log
