"""CPU oracle for the task bodies of the MPK decode megakernel.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module;
it is the checker used by the tests, by the smoke entry point and by the CPU
baseline leg of the benchmark.

Each function restates, in plain PyTorch on whatever device its inputs live on
(CPU in the unit tests), the arithmetic of one reference task body or of the
PyTorch function the reference's own test uses to check that body.  File:line
citations are relative to the root of mirage-project/mirage.

Parity status: PINNED.  tests/golden/ holds fixtures produced by executing the
reference's own test-oracle functions (extracted from its test files, see
tests/golden/make_golden.py) and by HuggingFace's Qwen3 implementation, and
tests/test_oracle_golden.py checks every function below against them.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

BF16 = torch.bfloat16
F32 = torch.float32


# --------------------------------------------------------------------------
# norms / linears / activations
# --------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm with fp32 statistics and a single bf16 rounding.

    Follows tests/runtime_python/test_multitoken_paged_attention.py:43-51 and
    tests/runtime_python/test_mode/test_rmsnorm_testmode.py:16-20; the kernel is
    include/mirage/persistent_kernel/tasks/hopper/rmsnorm_hopper.cuh:19-155
    (fp32 sum of squares, rsqrt(mean + eps)).
    """
    xf = x.to(F32)
    var = xf.pow(2).mean(-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps) * weight.to(F32)).to(x.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Y[B,N] = X[B,K] . W[N,K]^T (+ R), fp32 accumulate, one bf16 rounding.

    include/mirage/persistent_kernel/tasks/blackwell/linear_sm100_mpk.cuh:31-735;
    checked in the reference by tests/runtime_python/test_mode/
    test_qwen3_mlp_testmode.py:145-148.
    """
    y = x.to(F32) @ w.to(F32).T
    if residual is not None:
        y = y + residual.to(F32)
    return y.to(x.dtype)


def rmsnorm_linear(x, g, w, eps: float = 1e-6) -> torch.Tensor:
    """Fused RMSNorm + linear: ((x * rsqrt(mean(x^2)+eps)) * g) @ W^T.

    tests/runtime_python/test_norm_linear.py:14-20 (torch_rms_norm) for
    include/mirage/persistent_kernel/tasks/ampere/norm_linear.cuh:30-459.
    The normalised activations are rounded to bf16 before the matmul, which is
    what the unfused rmsnorm_layer -> linear_layer pair of the Qwen3 builder
    (python/mirage/mpk/models/qwen3/builder.py:325-338) produces.
    """
    return linear(rmsnorm(x, g, eps), w)


def silu_mul(mid: torch.Tensor, num_groups: int = 1) -> torch.Tensor:
    """SwiGLU on a group-interleaved [gate | up] tensor.

    include/mirage/persistent_kernel/tasks/ampere/silu_mul.cuh:20-42: silu in
    fp32, rounded to bf16, then a bf16 multiply by `up`.  `mid` is [B, 2*I]
    laid out as `num_groups` blocks of [gate I/g | up I/g] (the layout the
    builder's shuffle_tensors creates, python/mirage/mpk/models/utils.py:34-47).
    """
    b, two_i = mid.shape
    i = two_i // 2
    per = i // num_groups
    m = mid.view(b, num_groups, 2, per)
    gate, up = m[:, :, 0, :], m[:, :, 1, :]
    act = torch.nn.functional.silu(gate.to(F32)).to(mid.dtype)
    return (act * up).reshape(b, i)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather; negative ids give zero rows.

    include/mirage/persistent_kernel/tasks/ampere/embedding.cuh:43-72.
    """
    ids = ids.reshape(-1).to(torch.int64)
    out = table[ids.clamp(min=0)]
    out = out.clone()
    out[ids < 0] = 0
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Greedy token: lowest index among maxima.

    include/mirage/persistent_kernel/tasks/blackwell/argmax_sm100.cuh:79-167
    (strict '>' comparison so the first maximum wins).
    """
    return torch.argmax(logits.to(F32), dim=-1).to(torch.int64)


def shuffle_rows(tensors: Sequence[torch.Tensor], num_groups: int) -> torch.Tensor:
    """Interleave equal row-chunks of several matrices: [A0 B0 C0 A1 B1 C1 ...].

    python/mirage/mpk/models/utils.py:34-114 (shuffle_tensors, dim 0).
    """
    parts = [t.reshape(num_groups, t.shape[0] // num_groups, *t.shape[1:]) for t in tensors]
    return torch.cat(parts, dim=1).reshape(-1, *tensors[0].shape[1:]).contiguous()


# --------------------------------------------------------------------------
# rotary embedding
# --------------------------------------------------------------------------
def rope_tables(head_dim: int, max_pos: int, theta: float = 1e6):
    """bf16 cos/sin tables [max_pos, head_dim] in the NeoX (half-split) layout.

    demo/qwen3/models/modeling_qwen3.py:94-117 (cos/sin computed in fp32 from
    inv_freq = theta^(-2i/d), concatenated twice, cast to bf16).
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=F32) / head_dim))
    pos = torch.arange(max_pos, dtype=F32)
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(BF16), emb.sin().to(BF16)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin in fp32 on bf16-rounded inputs, bf16 result.

    tests/runtime_python/test_multitoken_paged_attention.py:21-40; kernel
    include/mirage/persistent_kernel/tasks/blackwell/norm_sm100.cuh:96-126.
    """
    xf = x.to(F32)
    return (xf * cos.to(F32) + rotate_half(xf) * sin.to(F32)).to(x.dtype)


# --------------------------------------------------------------------------
# paged GQA attention for one request
# --------------------------------------------------------------------------
def paged_attention_request(
    qkv: torch.Tensor,            # [n_new, (Hq + 2*Hkv) * D]; per kv head: [q*G | k | v]
    k_cache: torch.Tensor,        # [num_pages, page, Hkv, D]  (updated in place)
    v_cache: torch.Tensor,
    page_ids: Sequence[int],      # pages of this request, in order
    seq_len: int,                 # length INCLUDING the n_new tokens
    num_q_heads: int,
    num_kv_heads: int,
    q_norm_w: Optional[torch.Tensor],
    k_norm_w: Optional[torch.Tensor],
    cos: Optional[torch.Tensor],
    sin: Optional[torch.Tensor],
    eps: float = 1e-6,
) -> torch.Tensor:
    """Multi-token paged attention with fused QK-norm, RoPE and KV append.

    Restates torch_multitoken_paged_attention,
    tests/runtime_python/test_multitoken_paged_attention.py:54-122, generalised
    from one kv head to Hkv heads with the packed per-kv-head layout of
    include/mirage/persistent_kernel/tasks/blackwell/attention_sm100.cuh:34-666:
    new K (normalised, rotated) and V are written to the cache at positions
    seq_len-n_new .. seq_len-1, scores are scaled by 1/sqrt(D), the new tokens
    see each other causally, softmax in fp32.
    Returns [n_new, Hq * D] bf16.
    """
    n_new = qkv.shape[0]
    d = k_cache.shape[-1]
    page = k_cache.shape[1]
    g = num_q_heads // num_kv_heads
    packed = qkv.view(n_new, num_kv_heads, g + 2, d)
    q = packed[:, :, :g, :]                      # [n, Hkv, G, D]
    k_new = packed[:, :, g, :]                   # [n, Hkv, D]
    v_new = packed[:, :, g + 1, :]
    pos = torch.arange(seq_len - n_new, seq_len)
    if q_norm_w is not None:
        q = rmsnorm(q, q_norm_w, eps)
        k_new = rmsnorm(k_new, k_norm_w, eps)
    if cos is not None:
        q = apply_rope(q, cos[pos][:, None, None, :], sin[pos][:, None, None, :])
        k_new = apply_rope(k_new, cos[pos][:, None, :], sin[pos][:, None, :])
    for i, p in enumerate(pos.tolist()):
        pg, off = page_ids[p // page], p % page
        k_cache[pg, off] = k_new[i]
        v_cache[pg, off] = v_new[i]
    idx = torch.tensor(list(page_ids), dtype=torch.int64)
    kk = k_cache[idx].reshape(-1, num_kv_heads, d)[:seq_len].to(F32)   # [S, Hkv, D]
    vv = v_cache[idx].reshape(-1, num_kv_heads, d)[:seq_len].to(F32)
    scores = torch.einsum("nhgd,shd->nhgs", q.to(F32), kk) / math.sqrt(d)
    kv_pos = torch.arange(seq_len)
    mask = kv_pos[None, :] > pos[:, None]        # [n, S]
    scores = scores.masked_fill(mask[:, None, None, :], float("-inf"))
    p_attn = torch.softmax(scores, dim=-1)
    out = torch.einsum("nhgs,shd->nhgd", p_attn, vv)
    return out.reshape(n_new, num_q_heads * d).to(qkv.dtype)


# --------------------------------------------------------------------------
# tensor-parallel allreduce
# --------------------------------------------------------------------------
def allreduce(partials: Sequence[torch.Tensor]) -> torch.Tensor:
    """Sum over ranks in fp32, one bf16 rounding.

    include/mirage/persistent_kernel/tasks/blackwell/allreduce.cuh:377-450
    (multimem.ld_reduce ... acc::f32); reference check
    tests/runtime_python/hopper/allreduce/test_allreduce.py:40-56.
    """
    acc = partials[0].to(F32)
    for p in partials[1:]:
        acc = acc + p.to(F32)
    return acc.to(partials[0].dtype)
