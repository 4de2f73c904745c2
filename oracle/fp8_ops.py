"""CPU oracle for the FP8 (e4m3, block-scaled) task bodies of the MPK decode megakernel.

TEST INFRASTRUCTURE ONLY (see oracle/mpk_ops.py for the rules).

Vectorised restatement of the reference's FP8 helpers and kernels:
  * per-token, per-128-group quantisation with UE8M0 (power-of-two, rounded UP) scales packed four to a
    uint32 -- tests/runtime_python/blackwell/common/sm100_fp8_scale_layout.py:65-117 and
    include/mirage/persistent_kernel/tasks/blackwell/per_token_group_quantize_fp8.cuh:33-160;
  * the float32-scale variant of the same kernel (`scale_ue8m0=False`, :123-133);
  * de-quantisation, sm100_fp8_scale_layout.py:128-150;
  * the block-scaled linear: sum_k (a * 2^ea)(w * 2^ew) in fp32, one bf16 rounding, optional residual --
    tests/runtime_python/blackwell/sm100_linear_fp8/test_linear_1d2d_fp8.py:67-74.

Parity status: PINNED.  tests/golden/ref_fp8.pt is produced by importing the reference's helper module
(sm100_fp8_scale_layout.py, plain torch) on the CPU; tests/test_oracle_golden.py compares.
"""
from __future__ import annotations

import torch

BLOCK_K = 128
FP8_MAX = 448.0
E4M3 = torch.float8_e4m3fn


def _groups(x: torch.Tensor) -> torch.Tensor:
    b, k = x.shape
    assert k % BLOCK_K == 0
    return x.float().view(b, k // BLOCK_K, BLOCK_K)


def encode_ue8m0(scale: torch.Tensor) -> torch.Tensor:
    """ceil(log2(scale)) + 127 clamped to [0, 255] (scales are rounded UP to a power of two)."""
    e = torch.ceil(torch.log2(torch.clamp(scale.float(), min=1e-30))).to(torch.int32) + 127
    return e.clamp(0, 255)


def decode_ue8m0(e: torch.Tensor) -> torch.Tensor:
    return torch.exp2(e.float() - 127.0)


def quantize_fp8_ue8m0(x: torch.Tensor):
    """-> (q [B,K] e4m3, exps [B,K/128] int32, packed [B, ceil(K/512)] int64 holding uint32 values)."""
    g = _groups(x)
    amax = g.abs().amax(-1).clamp(min=1e-10)
    exps = encode_ue8m0(amax / FP8_MAX)
    scale = decode_ue8m0(exps)
    q = torch.clamp(g / scale[..., None], -FP8_MAX, FP8_MAX).to(E4M3).view(x.shape)
    b, ng = exps.shape
    pk = (ng + 3) // 4
    padded = torch.zeros(b, pk * 4, dtype=torch.int64)
    padded[:, :ng] = exps.to(torch.int64)
    packed = (padded.view(b, pk, 4) << torch.tensor([0, 8, 16, 24])).sum(-1)
    return q, exps, packed


def quantize_fp8_f32scale(x: torch.Tensor):
    """float32 scale = amax / 448 per (token, 128-group); -> (q e4m3, scale [B, K/128] f32)."""
    g = _groups(x)
    scale = g.abs().amax(-1).clamp(min=1e-10) / FP8_MAX
    q = torch.clamp(g / scale[..., None], -FP8_MAX, FP8_MAX).to(E4M3).view(x.shape)
    return q, scale


def dequant(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """scale: [B, K/128] float32 multipliers."""
    return (_groups(q) * scale[..., None]).reshape(q.shape)


def linear_fp8(xq, x_exps, wq, w_exps, residual=None) -> torch.Tensor:
    """Block-scaled FP8 linear with UE8M0 exponents for both operands; bf16 result."""
    x = dequant(xq, decode_ue8m0(x_exps))
    w = dequant(wq, decode_ue8m0(w_exps))
    y = x @ w.T
    if residual is not None:
        y = y + residual.float()
    return y.to(torch.bfloat16)


def unpack_ue8m0(packed: torch.Tensor, num_groups: int) -> torch.Tensor:
    """[B, pk] uint32 values (any integer dtype) -> [B, num_groups] exponents."""
    p = packed.to(torch.int64) & 0xFFFFFFFF
    e = torch.stack([(p >> s) & 0xFF for s in (0, 8, 16, 24)], dim=-1).reshape(p.shape[0], -1)
    return e[:, :num_groups].to(torch.int32)
