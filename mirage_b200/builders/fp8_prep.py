"""Host-side preparation of FP8 (e4m3) linear weights for the block-scaled linear tasks.

Checkpoints of the DeepSeek-V3 kind store a weight as e4m3 values plus one float32 scale per 128 x 128 block.
The block-scaled tensor-core instruction takes power-of-two scales (UE8M0, exponent only) per row and 128 columns,
so the reference re-quantises on the host (python/mirage/mpk/models/deepseek_v3/builder.py:475-542): de-quantise with
the checkpoint's block scales, pick for every (row, 128-column group) the smallest power of two s with
amax / 448 <= s, quantise again with s, and pack four consecutive exponents (biased by 127) into one uint32,
stored so that the words of one packed column are contiguous over the rows.  `requantize_for_ue8m0` does the same.
"""
from __future__ import annotations

from typing import Tuple

import torch

GROUP = 128
E4M3_MAX = 448.0


def dequantize_block_scaled(weight_fp8: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    """e4m3 [N, K] x float32 block scales [ceil(N/128), ceil(K/128)] -> float32 [N, K]."""
    n, k = weight_fp8.shape
    s = scale_inv.float().repeat_interleave(GROUP, 0)[:n].repeat_interleave(GROUP, 1)[:, :k]
    return weight_fp8.float() * s


def requantize_for_ue8m0(weight_fp8: torch.Tensor, scale_inv: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """-> (e4m3 [N, K], packed scales uint32 logical [N, ceil(K/512)] with the rows contiguous (strides (1, N4)),
    exponents int32 [N, K/128] for checking).  K must be a multiple of 128."""
    return quantize_ue8m0(dequantize_block_scaled(weight_fp8, scale_inv))


def quantize_ue8m0(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """A full-precision [N, K] weight -> e4m3 values with one power-of-two scale per row and 128 columns (the smallest
    power of two s with amax / 448 <= s), in the forms `requantize_for_ue8m0` returns."""
    n, k = weight.shape
    assert k % GROUP == 0, "K must be a multiple of 128"
    groups = k // GROUP
    w = weight.float().view(n, groups, GROUP)
    amax = w.abs().amax(-1).clamp(min=1e-12)
    exp = torch.ceil(torch.log2((amax / E4M3_MAX).clamp(min=1e-30)))
    q = (w / torch.exp2(exp)[..., None]).clamp(-E4M3_MAX, E4M3_MAX).reshape(n, k).to(torch.float8_e4m3fn)
    biased = (exp + 127).clamp(0, 254).to(torch.int64)
    return q.contiguous(), pack_ue8m0(biased), biased.to(torch.int32)


def pack_ue8m0(biased_exponents: torch.Tensor) -> torch.Tensor:
    """[N, groups] biased exponents -> uint32 [N, ceil(groups/4)], element (row, j) at row + j * N4 (N4 = N rounded
    up to 4): the column-major form the reference allocates for packed scales."""
    n, groups = biased_exponents.shape
    pk = (groups + 3) // 4
    padded = torch.zeros(n, pk * 4, dtype=torch.int64, device=biased_exponents.device)
    padded[:, :groups] = biased_exponents.to(torch.int64)
    p = padded.view(n, pk, 4)
    words = p[..., 0] | (p[..., 1] << 8) | (p[..., 2] << 16) | (p[..., 3] << 24)
    n4 = (n + 3) // 4 * 4
    out = torch.empty_strided((n, pk), (1, n4), dtype=torch.int32, device=words.device)
    out.copy_(words.to(torch.int64).where(words < 2 ** 31, words - 2 ** 32).to(torch.int32))
    return out.view(torch.uint32)


def packed_rows_contiguous(packed: torch.Tensor) -> torch.Tensor:
    """The same scale words as a plain row-major [N, pk] tensor (what `shuffle_tensors` interleaves)."""
    return packed.view(torch.int32).contiguous().view(torch.uint32)


def synthetic_block_scaled_weight(n: int, k: int, generator: torch.Generator, lo: float = 1e-3, hi: float = 1e-1):
    """Random e4m3 values with float32 128 x 128 block scales drawn log-uniformly from [lo, hi] -- the synthetic
    stand-in for an FP8 checkpoint tensor.  -> (e4m3 [N, K], float32 [ceil(N/128), ceil(K/128)])."""
    vals = (torch.randn(n, k, generator=generator) * 96.0).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    bn, bk = (n + GROUP - 1) // GROUP, (k + GROUP - 1) // GROUP
    u = torch.rand(bn, bk, generator=generator)
    scale = torch.exp(torch.log(torch.tensor(lo)) + u * (torch.log(torch.tensor(hi)) - torch.log(torch.tensor(lo))))
    return vals, scale.float()
