"""CPU oracle for the multi-head latent attention (MLA) decode tasks of the MPK decode megakernel.

TEST INFRASTRUCTURE ONLY (see oracle/mpk_ops.py for the rules).

Restates:
  * appending the new [c_latent (512) | k_pe (64)] rows of a request to the paged cache
    [pages, page_size, 576] -- include/mirage/persistent_kernel/tasks/blackwell/
    mla_kv_cache_gather_sm100.cuh:36-128 (step 1; k_pe rows may be padded to a wider stride);
  * absorbed multi-token decode: scores = q[576] . kv[576] * scale over the positions the token may see
    (token i of n new tokens of a sequence of length L sees positions < L - n + i + 1), softmax in fp32,
    output = probs . kv[:, :512], bf16 -- mla_mtp_decode_sm100.cuh / mla_reduce_sm100.cuh, oracle
    `pytorch_mla_ref` of tests/runtime_python/blackwell/sm100_mla/test_mla_mtp.py:44-69.

Parity status: PINNED.  tests/golden/ref_mla.pt is produced by executing `pytorch_mla_ref` of the reference's
test on the CPU; tests/test_oracle_golden.py compares.
"""
from __future__ import annotations

import math

import torch

D_K, D_V = 576, 512
# softmax scale the reference's generated call sites hard-code: (1 / sqrt(192)) * (0.1 * ln(40) + 1) ** 2
# (src/kernel/task_register.cc:3507-3516)
DEEPSEEK_SCALE = (1.0 / math.sqrt(192.0)) * (0.1 * math.log(40.0) + 1.0) ** 2


def mla_append(cache: torch.Tensor, c_latent_new: torch.Tensor, k_pe_new: torch.Tensor, pages, seq_len: int):
    """Write the n new rows at positions [seq_len - n, seq_len) of the request whose page list is `pages`."""
    n = c_latent_new.shape[0]
    page = cache.shape[1]
    for i in range(n):
        pos = seq_len - n + i
        row = cache[pages[pos // page], pos % page]
        row[:D_V] = c_latent_new[i, :D_V]
        row[D_V:] = k_pe_new[i, :D_K - D_V]


def gather_rows(cache: torch.Tensor, pages, seq_len: int) -> torch.Tensor:
    page = cache.shape[1]
    return torch.stack([cache[pages[p // page], p % page] for p in range(seq_len)])


def mla_decode_request(q: torch.Tensor, cache: torch.Tensor, pages, seq_len: int, scale: float) -> torch.Tensor:
    """q [n, H, 576] (the request's n new tokens, already appended to the cache) -> [n, H, 512] bf16."""
    n = q.shape[0]
    kv = gather_rows(cache, pages, seq_len).float()
    out = []
    for i in range(n):
        lim = seq_len - n + i + 1
        s = (q[i].float() @ kv[:lim].T) * scale
        p = torch.softmax(s, dim=-1)
        out.append((p @ kv[:lim, :D_V]).to(torch.bfloat16))
    return torch.stack(out)
