"""CPU oracle for the Gumbel-max sampling task of the MPK decode megakernel.

TEST INFRASTRUCTURE ONLY (see oracle/mpk_ops.py for the rules).

Restates include/mirage/persistent_kernel/tasks/common/sampling.cuh:100-226 as the reference instantiates it
(src/kernel/task_register.cc:2048-2079: 256 threads, 4 columns per thread, bf16 logits, philox offset 0):

  * the random bits come from NVIDIA cuRAND's Philox4x32-10 generator (a third-party dependency, not in the
    reference tree; shipped with CUDA 12.9): curand_init(seed, subsequence, offset 0) + one curand_uniform4.
    Philox4x32-10 is the published counter-based generator of Salmon, Moraes, Dror and Shaw ("Parallel random
    numbers: as easy as 1, 2, 3", SC'11): ten rounds of two 32x32->64 multiplications with a Weyl key schedule;
    cuRAND puts the subsequence in counter words 2 and 3, the seed in the key, and maps a word x to the uniform
    x * 2^-32 + 2^-33;
  * columns 4q .. 4q+3 of row r take the four outputs of the block with subsequence (r % rows_per_task) * V + 4q,
    computed in 32-bit arithmetic (sampling.cuh:196-199), where rows_per_task is the number of rows one reference
    task sees (1 when the layer's grid is one task per row, as in demo/qwen3/demo_sampling.py:588-594);
  * gumbel = -ln2 * log2(-log2(u + 1e-20) + 1e-20) in fp32, rounded to bf16; key = bf16(logit + gumbel) (one bf16
    rounding); the largest key wins and equal keys go to the HIGHEST column, which is the order the reference's
    block reduction resolves ties in (its `+` keeps the right operand unless the left is strictly greater).

Parity status: PINNED on a GPU.  tests/test_gpu_sampling.py runs the real cuRAND generator
(oracle/curand_pin.cu -> oracle/_ref/libcurand_pin.so) and compares its uniforms bit for bit with this file.  The
Gumbel transform uses the device's approximate log2 in the reference (it is compiled with -use_fast_math), which a
host cannot reproduce bit for bit -- near u = 1 the two differ by up to a bf16 step of the noise -- so the GPU tests
take the noise from that library (cuRAND + the same expression under the same flag) for the exact comparisons
and use this file's float64 log2 only within a stated tolerance.  The reference's own test of the task needs its
compiled runtime and is not run.
"""
from __future__ import annotations

import numpy as np
import torch

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)


def philox4x32_10(counter: np.ndarray, key) -> np.ndarray:
    """counter [n, 4] uint32, key (k0, k1) -> [n, 4] uint32."""
    c = counter.astype(np.uint64)
    c0, c1, c2, c3 = c[:, 0], c[:, 1], c[:, 2], c[:, 3]
    k0, k1 = int(key[0]) & 0xFFFFFFFF, int(key[1]) & 0xFFFFFFFF
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint64(k0), lo1, hi0 ^ c3 ^ np.uint64(k1), lo0
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32)


def curand_uniform(x: np.ndarray) -> np.ndarray:
    """uint32 -> float32 in (0, 1]: x * 2^-32 + 2^-33 as one fused multiply-add."""
    a = np.float64(np.float32(2.3283064e-10))
    b = np.float64(np.float32(2.3283064e-10) / np.float32(2.0))
    return (x.astype(np.float32).astype(np.float64) * a + b).astype(np.float32)


def gumbel_from_uniform(u: np.ndarray) -> np.ndarray:
    f32 = np.float32
    inner = (-np.log2((u + f32(1e-20)).astype(np.float64))).astype(np.float32)
    outer = np.log2((inner + f32(1e-20)).astype(np.float64)).astype(np.float32)
    return (f32(-0.6931471806) * outer).astype(np.float32)


def uniforms(seed: int, first_subsequence: int, groups: int) -> np.ndarray:
    """The 4 * groups uniforms of the Philox blocks with subsequence first + 4 g, g < groups."""
    sub = np.uint64(first_subsequence) + np.uint64(4) * np.arange(groups, dtype=np.uint64)
    ctr = np.zeros((groups, 4), dtype=np.uint32)
    ctr[:, 2] = (sub & _MASK).astype(np.uint32)
    ctr[:, 3] = (sub >> np.uint64(32)).astype(np.uint32)
    bits = philox4x32_10(ctr, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    return curand_uniform(bits.reshape(-1))


def gumbel_row(seed: int, local_row: int, vocab: int) -> torch.Tensor:
    """bf16 noise of one row: [vocab]."""
    groups = (vocab + 3) // 4
    first = (local_row * vocab) & 0xFFFFFFFF           # 32-bit product, as the reference forms it
    sub32 = (np.uint64(first) + np.uint64(4) * np.arange(groups, dtype=np.uint64)) & _MASK
    ctr = np.zeros((groups, 4), dtype=np.uint32)
    ctr[:, 2] = sub32.astype(np.uint32)
    bits = philox4x32_10(ctr, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    g = gumbel_from_uniform(curand_uniform(bits.reshape(-1)))[:vocab]
    return torch.from_numpy(g).to(torch.bfloat16)


def sampling_keys(logits: torch.Tensor, seed: int, rows_per_task: int = 1, noise_fn=None) -> torch.Tensor:
    """logits [B, V] bf16 -> keys [B, V] bf16.  `noise_fn(seed, local_row, V)` replaces gumbel_row (the tests pass the
    real cuRAND stream with the device's own log2 there, which makes the comparison exact)."""
    B, V = logits.shape
    noise_fn = noise_fn or gumbel_row
    noise = {}
    out = torch.empty(B, V, dtype=torch.bfloat16)
    for b in range(B):
        lr = b % max(rows_per_task, 1)
        if lr not in noise:
            noise[lr] = noise_fn(seed, lr, V)
        out[b] = (logits[b].to(torch.bfloat16).float() + noise[lr].float()).to(torch.bfloat16)
    return out


def sampling_from_logits(logits: torch.Tensor, seed: int, rows_per_task: int = 1, noise_fn=None) -> torch.Tensor:
    """-> ids [B] int64 (largest key, ties to the highest column)."""
    keys = sampling_keys(logits, seed, rows_per_task, noise_fn).float()
    V = keys.shape[1]
    rev = torch.flip(keys, dims=[1])
    return (V - 1 - torch.argmax(rev, dim=1)).to(torch.int64)   # argmax returns the first maximum of the reversed row
