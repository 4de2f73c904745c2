"""CPU oracle for the mixture-of-experts task bodies of the MPK decode megakernel.

TEST INFRASTRUCTURE ONLY (see oracle/mpk_ops.py for the rules).

Restates, vectorised over tokens:
  * group-aware sigmoid top-k routing -- include/mirage/persistent_kernel/tasks/blackwell/
    topk_sigmoid_sm100.cuh:75-362 (sigmoid in fp32, selection on score + bias, group score = sum of the two
    largest biased scores of the group, `topk_group` groups kept (ties: lowest group), other groups masked
    to -10000, top-k experts by repeated argmax (ties: lowest expert), weights = unbiased scores divided by
    (their sum in selection order + 1e-20), times the scaling factor; routing_indices[e, b] = 1-based slot
    or 0; list of active experts + count at index num_experts; the logits are zeroed afterwards);
  * block-scaled FP8 grouped GEMM for the expert projections -- fp8_group_gemm_sm100.cuh: float32 scales per
    (row, 128 columns) are FLOORED to a power of two by taking their exponent bits (:1378), fp32 accumulation,
    one bf16 rounding; tests/runtime_python/blackwell/sm100_fp8_moe/test_fp8_moe_gemm.py:40-190;
  * bf16 grouped GEMM (moe_w13_linear / moe_w2_linear), silu-mul on [gate | up] halves
    (tasks/ampere/silu_mul.cuh:20-42) and the weighted sum over experts plus residual
    (mul_sum_add_sm100.cuh:19-49).

Parity status: PINNED.  tests/golden/ref_moe.pt is produced by executing the reference tests' own oracle
functions (reference_sigmoid_routing, quantize_to_fp8, dequantize_fp8, float32_to_ue8m0_approx,
reference_moe_w13, reference_moe_w2) on the CPU; tests/test_oracle_golden.py compares.
"""
from __future__ import annotations

import torch

E4M3 = torch.float8_e4m3fn


def topk_sigmoid_routing(logits: torch.Tensor, bias: torch.Tensor, *, topk: int, num_groups: int, topk_group: int,
                         scaling: float):
    """logits [B, E] (bf16 or fp32), bias [E] fp32 ->
    (weights [B, topk] fp32, routing_indices [E, B] int32, active [E + 1] int32, chosen [B, topk] int64)."""
    B, E = logits.shape
    per = E // num_groups
    scores = 1.0 / (1.0 + torch.exp(-logits.float()))
    biased = scores + bias.float().unsqueeze(0)
    grouped = biased.view(B, num_groups, per)
    top2 = grouped.topk(2, dim=-1).values
    gscore = top2[..., 0] + top2[..., 1]
    selected = torch.zeros(B, num_groups, dtype=torch.bool)
    work = gscore.clone()
    for _ in range(topk_group):
        best = torch.full((B,), -1, dtype=torch.int64)
        best_s = torch.full((B,), -1e30)
        for g in range(num_groups):                     # strict '>' in ascending order: lowest group wins ties
            better = (~selected[:, g]) & (work[:, g] > best_s)
            best = torch.where(better, torch.full_like(best, g), best)
            best_s = torch.where(better, work[:, g], best_s)
        best = best.clamp(min=0)
        selected[torch.arange(B), best] = True
    masked = torch.where(selected.unsqueeze(-1).expand(B, num_groups, per).reshape(B, E), biased,
                         torch.full_like(biased, -10000.0))
    chosen = torch.zeros(B, topk, dtype=torch.int64)
    for k in range(topk):
        mx = masked.max(dim=-1, keepdim=True).values
        idx = torch.where(masked == mx, torch.arange(E).expand(B, E), torch.full((B, E), E)).min(dim=-1).values
        chosen[:, k] = idx
        masked[torch.arange(B), idx] = -10000.0
    picked = scores.gather(1, chosen)
    total = torch.zeros(B)
    for k in range(topk):                               # sequential fp32 sum in selection order
        total = total + picked[:, k]
    inv = 1.0 / (total + 1e-20)
    weights = picked * inv.unsqueeze(-1) * torch.tensor(scaling, dtype=torch.float32)
    routing = torch.zeros(E, B, dtype=torch.int32)
    for k in range(topk):
        routing[chosen[:, k], torch.arange(B)] = k + 1
    act = (routing != 0).any(dim=1).nonzero().reshape(-1).to(torch.int32)
    active = torch.full((E + 1,), -1, dtype=torch.int32)
    active[:act.numel()] = act
    active[E] = act.numel()
    return weights, routing, active, chosen


def topk_softmax_routing(logits: torch.Tensor, *, topk: int):
    """Softmax top-k routing: include/mirage/persistent_kernel/tasks/blackwell/topk_softmax_sm100.cuh:75-310 and the
    expression of its test, tests/runtime_python/blackwell/sm100_moe/test_gate_topk.py:34-43 -- softmax over the experts
    in fp32 (max subtracted), the k largest probabilities (repeated argmax, ties to the lower expert, :237-249), weights
    divided by the sum of the selected probabilities (renormalize = true at the generated call site,
    src/kernel/task_register.cc:2338).  -> (weights [B, topk] fp32, routing_indices [E, B] int32, active [E + 1] int32
    ascending, chosen [B, topk])."""
    B, E = logits.shape
    x = logits.float()
    p = torch.exp(x - x.amax(dim=1, keepdim=True))
    p = p / p.sum(dim=1, keepdim=True)
    masked = p.clone()
    chosen = torch.zeros(B, topk, dtype=torch.int64)
    for k in range(topk):
        mx = masked.max(dim=-1, keepdim=True).values
        idx = torch.where(masked == mx, torch.arange(E).expand(B, E), torch.full((B, E), E)).min(dim=-1).values
        chosen[:, k] = idx
        masked[torch.arange(B), idx] = -1.0
    picked = p.gather(1, chosen)
    total = torch.zeros(B)
    for k in range(topk):
        total = total + picked[:, k]
    weights = picked / total.unsqueeze(-1)
    routing = torch.zeros(E, B, dtype=torch.int32)
    for k in range(topk):
        routing[chosen[:, k], torch.arange(B)] = k + 1
    act = (routing != 0).any(dim=1).nonzero().reshape(-1).to(torch.int32)
    active = torch.full((E + 1,), -1, dtype=torch.int32)
    active[:act.numel()] = act
    active[E] = act.numel()
    return weights, routing, active, chosen


def quantize_fp8_f32(x: torch.Tensor):
    """Per-128-column float32-scale quantisation of the last dimension (test_fp8_moe_gemm.py:40-51)."""
    shape = x.shape
    blocks = x.float().reshape(*shape[:-1], shape[-1] // 128, 128)
    scale = (blocks.abs().amax(-1) / 448.0).clamp(min=1e-12)
    q = (blocks / scale.unsqueeze(-1)).reshape(shape).to(E4M3)
    return q, scale.float()


def floor_pow2(scale: torch.Tensor) -> torch.Tensor:
    """2 ** (exponent field - 127): what the grouped GEMM makes of a float32 scale."""
    e = (scale.float().contiguous().view(torch.int32) >> 23) & 0xFF
    return torch.exp2(e.float() - 127.0)


def _deq(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    shape = q.shape
    return (q.float().reshape(*shape[:-1], shape[-1] // 128, 128) * scale.unsqueeze(-1)).reshape(shape)


def moe_gemm_fp8(xq, xs, wq, ws, routing, *, topk: int, per_slot_input: bool):
    """Expert projections on e4m3 operands.

    xq [B, K] (w13: one row per token) or [B, topk, K] (w2: one row per token and slot), xs matching float32
    scales; wq [E, N, K], ws [E, N, K/128]; routing [E, B].  -> [B, topk, N] bf16 (unrouted slots zero).
    """
    E, N, K = wq.shape
    B = routing.shape[1]
    out = torch.zeros(B, topk, N, dtype=torch.bfloat16)
    xd = _deq(xq, floor_pow2(xs))
    for e in range(E):
        toks = routing[e].nonzero().reshape(-1)
        if toks.numel() == 0:
            continue
        wd = _deq(wq[e], floor_pow2(ws[e]))
        for b in toks.tolist():
            slot = int(routing[e, b]) - 1
            row = xd[b, slot] if per_slot_input else xd[b]
            out[b, slot] = (row @ wd.T).to(torch.bfloat16)
    return out


def moe_gemm_bf16(x, w, routing, *, topk: int, per_slot_input: bool):
    """bf16 expert projections (moe_w13_linear / moe_w2_linear): fp32 accumulation, one bf16 rounding."""
    E, N, K = w.shape
    B = routing.shape[1]
    out = torch.zeros(B, topk, N, dtype=torch.bfloat16)
    for e in range(E):
        for b in routing[e].nonzero().reshape(-1).tolist():
            slot = int(routing[e, b]) - 1
            row = x[b, slot] if per_slot_input else x[b]
            out[b, slot] = (row.float() @ w[e].float().T).to(torch.bfloat16)
    return out


def moe_silu_mul(mid: torch.Tensor) -> torch.Tensor:
    """[B, topk, 2I] -> [B, topk, I]: bf16(silu(gate)) * up with the product rounded to bf16."""
    I = mid.shape[-1] // 2
    g = mid[..., :I].float()
    act = (g / (1.0 + torch.exp(-g))).to(torch.bfloat16)
    return (act.float() * mid[..., I:].float()).to(torch.bfloat16)


def moe_mul_sum_add(inp: torch.Tensor, weights: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """out[b] = residual[b] + sum_k inp[b, k] * weights[b, k], accumulated in fp32 in slot order."""
    acc = residual.float().clone()
    for k in range(inp.shape[1]):
        acc = acc + inp[:, k].float() * weights[:, k:k + 1].float()
    return acc.to(torch.bfloat16)
