"""Synthetic FP8 'checkpoints' for the decoder tests: e4m3 projection weights with float32 128 x 128 block scales
drawn log-uniformly from [1e-3, 1e-1]; the stored values are N(0, 0.02) / scale, so that value x scale keeps the
magnitude of an ordinary random-init weight."""
import torch

PROJ = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
        "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight")


def fp8_checkpoint(cfg, weights, seed):
    g = torch.Generator().manual_seed(seed)
    lo, hi = torch.log(torch.tensor(1e-3)), torch.log(torch.tensor(1e-1))
    out = {}
    for i in range(cfg.num_layers):
        for k in PROJ:
            name = f"model.layers.{i}.{k}"
            n, kk = weights[name].shape
            scale = torch.exp(lo + torch.rand((n + 127) // 128, (kk + 127) // 128, generator=g) * (hi - lo)).float()
            per_elem = scale.repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :kk]
            q = (torch.randn(n, kk, generator=g) * 0.02 / per_elem).clamp(-448, 448).to(torch.float8_e4m3fn)
            out[name] = (q, scale)
    return out
