"""Generate the golden fixtures in this directory from the reference itself.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py <path of the mirage-project/mirage checkout>

The reference's per-kernel tests are scripts that build a CUDA extension at import
time, so they cannot be imported on a CPU-only machine.  Their *oracle functions*
are plain PyTorch, though: this script parses each test file, executes only the
selected function definitions (ast.FunctionDef nodes, unmodified) in a namespace
that provides torch/numpy and the module-level constants those functions read, and
runs them on the CPU with seeded inputs.  A second group of fixtures comes from
HuggingFace transformers' Qwen3ForCausalLM on a tiny configuration.

Outputs (torch.save dictionaries of small tensors):
  ref_rmsnorm.pt          torch_rmsnorm      tests/runtime_python/test_mode/test_rmsnorm_testmode.py:16-20
  ref_norm_linear.pt      torch_rms_norm     tests/runtime_python/test_norm_linear.py:14-20
  ref_paged_attention.pt  torch_multitoken_paged_attention (+rmsnorm, apply_rotary_pos_emb)
                                             tests/runtime_python/test_multitoken_paged_attention.py:21-122
  ref_mlp.pt              MLP reference      tests/runtime_python/test_mode/test_qwen3_mlp_testmode.py:145-148
  ref_allreduce.pt        sum over ranks     tests/runtime_python/hopper/allreduce/test_allreduce.py
  ref_fp8.pt              quantize_to_fp8_packed_ue8m0 / dequant_from_packed_ue8m0 / FP8 linear reference
                                             tests/runtime_python/blackwell/common/sm100_fp8_scale_layout.py:65-150,
                                             tests/runtime_python/blackwell/sm100_linear_fp8/test_linear_1d2d_fp8.py:67-74
  ref_moe.pt              reference_sigmoid_routing   tests/runtime_python/blackwell/sm100_moe_sigmoid/test_gate_topk_sigmoid.py:27-76
                          quantize_to_fp8 / dequantize_fp8 / float32_to_ue8m0_approx / reference_moe_w13 / reference_moe_w2
                                             tests/runtime_python/blackwell/sm100_fp8_moe/test_fp8_moe_gemm.py:40-190
                          (string constants "cuda" inside those functions are rewritten to "cpu"; nothing else is changed)
  ref_mla.pt              pytorch_mla_ref   tests/runtime_python/blackwell/sm100_mla/test_mla_mtp.py:44-69
  qwen3_tiny_hf.pt        HF Qwen3ForCausalLM logits for a 2-layer configuration
"""
from __future__ import annotations

import ast
import io
import contextlib
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


class _CudaToCpu(ast.NodeTransformer):
    """device="cuda" literals -> "cpu" (the only edit ever made to an extracted reference function)."""

    def visit_Constant(self, node):
        return ast.copy_location(ast.Constant("cpu"), node) if node.value == "cuda" else node


def load_functions(path: str, names, extra_globals=None, on_cpu=False):
    """Execute only the named top-level function definitions of a python file."""
    src = open(path).read()
    tree = ast.parse(src)
    keep = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    if on_cpu:
        keep = [ast.fix_missing_locations(_CudaToCpu().visit(n)) for n in keep]
    missing = set(names) - {n.name for n in keep}
    assert not missing, f"{path}: functions not found: {missing}"
    ns = {"torch": torch, "np": np, "F": F, "__name__": "ref_extract"}
    ns.update(extra_globals or {})
    exec(compile(ast.Module(body=keep, type_ignores=[]), path, "exec"), ns)
    return ns


def main(ref_root: str):
    T = os.path.join(ref_root, "tests", "runtime_python")
    bf16 = torch.bfloat16

    # ---- rmsnorm --------------------------------------------------------
    ns = load_functions(os.path.join(T, "test_mode", "test_rmsnorm_testmode.py"), ["torch_rmsnorm"])
    g = torch.Generator().manual_seed(11)
    x = torch.randn(4, 4096, generator=g).to(bf16)
    w = torch.randn(4096, generator=g).to(bf16)
    torch.save({"x": x, "w": w, "eps": 1e-6, "out": ns["torch_rmsnorm"](x, w, 1e-6)},
               os.path.join(HERE, "ref_rmsnorm.pt"))

    # ---- fused norm + linear (BASELINE config 1 shape, reduced N) -------
    ns = load_functions(os.path.join(T, "test_norm_linear.py"), ["torch_rms_norm"])
    g = torch.Generator().manual_seed(0)
    x = torch.randn(8, 4096, generator=g).to(bf16)
    gam = (1 + 0.02 * torch.randn(1, 4096, generator=g)).to(bf16)
    W = (0.02 * torch.randn(24, 4096, generator=g)).to(bf16)
    # the reference function runs in the dtype of its inputs; evaluate it in fp32 on the
    # bf16-valued inputs so the fixture holds the exact formula, not CPU bf16 matmul noise
    out = ns["torch_rms_norm"](x.float(), gam.float(), W.float(), 1e-6)
    torch.save({"x": x, "g": gam, "w": W, "eps": 1e-6, "out_f32": out},
               os.path.join(HERE, "ref_norm_linear.pt"))

    # ---- multi-token paged attention -----------------------------------
    consts = dict(qo_heads=4, kv_heads=1, head_dim=128, page_size=64, max_num_pages=3,
                  prompt_len=40, max_tokens=3, device="cpu", dtype=torch.float32)
    ns = load_functions(os.path.join(T, "test_multitoken_paged_attention.py"),
                        ["rotate_half", "apply_rotary_pos_emb", "rmsnorm",
                         "torch_multitoken_paged_attention"], consts)
    g = torch.Generator().manual_seed(7)
    H, D, P = 4, 128, 64
    n_new, prompt_len = consts["max_tokens"], consts["prompt_len"]
    kc = torch.randn(3, P, D, generator=g).to(bf16)
    vc = torch.randn(3, P, D, generator=g).to(bf16)
    qkv = torch.randn(n_new, (H + 2) * D, generator=g).to(bf16)
    cos = torch.randn(64, D, generator=g).to(bf16)
    sin = torch.randn(64, D, generator=g).to(bf16)
    qn = torch.randn(1, D, generator=g).to(bf16)
    kn = torch.randn(1, D, generator=g).to(bf16)
    page_ids = torch.tensor([2, 0, 1], dtype=torch.int32)
    indptr = torch.tensor([0, 1], dtype=torch.int32)
    last = torch.tensor([prompt_len + n_new], dtype=torch.int32)
    # the reference test pre-writes the raw new K/V into the cache, then calls its oracle
    kc_ref, vc_ref = kc.clone(), vc.clone()
    kc_ref[page_ids[0], prompt_len:prompt_len + n_new] = qkv[:, H * D:(H + 1) * D]
    vc_ref[page_ids[0], prompt_len:prompt_len + n_new] = qkv[:, (H + 1) * D:]
    q = qkv[:, :H * D].reshape(n_new, H, D)
    with contextlib.redirect_stdout(io.StringIO()):
        # evaluated in fp32 on bf16-valued inputs except where the function itself rounds
        out = ns["torch_multitoken_paged_attention"](
            q.clone(), kc_ref, vc_ref, indptr, page_ids, last, 0, n_new, True, True,
            qn, kn, cos[:prompt_len + n_new + 1], sin[:prompt_len + n_new + 1], eps=1e-6)
    torch.save({"qkv": qkv, "k_cache": kc, "v_cache": vc, "page_ids": page_ids,
                "seq_len": prompt_len + n_new, "cos": cos, "sin": sin, "q_norm": qn, "k_norm": kn,
                "out": out.float(), "k_cache_after": kc_ref}, os.path.join(HERE, "ref_paged_attention.pt"))

    # ---- MLP (gate/up -> silu*up -> down + residual) --------------------
    # tests/runtime_python/test_mode/test_qwen3_mlp_testmode.py:145-148 is inline code, not a
    # function; the four statements are evaluated here through the same torch calls.
    g = torch.Generator().manual_seed(3)
    B, Hd, I = 8, 256, 128
    w_gate = (torch.randn(I, Hd, generator=g) * 0.01).to(bf16)
    w_up = (torch.randn(I, Hd, generator=g) * 0.01).to(bf16)
    w_down = (torch.randn(Hd, I, generator=g) * 0.01).to(bf16)
    inp = torch.randn(B, Hd, generator=g).to(bf16)
    res = torch.randn(B, Hd, generator=g).to(bf16)
    src = open(os.path.join(T, "test_mode", "test_qwen3_mlp_testmode.py")).read().splitlines()
    block = "\n".join(l.strip() for l in src[144:148])
    assert "ref_gate" in block and "ref_out" in block, block
    env = dict(torch=torch, input_act=inp, w_gate=w_gate, w_up=w_up, w_down=w_down,
               residual=res, dtype=bf16)
    exec(block, env)
    torch.save({"x": inp, "w_gate": w_gate, "w_up": w_up, "w_down": w_down, "residual": res,
                "out": env["ref_out"]}, os.path.join(HERE, "ref_mlp.pt"))

    # ---- allreduce = sum over ranks -----------------------------------
    parts = []
    for r in range(4):
        gg = torch.Generator().manual_seed(1234 + r)   # test_allreduce.py:99 seeds 1234 + rank
        parts.append(torch.randn(4, 512, generator=gg).to(bf16))
    torch.save({"parts": parts, "out_f32": torch.stack([p.float() for p in parts]).sum(0)},
               os.path.join(HERE, "ref_allreduce.pt"))

    # ---- FP8 quantise / dequantise / block-scaled linear ---------------
    # the reference's helper module is plain torch: import it as it is
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "ref_fp8_layout", os.path.join(T, "blackwell", "common", "sm100_fp8_scale_layout.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    g = torch.Generator().manual_seed(1234)          # seed of test_linear_1d2d_fp8.py:22
    xf = torch.randn(3, 512, generator=g).to(bf16)
    xf[1, :128] *= 37.0                               # a group with a large amax
    xf[2, 128:256] = 0                                # an all-zero group
    wf = torch.randn(24, 512, generator=g).to(bf16)
    xq, xs = ref.quantize_to_fp8_packed_ue8m0(xf)
    wq, ws = ref.quantize_to_fp8_packed_ue8m0(wf)
    x_ref, w_ref = ref.dequant_from_packed_ue8m0(xq, xs), ref.dequant_from_packed_ue8m0(wq, ws)
    resid = torch.randn(3, 24, generator=g).to(bf16)
    out = (torch.matmul(x_ref, w_ref.T) + resid.float()).to(bf16)     # test_linear_1d2d_fp8.py:67-71
    torch.save({"x": xf, "w": wf, "xq": xq.view(torch.uint8), "xs": xs.to(torch.int64), "wq": wq.view(torch.uint8),
                "ws": ws.to(torch.int64), "x_deq": x_ref, "residual": resid, "out": out},
               os.path.join(HERE, "ref_fp8.pt"))

    # ---- mixture of experts: routing, FP8 grouped GEMM ----------------------
    B = 5
    consts = dict(NUM_EXPERTS=64, NUM_EXPERTS_PER_TOK=4, NUM_GROUPS=8, TOPK_GROUP=3, ROUTED_SCALING_FACTOR=2.5,
                  EXPERTS_PER_GROUP=8)
    ns = load_functions(os.path.join(T, "blackwell", "sm100_moe_sigmoid", "test_gate_topk_sigmoid.py"),
                        ["reference_sigmoid_routing"], consts, on_cpu=True)
    g = torch.Generator().manual_seed(42)             # SEED of test_gate_topk_sigmoid.py:19
    logits = torch.randn(B, 64, generator=g).to(bf16)
    rbias = torch.randn(64, generator=g) * 0.1
    r_w, r_idx, r_act = ns["reference_sigmoid_routing"](logits, rbias, B)
    moe = {"logits": logits, "bias": rbias, "route_consts": consts, "weights": r_w, "routing": r_idx,
           "expert_active": r_act}
    # grouped GEMM on a reduced DeepSeek shape: 6 experts, top-2, K 256, 2I = 48, hidden 256, I 128
    gconst = dict(BATCH_SIZE=4, OUTPUT_SIZE=48, K=256, NUM_EXPERTS=6, NUM_TOPK=2, W2_OUTPUT_SIZE=256,
                  W2_REDUCTION_SIZE=128)
    ns = load_functions(os.path.join(T, "blackwell", "sm100_fp8_moe", "test_fp8_moe_gemm.py"),
                        ["quantize_to_fp8", "dequantize_fp8", "float32_to_ue8m0_approx", "reference_moe_w13",
                         "reference_moe_w2"], gconst, on_cpu=True)
    g = torch.Generator().manual_seed(7)
    token_to_experts = {0: [3, 1], 1: [0, 5], 2: [1, 4], 3: [5, 3]}
    routing = torch.zeros(6, 4, dtype=torch.int32)
    for tok, ex in token_to_experts.items():
        for slot, e in enumerate(ex):
            routing[e, tok] = slot + 1
    x13 = torch.randn(4, 256, generator=g).to(bf16)
    x13q, x13s = ns["quantize_to_fp8"](x13.float())
    w13 = (0.05 * torch.randn(6, 48, 256, generator=g)).to(bf16)
    w13q, w13s = ns["quantize_to_fp8"](w13.float())
    out13 = ns["reference_moe_w13"](x13q, x13s, w13q, w13s, 4, token_to_experts)
    x2 = torch.randn(4, 2, 128, generator=g).to(bf16)
    x2q, x2s = ns["quantize_to_fp8"](x2.float())
    w2 = (0.05 * torch.randn(6, 256, 128, generator=g)).to(bf16)
    w2q, w2s = ns["quantize_to_fp8"](w2.float())
    out2 = ns["reference_moe_w2"](x2q, x2s, w2q, w2s, 4, token_to_experts)
    moe.update({"g_routing": routing, "x13": x13, "x13q": x13q.view(torch.uint8), "x13s": x13s, "w13q": w13q.view(torch.uint8),
                "w13s": w13s, "out13": out13, "x2": x2, "x2q": x2q.view(torch.uint8), "x2s": x2s,
                "w2q": w2q.view(torch.uint8), "w2s": w2s, "out2": out2})
    torch.save(moe, os.path.join(HERE, "ref_moe.pt"))

    # ---- MLA multi-token decode ----------------------------------------------
    ns = load_functions(os.path.join(T, "blackwell", "sm100_mla", "test_mla_mtp.py"), ["pytorch_mla_ref"],
                        dict(D_V=512, D_K=576, NUM_HEADS=16))
    g = torch.Generator().manual_seed(42)             # torch.manual_seed(42) of test_mla_mtp.py:82
    mla = {}
    for q_len, kv_len in ((1, 100), (3, 45)):
        Q = (torch.randn(1, q_len, 16, 576, generator=g) * 0.1).to(bf16)
        KV = (torch.randn(1, kv_len, 576, generator=g) * 0.1).to(bf16)
        mla[f"q{q_len}"] = {"Q": Q, "KV": KV, "kv_len": kv_len, "scale": 0.135234,
                            "out": ns["pytorch_mla_ref"](Q, KV, 0.135234, kv_len, q_len)}
    torch.save(mla, os.path.join(HERE, "ref_mla.pt"))

    # ---- HF Qwen3 tiny -------------------------------------------------
    from transformers import Qwen3Config as HFConfig
    from transformers.models.qwen3.modeling_qwen3 import Qwen3ForCausalLM
    from oracle.qwen3_decoder import Qwen3Config, make_weights
    cfg = Qwen3Config.tiny()
    hf_cfg = HFConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                      intermediate_size=cfg.intermediate_size, num_hidden_layers=cfg.num_layers,
                      num_attention_heads=cfg.num_q_heads, num_key_value_heads=cfg.num_kv_heads,
                      head_dim=cfg.head_dim, max_position_embeddings=cfg.max_position,
                      rms_norm_eps=cfg.rms_eps, rope_theta=cfg.rope_theta, tie_word_embeddings=False,
                      attention_bias=False, use_sliding_window=False)
    hf_cfg.rope_parameters = {"rope_type": "default", "rope_theta": cfg.rope_theta}
    model = Qwen3ForCausalLM(hf_cfg).to(bf16).eval()
    weights = make_weights(cfg, seed=1001)
    missing, unexpected = model.load_state_dict(weights, strict=False)
    assert not unexpected, unexpected
    assert all("rotary" in m or "inv_freq" in m for m in missing), missing
    g = torch.Generator().manual_seed(2001)
    ids = torch.randint(0, cfg.vocab_size, (1, 24), generator=g)
    with torch.no_grad():
        logits = model(input_ids=ids).logits[0]
    torch.save({"seed": 1001, "ids": ids[0], "logits": logits.float()},
               os.path.join(HERE, "qwen3_tiny_hf.pt"))
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".pt"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of the mirage-project/mirage checkout>")
    main(sys.argv[1])
