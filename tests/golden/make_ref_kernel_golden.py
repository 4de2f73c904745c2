"""Writes tests/golden/ref_kernel_outputs.pt: outputs of the REFERENCE'S OWN compiled sm100 kernels on seeded inputs.

    python baseline/build_ref_kernels.py <reference checkout>      # once, where the reference sources are
    python tests/golden/make_ref_kernel_golden.py <output.pt>       # on a B200

The two kernels are the ones `bench.py --impl ref_kernel` times: the FP8 expert GEMM of the DeepSeek-V3 W13 shape
(tests/runtime_python/blackwell/sm100_fp8_moe/runtime_kernel_wrapper.cu, entry `fp8_moe_gemm_2d`, grid 8 x 16) and the
16-head absorbed-MLA decode + merge (mla_mtp_decode_tp8_sm100.cuh behind baseline/ref_mla_tp8_ext.cu).  The inputs are
too large to commit (7.5 GB of expert weights) and are regenerated from their seeds by `bench.moe_w13_inputs` /
`bench.mla_dense_inputs` (torch's counter-based CUDA generator); the fixture stores the kernels' outputs, the small
routing tensors, and checksums of the inputs so that a test can tell a generator that drifted from a kernel that did."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import bench  # noqa: E402
from gpu_util import input_checksums  # noqa: E402


QUANTIZE_CASES = [(1, 4096, 11), (8, 7168, 12), (64, 4096, 13), (5, 2048, 14), (3, 768, 15)]
# (the reference's stand-alone routing wrapper launches one CTA that routes one token per warp: 8 tokens at most)
ROUTING_CASES = [(1, 21), (8, 22), (4, 23), (7, 24)]


def quantize_case_input(B, H, seed):
    """bf16 rows with a spread of magnitudes per 128-group, one all-zero group and one group holding the bf16 maximum."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, H, generator=g) * torch.exp(torch.randn(B, H // 128, generator=g) * 2.0).repeat_interleave(128, dim=1)
    x[0, :128] = 0.0
    if B > 1:
        x[1, 128:256] = 3.0e38
    return x.to(torch.bfloat16)


def routing_case_input(B, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(B, 256, generator=g, dtype=torch.float32).to(torch.bfloat16)
    bias = torch.randn(256, generator=g, dtype=torch.float32) * 0.1
    return logits, bias


# (cached positions, new tokens, page holding the request, seed)
ATTENTION_CASES = [(8, 4, 0, 31), (300, 1, 1, 32), (496, 8, 1, 33), (0, 5, 0, 34), (63, 2, 1, 35)]


def attention_case_input(prefix, n_new, seed):
    """qkv rows of the new tokens, a two-page cache [2, 4096, 128] whose first `prefix` rows of both pages are filled,
    norm weights near 1 and random rotary tables [513, 128] (as the reference's own test draws them)."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    kc = torch.zeros(2, 4096, 128)
    vc = torch.zeros(2, 4096, 128)
    kc[:, :prefix] = r(2, prefix, 128)
    vc[:, :prefix] = r(2, prefix, 128)
    bf = torch.bfloat16
    return {"qkv": r(n_new, 6 * 128).to(bf), "k_cache": kc.to(bf), "v_cache": vc.to(bf),
            "q_norm": (1.0 + 0.1 * r(128)).to(bf), "k_norm": (1.0 + 0.1 * r(128)).to(bf),
            "cos": r(513, 128).to(bf), "sin": r(513, 128).to(bf)}


def main(path):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    fixture = {}
    rk = bench.load_ref_extension("runtime_kernel_fp8_moe")
    assert rk is not None, "baseline/_ref/runtime_kernel_fp8_moe is not built"
    t = bench.moe_w13_inputs(dev)
    out = torch.zeros(t["B"], t["topk"], t["N"], dtype=torch.bfloat16, device=dev)
    rk.fp8_moe_gemm_2d(t["xq"], t["xs"], t["w"], t["ws"], t["routing"], t["mask"], out, 8, 16)
    torch.cuda.synchronize()
    fixture["moe_w13"] = {"out": out.cpu(), "routing": t["routing"].cpu(), "mask": t["mask"].cpu(),
                          "checksums": input_checksums(t, ("w", "ws", "xq", "xs"))}
    del t, out
    torch.cuda.empty_cache()
    mla = bench.load_ref_extension("ref_mla_tp8")
    assert mla is not None, "baseline/_ref/ref_mla_tp8 is not built"
    t = bench.mla_dense_inputs(dev)
    qpad = torch.zeros(t["B"], 2, 16, 576, dtype=torch.bfloat16, device=dev)
    qpad[:, 0] = t["q"][:, 0]
    out = torch.zeros(t["B"], 2, 16, 512, dtype=torch.bfloat16, device=dev)
    mla.init(qpad, t["kv"], 1, t["scale"])
    mla.run(out)
    torch.cuda.synchronize()
    fixture["mla_dense"] = {"out": out[:, 0].reshape(t["B"], 16 * 512).cpu(), "scale": t["scale"],
                            "checksums": input_checksums(t, ("q", "kv"))}
    del t, out, qpad
    torch.cuda.empty_cache()

    # per-token x 128 quantisation to e4m3 + packed UE8M0 scales: inputs small enough to regenerate on the CPU generator
    qz = bench.load_ref_extension("runtime_kernel_blackwell_quantize_fp8")
    if qz is not None:
        cases = {}
        for (B, H, seed) in QUANTIZE_CASES:
            x = quantize_case_input(B, H, seed).to(dev)
            q = torch.zeros(B, H, dtype=torch.float8_e4m3fn, device=dev)
            packed = (H // 128 + 3) // 4
            sc = torch.zeros(packed * ((B + 3) // 4 * 4), dtype=torch.int32, device=dev)
            sc_view = torch.as_strided(sc, (B, packed), (1, (B + 3) // 4 * 4))     # the column-major form the kernels share
            qz.quantize_fp8_sm100(x, q, sc_view, 128)
            torch.cuda.synchronize()
            cases[(B, H, seed)] = {"q": q.view(torch.uint8).cpu(), "scale_words": sc.view(packed, -1)[:, :B].cpu()}
        fixture["quantize_fp8"] = cases

    # grouped sigmoid top-k routing (256 experts, 8 groups, top-4 groups, top-8 experts, scaling 2.5) and softmax top-k
    rt = bench.load_ref_extension("runtime_kernel_moe_sigmoid")
    if rt is not None:
        cases = {}
        for (B, seed) in ROUTING_CASES:
            logits, bias = routing_case_input(B, seed)
            w = torch.zeros(B, 8, dtype=torch.float32, device=dev)
            idx = torch.zeros(256, B, dtype=torch.int32, device=dev)
            act = torch.zeros(257, dtype=torch.int32, device=dev)
            rt.topk_sigmoid_sm100(logits.to(dev).clone(), bias.to(dev), w, idx, act, 2.5, 8, 4)
            torch.cuda.synchronize()
            w2 = torch.zeros(B, 8, dtype=torch.float32, device=dev)
            idx2 = torch.zeros(256, B, dtype=torch.int32, device=dev)
            act2 = torch.zeros(257, dtype=torch.int32, device=dev)
            rt.topk_softmax_sm100(logits.to(dev).clone(), w2, idx2, act2)
            torch.cuda.synchronize()
            cases[(B, seed)] = {"sigmoid": (w.cpu(), idx.cpu(), act.cpu()), "softmax": (w2.cpu(), idx2.cpu(), act2.cpu())}
        fixture["routing"] = cases

    # fused q/k RMSNorm + RoPE + append + causal attention of one request (4 query heads, 1 kv head, head_dim 128); the
    # wrapper is compiled for pages of 4096 rows and sequences of at most 512 positions, 8 new tokens at most
    rk_generic = bench.load_ref_extension("runtime_kernel")
    if rk_generic is not None:
        cases = {}
        for case in ATTENTION_CASES:
            prefix, n_new, page, seed = case
            t = attention_case_input(prefix, n_new, seed)
            kc, vc = t["k_cache"].to(dev), t["v_cache"].to(dev)
            out = torch.zeros(n_new * 4, 128, dtype=torch.bfloat16, device=dev)
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
            rk_generic.multitoken_paged_attention(
                t["qkv"].to(dev), kc, vc, out, i32([0, n_new]), i32([0, 1]), i32([page, 1 - page]), i32([prefix + n_new]), 0,
                True, True, t["q_norm"].to(dev), t["k_norm"].to(dev), t["cos"].to(dev), t["sin"].to(dev), 1e-6, 1e-6)
            torch.cuda.synchronize()
            cases[case] = {"out": out.cpu(), "k_rows": kc[page, prefix:prefix + n_new].cpu(),
                           "v_rows": vc[page, prefix:prefix + n_new].cpu()}
        fixture["paged_attention"] = cases

    torch.save(fixture, path)
    print("wrote", path, sorted(fixture))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
