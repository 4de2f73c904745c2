"""Benchmark: Qwen3-8B-shaped bf16 greedy decode through the megakernel.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--context C] [--impl reference]

One "step" is one decode iteration of the whole model (one megakernel launch) over a batch of B
requests, i.e. B tokens.  At batch 1 the metric is ms/token; at batch > 1 it is tok/s.  Weights are
random-init, the context is random token ids fed through the same graph before timing starts
(data = synthetic).  For N > 1 run under torchrun (one rank per GPU, tensor parallel); rank 0 prints
one JSON line.

The timed region is K launches between two CUDA events on the launch stream, after W warm-up steps, with
a barrier + synchronize on both sides and the maximum over ranks.  The 15 GB of weights are far larger
than L2, so every step streams them from HBM again; no extra flush is needed.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

QWEN3_8B = dict(num_layers=36, hidden_size=4096, num_q_heads=32, num_kv_heads=8, head_dim=128,
                intermediate_size=12288, vocab_size=151936)


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs (read-only query)."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                self.rows.append([c.strip() for c in out.strip().split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=10)

    def summary(self):
        sm = sorted(int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def make_gpu_weights(shape, seed, device):
    """Random-init weights generated on the device (N(0,0.02) linears, 1 + N(0,0.02) norms)."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    lin = lambda n, k: (torch.randn(n, k, generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    norm = lambda n: (1 + torch.randn(n, generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    h, d = shape["hidden_size"], shape["head_dim"]
    w = {"model.embed_tokens.weight": lin(shape["vocab_size"], h)}
    for i in range(shape["num_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = norm(h)
        w[p + "self_attn.q_proj.weight"] = lin(shape["num_q_heads"] * d, h)
        w[p + "self_attn.k_proj.weight"] = lin(shape["num_kv_heads"] * d, h)
        w[p + "self_attn.v_proj.weight"] = lin(shape["num_kv_heads"] * d, h)
        w[p + "self_attn.q_norm.weight"] = norm(d)
        w[p + "self_attn.k_norm.weight"] = norm(d)
        w[p + "self_attn.o_proj.weight"] = lin(h, shape["num_q_heads"] * d)
        w[p + "post_attention_layernorm.weight"] = norm(h)
        w[p + "mlp.gate_proj.weight"] = lin(shape["intermediate_size"], h)
        w[p + "mlp.up_proj.weight"] = lin(shape["intermediate_size"], h)
        w[p + "mlp.down_proj.weight"] = lin(h, shape["intermediate_size"])
    w["model.norm.weight"] = norm(h)
    w["lm_head.weight"] = lin(shape["vocab_size"], h)
    return w


FP8_PROJECTIONS = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                   "self_attn.o_proj.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight")


def make_fp8_checkpoint(weights, shape, seed, device):
    """The FP8 form of the random-init decoder: every projection as e4m3 values with float32 128 x 128 block scales
    drawn log-uniformly from [1e-3, 1e-1]; value x scale reproduces the N(0, 0.02) bf16 weight to e4m3 precision.
    Generated on the device, layer by layer."""
    import math
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    lo, hi = math.log(1e-3), math.log(1e-1)
    out = {}
    for i in range(shape["num_layers"]):
        for k in FP8_PROJECTIONS:
            name = f"model.layers.{i}.{k}"
            w = weights[name]
            n, kk = w.shape
            scale = torch.exp(lo + torch.rand((n + 127) // 128, (kk + 127) // 128, generator=g, device=device) * (hi - lo))
            per_elem = scale.repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :kk]
            out[name] = ((w.float() / per_elem).clamp(-448, 448).to(torch.float8_e4m3fn), scale.float())
    return out


def cpu_reference_ms_per_token(shape, context, batch, steps=2, warmup=1):
    """The CPU oracle (a port of the reference's PyTorch forward) on the host cores.

    Every timed step is a real forward of the full-depth graph (all `num_layers` layers, lm_head, argmax) at the
    benchmark's context length.  What is bounded is memory and set-up time: one layer's random weights are drawn
    and shared by all layers (same shapes, same arithmetic, same bytes streamed per layer -- a 386 MB layer does not
    stay in the host caches), and the KV cache is filled with random rows instead of running a CPU prefill.
    Returns (ms per token, description, cores, ms per step)."""
    import torch
    from oracle.qwen3_decoder import Qwen3Config, Qwen3Oracle, make_weights
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    one = Qwen3Config(num_layers=1, hidden_size=shape["hidden_size"], num_q_heads=shape["num_q_heads"],
                      num_kv_heads=shape["num_kv_heads"], head_dim=shape["head_dim"],
                      intermediate_size=shape["intermediate_size"], vocab_size=shape["vocab_size"])
    w = make_weights(one, seed=1)
    layers = shape["num_layers"]
    for key in [k for k in w if k.startswith("model.layers.0.")]:
        for i in range(1, layers):
            w[key.replace("model.layers.0.", f"model.layers.{i}.")] = w[key]
    cfg = Qwen3Config(num_layers=layers, hidden_size=one.hidden_size, num_q_heads=one.num_q_heads,
                      num_kv_heads=one.num_kv_heads, head_dim=one.head_dim, intermediate_size=one.intermediate_size,
                      vocab_size=one.vocab_size)
    page = 64
    pages_per_req = (context + steps + warmup + page) // page
    orc = Qwen3Oracle(cfg, w, max_num_pages=pages_per_req * batch, page_size=page)
    g = torch.Generator().manual_seed(0)
    filler = torch.randn(orc.k_cache[0].shape, generator=g).to(torch.bfloat16)
    for kc in orc.k_cache + orc.v_cache:      # a random "prefilled" cache: same arithmetic, no CPU prefill
        kc.copy_(filler)
    ids = torch.randint(0, cfg.vocab_size, (batch,), generator=g)
    times = []
    for it in range(warmup + steps):
        reqs = [((b, b + 1), list(range(b * pages_per_req, (b + 1) * pages_per_req)), context + 1 + it)
                for b in range(batch)]
        t0 = time.perf_counter()
        logits = orc.forward_tokens(ids, reqs)
        ids = logits.float().argmax(-1)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    step_s = sum(times) / len(times)
    sample = (f"{steps} timed decode steps (after {warmup} warm-up) of the full {layers}-layer graph + lm_head at "
              f"context {context}, batch {batch}; one layer's random weights shared by all layers, random KV rows")
    return step_s * 1e3 / batch, sample, cores, step_s * 1e3


def run_reference(args):
    """`--impl reference`: the reference's CPU path for the same metric (the CPU oracle port; the reference's
    own megakernel cannot be built in this image and its PyTorch model needs its CUDA extension).  Each of the
    `--steps` timed steps is a real full-depth decode step on the host cores; the step count is capped so that
    the run ends within a few minutes, and the line reports the count that ran."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    shape = dict(QWEN3_8B, num_layers=args.layers)
    steps = max(1, min(args.steps, 12))
    warm = max(1, min(args.warmup, 2))
    ms_tok, sample, cores, ms_step = cpu_reference_ms_per_token(shape, args.context, args.batch, steps=steps, warmup=warm)
    bs1 = args.batch == 1
    value = ms_tok if bs1 else 1e3 / ms_tok
    unit = "ms/token" if bs1 else "tok/s"
    line = {"impl": "reference", "metric": metric_name(args.batch), "value": value, "unit": unit, "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": ms_step,
            "higher_is_better": not bs1, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(args),
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def metric_name(batch, fp8=False):
    model = "qwen3_8b_fp8" if fp8 else "qwen3_8b"
    return f"{model}_decode_ms_per_token_bs1" if batch == 1 else f"{model}_decode_tok_per_s_bs{batch}"


def workload_config(args):
    kind = "FP8 e4m3 projections (128x128 block scales), bf16 activations" if args.fp8 else "bf16"
    return {"workload": f"Qwen3-8B-shape decoder, 36 layers, {kind}, batch {args.batch}, context {args.context}, "
                        f"paged KV (page 64), greedy decode, TP={args.gpus}",
            "global_batch": args.batch, "context": args.context, "parallelism": f"tp{args.gpus}",
            "l2": "weights (%s) exceed L2; every step re-streams them from HBM" % ("8.4 GB" if args.fp8 else "15 GB")}


def moe_w13_inputs(dev, seed=3013):
    """Seeded inputs of the routed experts' first projection at the DeepSeek-V3 shape the reference's stand-alone
    expert-GEMM wrapper is compiled for (tests/runtime_python/blackwell/sm100_fp8_moe/runtime_kernel_wrapper.cu:43-53:
    16 tokens, 256 experts, top-8, N = 4096, K = 7168), in the layouts the reference's operator takes: e4m3 activations
    with float32 per-128 scales, e4m3 weights [E, N, K] with float32 row x 128 scales, routing [E, tokens] (slot + 1 or
    0), mask = activated expert ids followed at [E] by their count.  Generated on the device (cuda generator)."""
    import torch
    E, topk, N, K, B = 256, 8, 4096, 7168, 16
    g = torch.Generator(device=dev).manual_seed(seed)
    w = torch.empty(E, N, K, dtype=torch.float8_e4m3fn, device=dev)
    for e in range(E):
        w[e] = (torch.randn(N, K, generator=g, device=dev) * 0.5).to(torch.float8_e4m3fn)
    ws = torch.rand(E, N, K // 128, generator=g, device=dev) * 0.01 + 0.001
    x = torch.randn(B, K, generator=g, device=dev)
    blocks = x.reshape(B, K // 128, 128)
    xs = (blocks.abs().amax(dim=-1) / 448.0).clamp(min=1e-12).float()
    xq = (blocks / xs.unsqueeze(-1)).reshape(B, K).to(torch.float8_e4m3fn)
    cg = torch.Generator().manual_seed(seed + 1)
    routing = torch.zeros(E, B, dtype=torch.int32)
    for i in range(B):
        for slot, e in enumerate(torch.randperm(E, generator=cg)[:topk].tolist()):
            routing[e, i] = slot + 1
    active = [e for e in range(E) if bool(routing[e].any())]
    mask = torch.zeros(E + 1, dtype=torch.int32)
    mask[:len(active)] = torch.tensor(active, dtype=torch.int32)
    mask[E] = len(active)
    nbytes = len(active) * (N * K + N * (K // 128) * 4)
    return dict(E=E, topk=topk, N=N, K=K, B=B, w=w, ws=ws.contiguous(), xq=xq.contiguous(), xs=xs.contiguous(),
                routing=routing.to(dev), mask=mask.to(dev), n_active=len(active), bytes=nbytes)


def build_moe_w13_graph(mi, t):
    """The repo's side of the moe_w13 workload: a test-mode graph holding the one expert-projection layer."""
    params = mi.PersistentKernel.get_default_init_parameters()
    params.update(test_mode=True, num_workers=0, max_num_batched_tokens=t["B"], max_num_batched_requests=t["B"])
    pk = mi.PersistentKernel(**params)
    out = pk.new_tensor(dims=(t["B"], t["topk"], t["N"]), dtype=mi.bfloat16, name="mid", io_category="cuda_tensor")
    pk.moe_w13_fp8_layer(input_fp8=pk.attach_input(t["xq"], "xq"), input_scale=pk.attach_input(t["xs"], "xs"),
                         weight_fp8=pk.attach_input(t["w"], "w13"), weight_scale=pk.attach_input(t["ws"], "w13s"),
                         moe_routing_indices=pk.attach_input(t["routing"], "idx"),
                         moe_mask=pk.attach_input(t["mask"], "mask"), output=out, grid_dim=(32, 1, 1),
                         block_dim=(128, 1, 1))
    pk.compile()
    return pk, out


def mla_dense_inputs(dev, requests=32, kv_len=4096, seed=3014):
    """Seeded inputs of absorbed-MLA decode at the tensor-parallel-8 shape: 16 local heads, one query token per request,
    a dense [requests, kv_len, 576] bf16 latent cache (the layout the reference's stand-alone kernel reads)."""
    import torch
    g = torch.Generator(device=dev).manual_seed(seed)
    q = (torch.randn(requests, 1, 16, 576, generator=g, device=dev) * 0.3).to(torch.bfloat16)
    kv = (torch.randn(requests, kv_len, 576, generator=g, device=dev) * 0.3).to(torch.bfloat16)
    return dict(B=requests, kv_len=kv_len, q=q, kv=kv, scale=576 ** -0.5, bytes=requests * kv_len * 576 * 2)


def build_mla_dense_graph(mi, t):
    """The repo's side of the mla_dense workload: decode + merge tasks over the dense cache, as a test-mode graph."""
    import torch
    B, H, kv_len = t["B"], 16, t["kv_len"]
    S = (kv_len + 127) // 128
    params = mi.PersistentKernel.get_default_init_parameters()
    params.update(test_mode=True, num_workers=0, max_num_batched_tokens=B, max_num_batched_requests=B)
    pk = mi.PersistentKernel(**params)
    out = torch.zeros(B, H * 512, dtype=torch.bfloat16, device=t["q"].device)
    po = pk.new_tensor(dims=(B * H * S, 512), dtype=mi.bfloat16, name="po", io_category="cuda_tensor")
    lse = pk.new_tensor(dims=(B * H * S,), dtype=mi.float32, name="lse", io_category="cuda_tensor")
    pk.mla_mtp_decode_layer(pk.attach_input(t["q"].reshape(B, H * 576), "q"),
                            pk.attach_input(t["kv"].reshape(B * kv_len, 576), "kv"), po, lse, 1, kv_len,
                            sm_scale=t["scale"])
    pk.mla_mtp_reduce_layer(po, lse, pk.attach_input(out, "out"), 1, kv_len)
    pk.compile()
    return pk, out


def load_ref_extension(name):
    import importlib.util
    so = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", name, name + ".so")
    if not os.path.exists(so):
        return None
    import torch  # noqa: F401  (the extension links against torch's libraries)
    spec = importlib.util.spec_from_file_location(name, so)
    try:
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    except (ImportError, OSError) as e:      # e.g. no CUDA driver on this machine
        print(f"bench.py: {so} cannot be loaded here: {e}", file=sys.stderr)
        return None
    return mod


def time_launches(fn, K, Wm):
    import torch
    for _ in range(Wm):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(K):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return sum(times) / len(times) * 1e3


def run_ref_kernel_mla(args):
    """`--impl ref_kernel --workload mla_dense`: the reference's 16-head absorbed-MLA decode + merge device functions
    (baseline/ref_mla_tp8_ext.cu around mla_mtp_decode_tp8_sm100.cuh) on the tensors of `mla_dense_inputs`; the same
    tensors then go through this repo's tasks once and the largest output difference is reported."""
    import torch
    rk = load_ref_extension("ref_mla_tp8")
    if rk is None:
        print(json.dumps({"impl": "ref_kernel", "unavailable": "baseline/_ref/ref_mla_tp8 not built or not loadable here "
                          "(python baseline/build_ref_kernels.py <reference checkout>)"}))
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    t = mla_dense_inputs(dev, kv_len=args.context if args.context != 1024 else 4096)
    B = t["B"]
    qpad = torch.zeros(B, 2, 16, 576, dtype=torch.bfloat16, device=dev)      # the kernel wants an even query count
    qpad[:, 0] = t["q"][:, 0]
    out = torch.zeros(B, 2, 16, 512, dtype=torch.bfloat16, device=dev)
    rk.init(qpad, t["kv"], 1, t["scale"])
    K, Wm = args.steps if args.steps != 128 else 20, max(args.warmup, 3)
    with ClockSampler(0) as clocks:
        us = time_launches(lambda: rk.run(out), K, Wm)
    import mirage_b200 as mi
    pk, mine = build_mla_dense_graph(mi, t)
    pk.run_test_mode()
    torch.cuda.synchronize()
    assert pk.status().error == 0
    ref = out[:, 0].reshape(B, 16 * 512).float()
    diff = (mine.float() - ref).abs().max().item()
    peak, peak_kind = measured_peak_gbs()
    achieved = t["bytes"] / (us * 1e-6) / 1e9
    print(json.dumps({
        "impl": "ref_kernel", "metric": "mla_dense_us_b%d_ctx%d" % (B, t["kv_len"]), "value": us, "unit": "us/launch",
        "n_gpus": 1, "steps": K, "warmup": Wm, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "reference mla_mtp_tp8_main + mla_mtp_tp8_reduce, %d requests x %d cached positions, 16 "
                               "local heads, 1 query token (padded to 2), dense cache" % (B, t["kv_len"]),
                   "l2": "cache rows per launch exceed L2"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": peak_kind, "kernel": "mla_mtp_tp8_main + mla_mtp_tp8_reduce",
                     "algorithmic_bytes_per_launch": t["bytes"]},
        "gpu_launches": 2 * K, "clocks": clocks.summary(),
        "repo_vs_ref_kernel": {"max_abs_diff": diff, "max_abs_ref": ref.abs().max().item()}}))


def run_ref_kernel(args):
    """`--impl ref_kernel --workload moe_w13`: the reference's own stand-alone sm100 FP8 expert GEMM (built unmodified
    by baseline/build_ref_kernels.py into baseline/_ref/) on the tensors `moe_w13_inputs` makes, timed per launch with
    CUDA events over the grids the reference's bench_fp8_moe_gemm.py tries; the best grid is the line's value.  The same
    tensors then go through this repo's graph once, and the line carries the largest difference between the two
    outputs over the (token, slot) rows that were routed.  One GPU only."""
    import torch
    if args.workload == "mla_dense":
        return run_ref_kernel_mla(args)
    if args.workload != "moe_w13":
        print(json.dumps({"impl": "ref_kernel", "unavailable": "only --workload moe_w13 and mla_dense have a reference "
                          "kernel built for a full-size shape"}))
        return
    rk = load_ref_extension("runtime_kernel_fp8_moe")
    if rk is None:
        print(json.dumps({"impl": "ref_kernel", "unavailable": "baseline/_ref/runtime_kernel_fp8_moe not built or not loadable here "
                          "(python baseline/build_ref_kernels.py <reference checkout>)"}))
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    t = moe_w13_inputs(dev)
    out = torch.zeros(t["B"], t["topk"], t["N"], dtype=torch.bfloat16, device=dev)
    K, Wm = args.steps if args.steps != 128 else 20, max(args.warmup, 3)
    grids, best = {}, None
    with ClockSampler(0) as clocks:
        for es, ns in ((4, 32), (8, 16), (16, 8), (32, 4)):
            rk.fp8_moe_gemm_bench_setup(t["w"], es, ns)
            launch = lambda: rk.fp8_moe_gemm_bench_launch(t["xq"], t["xs"], t["ws"], t["routing"], t["mask"], out)
            for _ in range(Wm):
                launch()
            torch.cuda.synchronize()
            times = []
            for _ in range(K):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                launch()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            rk.fp8_moe_gemm_bench_cleanup()
            grids["%dx%d" % (es, ns)] = sum(times) / len(times) * 1e3
            if best is None or grids["%dx%d" % (es, ns)] < grids[best]:
                best = "%dx%d" % (es, ns)
    es, ns = (int(v) for v in best.split("x"))
    out.zero_()
    rk.fp8_moe_gemm_2d(t["xq"], t["xs"], t["w"], t["ws"], t["routing"], t["mask"], out, es, ns)
    import mirage_b200 as mi
    pk, mine = build_moe_w13_graph(mi, t)
    pk.run_test_mode()
    torch.cuda.synchronize()
    assert pk.status().error == 0
    got = pk.tensor_as_torch(mine).float()
    routed = (t["routing"].t() > 0)                               # [B, E]
    slots = torch.zeros(t["B"], t["topk"], dtype=torch.bool, device=dev)
    for i in range(t["B"]):
        slots[i, (t["routing"][:, i][routed[i]] - 1).long()] = True
    diff = ((got - out.float()).abs() * slots.unsqueeze(-1)).max().item()
    scale = (out.float().abs() * slots.unsqueeze(-1)).max().item()
    us = grids[best]
    peak, peak_kind = measured_peak_gbs()
    achieved = t["bytes"] / (us * 1e-6) / 1e9
    print(json.dumps({
        "impl": "ref_kernel", "metric": "moe_w13_us_b16", "value": us, "unit": "us/launch", "n_gpus": 1, "steps": K,
        "warmup": Wm, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "e4m3", "data": "synthetic",
        "config": {"workload": "reference fp8_moe_group_gemm_sm100 stand-alone wrapper, %d of 256 experts active, top-8, "
                               "N 4096, K 7168, 16 tokens; grid %s (best of %s)" % (t["n_active"], best, sorted(grids)),
                   "l2": "bytes per launch exceed L2; each launch re-streams them", "grids_us": grids},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": peak_kind, "kernel": "dsv3_fp8_moe_2d_kernel",
                     "algorithmic_bytes_per_launch": t["bytes"]},
        "gpu_launches": K, "clocks": clocks.summary(),
        "repo_vs_ref_kernel": {"max_abs_diff": diff, "max_abs_ref": scale}}))


def run_block_workload(args):
    """One block of FP8 / MoE / MLA tasks as a test-mode graph, timed per launch with CUDA events.  The bytes a
    launch must read exceed L2 in every case, so consecutive launches re-stream them from HBM."""
    import torch
    import mirage_b200 as mi
    from mirage_b200.builders import fp8_prep

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(3005)
    B = args.batch if args.batch > 1 else {"fp8_layer": 64, "moe_block": 32, "mla_decode": 32, "moe_w13": 16, "mla_dense": 32}[args.workload]
    params = mi.PersistentKernel.get_default_init_parameters()
    params.update(test_mode=True, num_workers=0, max_num_batched_tokens=B, max_num_batched_requests=B)
    keep = []

    def rnd(*shape, scale=1.0, dtype=torch.bfloat16):
        t = (torch.randn(*shape, generator=g) * scale).to(dtype).to(dev)
        keep.append(t)
        return t

    def fp8_weight(n, k):      # e4m3 weight with packed UE8M0 row scales, quantised in slabs on the device
        q = torch.empty(n, k, dtype=torch.float8_e4m3fn, device=dev)
        sc = torch.empty(n, (k // 128 + 3) // 4, dtype=torch.int32, device=dev)
        for r in range(0, n, 4096):
            slab = (torch.randn(min(4096, n - r), k, generator=g) * 0.02).to(torch.bfloat16).to(dev)
            wq, packed, _ = fp8_prep.quantize_ue8m0(slab)
            q[r:r + wq.shape[0]] = wq
            sc[r:r + wq.shape[0]] = fp8_prep.packed_rows_contiguous(packed).view(torch.int32)
        keep.extend([q, sc])
        return q, sc.view(torch.uint32)

    if args.workload == "fp8_layer":
        # the four projections of one Qwen3-8B-shape layer with e4m3 weights, 64 tokens: quantise -> linear_fp8
        pk = mi.PersistentKernel(**params)
        nt = lambda dims, dt, name: pk.new_tensor(dims=dims, dtype=dt, name=name, io_category="cuda_tensor")
        H, I = 4096, 12288
        x = pk.attach_input(rnd(B, H), "x")
        bytes_alg = 0

        def fp8_linear(inp, k, n, name, residual=None):
            nonlocal bytes_alg
            q = nt((B, k), mi.float8_e4m3, name + "_q")
            s = nt(((k // 128 + 3) // 4, (B + 3) // 4 * 4), mi.uint32, name + "_s")
            wq, ws = fp8_weight(n, k)
            out = nt((B, n), mi.bfloat16, name + "_y")
            pk.quantize_fp8_layer(input=inp, output_fp8=q, output_scale=s, grid_dim=(B, 1, 1), block_dim=(128, 1, 1))
            kw = dict(input_fp8=q, input_scale=s, weight_fp8=pk.attach_input(wq, name + "_w"),
                      weight_scale=pk.attach_input(ws, name + "_ws"), output=out, grid_dim=(n // 128, 1, 1),
                      block_dim=(128, 1, 1))
            if residual is None:
                pk.linear_fp8_layer(**kw)
            else:
                pk.linear_fp8_with_residual_layer(residual=residual, **kw)
            bytes_alg += n * k
            return out

        qkv = fp8_linear(x, H, 6144, "qkv")
        o = fp8_linear(pk.attach_input(rnd(B, H), "attn"), H, H, "o", residual=x)
        gu = fp8_linear(o, H, 2 * I, "gate_up")
        act = nt((B, I), mi.bfloat16, "act")
        pk.silu_mul_layer(input=gu, output=act, grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
        fp8_linear(act, I, H, "down", residual=o)
        metric, unit_work = "fp8_layer_us_b%d" % B, "e4m3 weights of one Qwen3-8B-shape layer (192.9 MB), %d tokens" % B
    elif args.workload == "moe_block":
        # routed experts of a DeepSeek-V3-style layer: 256 experts, top-8, hidden 7168, expert width 2048
        E, topk, H, I = 256, 8, 7168, 2048
        pk = mi.PersistentKernel(**params)
        nt = lambda dims, dt, name: pk.new_tensor(dims=dims, dtype=dt, name=name, io_category="cuda_tensor")
        x = pk.attach_input(rnd(B, H), "x")
        logits = rnd(B, E)
        logits_src = logits.clone()
        bias = rnd(E, scale=0.1, dtype=torch.float32)
        w13 = torch.empty(E, 2 * I, H, dtype=torch.float8_e4m3fn, device=dev)
        w2 = torch.empty(E, H, I, dtype=torch.float8_e4m3fn, device=dev)
        for e in range(E):      # random e4m3 bit patterns with exponents in a narrow band (no NaN codes)
            w13[e] = (torch.randn(2 * I, H, generator=g) * 0.5).to(torch.float8_e4m3fn).to(dev)
            w2[e] = (torch.randn(H, I, generator=g) * 0.5).to(torch.float8_e4m3fn).to(dev)
        w13s = (torch.rand(E, 2 * I, H // 128, generator=g) * 0.01 + 0.001).to(dev)
        w2s = (torch.rand(E, H, I // 128, generator=g) * 0.01 + 0.001).to(dev)
        keep.extend([w13, w2, w13s, w2s, logits_src])
        t_w, t_idx, t_mask = nt((B, topk), mi.float32, "tw"), nt((E, B), mi.int32, "idx"), nt((E + 1,), mi.int32, "mask")
        xq, xs = nt((B, H), mi.float8_e4m3, "xq"), nt((B, H // 128), mi.float32, "xs")
        mid, act = nt((B, topk, 2 * I), mi.bfloat16, "mid"), nt((B, topk, I), mi.bfloat16, "act")
        aq, asc = nt((B, topk, I), mi.float8_e4m3, "aq"), nt((B, topk, I // 128), mi.float32, "as")
        down, y = nt((B, topk, H), mi.bfloat16, "down"), nt((B, H), mi.bfloat16, "y")
        pk.moe_topk_sigmoid_routing_layer(input=pk.attach_input(logits, "logits"), bias=pk.attach_input(bias, "bias"),
                                          output=(t_w, t_idx, t_mask), grid_dim=(1, 1, 1), block_dim=(256, 1, 1))
        pk.quantize_fp8_layer(input=x, output_fp8=xq, output_scale=xs, grid_dim=(B, 1, 1), block_dim=(128, 1, 1),
                              scale_ue8m0=False)
        pk.moe_w13_fp8_layer(input_fp8=xq, input_scale=xs, weight_fp8=pk.attach_input(w13, "w13"),
                             weight_scale=pk.attach_input(w13s, "w13s"), moe_routing_indices=t_idx, moe_mask=t_mask,
                             output=mid, grid_dim=(32, 1, 1), block_dim=(128, 1, 1))
        pk.moe_silu_mul_layer(input=mid, output=act, grid_dim=(B, topk, 1), block_dim=(128, 1, 1))
        pk.quantize_fp8_layer(input=act, output_fp8=aq, output_scale=asc, grid_dim=(B * topk, 1, 1), block_dim=(128, 1, 1),
                              scale_ue8m0=False)
        pk.moe_w2_fp8_layer(input_fp8=aq, input_scale=asc, weight_fp8=pk.attach_input(w2, "w2"),
                            weight_scale=pk.attach_input(w2s, "w2s"), moe_routing_indices=t_idx, moe_mask=t_mask,
                            output=down, grid_dim=(32, 1, 1), block_dim=(128, 1, 1))
        pk.moe_mul_sum_add_layer(input=down, weight=t_w, residual=x, output=y, grid_dim=(B, 1, 1), block_dim=(128, 1, 1))
        # bytes: the e4m3 panels (and float32 row scales) of the experts the routing task activates: their number is
        # read from the task's own output (last entry of the mask tensor) after the warm-up launches
        moe_mask_tensor = t_mask
        moe_bytes = lambda n_act: n_act * (2 * I * H + H * I) + n_act * 4 * (2 * I * (H // 128) + H * (I // 128))
        metric = "moe_block_us_b%d" % B
        unit_work = "%d of 256 experts active, top-8, hidden 7168, expert width 2048, " + "%d tokens" % B
    elif args.workload == "moe_w13":
        # the routed experts' first projection alone, at the shape and on the tensors the reference's stand-alone
        # kernel is timed on by `--impl ref_kernel`
        t = moe_w13_inputs(dev)
        B = t["B"]
        pk, _ = build_moe_w13_graph(mi, t)
        keep.append(t)
        bytes_alg = t["bytes"]
        metric = "moe_w13_us_b16"
        unit_work = "%d of 256 experts active, top-8, N 4096, K 7168, 16 tokens" % t["n_active"]
    elif args.workload == "mla_dense":
        # absorbed MLA decode + merge over a dense cache, on the tensors `--impl ref_kernel` gives the reference's kernel
        t = mla_dense_inputs(dev, kv_len=args.context if args.context != 1024 else 4096)
        B = t["B"]
        pk, _ = build_mla_dense_graph(mi, t)
        keep.append(t)
        bytes_alg = t["bytes"]
        metric = "mla_dense_us_b%d_ctx%d" % (B, t["kv_len"])
        unit_work = "%d requests x %d cached positions, 16 local heads, 1 query token, dense cache" % (B, t["kv_len"])
    else:
        # absorbed MLA decode at the tensor-parallel-8 shape: 16 local heads, 32 requests, context 4096
        Hh, ctx, page = 16, args.context if args.context != 1024 else 4096, 64
        per = (ctx + page - 1) // page
        npages = B * per
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        meta = {"qo_indptr_buffer": i32(list(range(B + 1))), "paged_kv_indptr_buffer": i32([per * i for i in range(B + 1)]),
                "paged_kv_indices_buffer": i32(torch.randperm(npages, generator=g).tolist()),
                "paged_kv_last_page_len_buffer": i32([(ctx - 1) % page + 1] * B)}
        params.update(max_num_pages=npages, page_size=page, max_seq_length=per * page, meta_tensors=meta)
        pk = mi.PersistentKernel(**params)
        nt = lambda dims, dt, name: pk.new_tensor(dims=dims, dtype=dt, name=name, io_category="cuda_tensor")
        S = (per * page + 127) // 128
        cache = rnd(npages, page, 576, scale=0.3)
        contiguous = nt((8, 576), mi.bfloat16, "contiguous_kv")
        po, lse = nt((B * Hh * S, 512), mi.bfloat16, "po"), nt((B * Hh * S,), mi.float32, "lse")
        out = nt((B, Hh * 512), mi.bfloat16, "attn_out")
        pk.mla_kv_gather_layer(c_latent_new=pk.attach_input(rnd(B, 512, scale=0.3), "lat"),
                               k_pe_new=pk.attach_input(rnd(B, 128, scale=0.3), "pe"), paged_cache=pk.attach_input(cache, "cache"),
                               contiguous_kv=contiguous, mla_params=(576, 512, page), grid_dim=(B, 1, 1), block_dim=(128, 1, 1))
        pk.mla_mtp_decode_layer(pk.attach_input(rnd(B, Hh * 576, scale=0.3), "q"), contiguous, po, lse, B, per * page)
        pk.mla_mtp_reduce_layer(po, lse, out, B, per * page)
        bytes_alg = B * ctx * 576 * 2
        metric = "mla_decode_us_b%d_ctx%d" % (B, ctx)
        unit_work = "latent cache rows of %d requests x %d positions (16 local heads), append + decode + merge" % (B, ctx)
    if args.workload not in ("moe_w13", "mla_dense"):
        pk.compile()
    K, Wm = args.steps if args.steps != 128 else 20, max(args.warmup, 3)

    def relaunch():
        if args.workload == "moe_block":
            logits.copy_(logits_src)        # the routing task zeroes its logits
        pk.run_test_mode()

    for _ in range(Wm):
        relaunch()
    torch.cuda.synchronize()
    if args.workload == "moe_block":
        n_act = int(pk.tensor_as_torch(moe_mask_tensor)[-1].item())
        bytes_alg, unit_work = moe_bytes(n_act), unit_work % n_act
    times = []
    with ClockSampler(0) as clocks:
        for _ in range(K):
            if args.workload == "moe_block":
                logits.copy_(logits_src)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            pk.step(1)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    assert pk.status().error == 0
    ms = sum(times) / len(times)
    peak, peak_kind = measured_peak_gbs()
    achieved = bytes_alg / (ms * 1e-3) / 1e9
    info = pk.graph_info()
    print(json.dumps({
        "metric": metric, "value": ms * 1e3, "unit": "us/launch", "n_gpus": 1, "steps": K, "warmup": Wm,
        "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "e4m3" if args.workload not in ("mla_decode", "mla_dense") else "bf16", "data": "synthetic",
        "config": {"workload": unit_work, "l2": "bytes per launch exceed L2; each launch re-streams them"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": peak_kind, "kernel": "mpk_megakernel<general>",
                     "algorithmic_bytes_per_launch": bytes_alg},
        "gpu_launches": K, "clocks": clocks.summary(), "tasks_per_launch": info["num_tasks"]}))


def synthetic_deepseek_state(shape, world, rank, dev, seed):
    """This rank's prepared DeepSeek-V3 tensors (the forms mirage_b200.builders.deepseek_v3.prepare_state produces),
    generated on the device: N(0, 0.02) weights quantised where the graph wants FP8, experts as random e4m3 with float32
    per-row scales in [1e-3, 1.1e-2]."""
    import torch
    from mirage_b200.builders import fp8_prep
    from mirage_b200.builders.deepseek_v3 import D_K, D_LATENT
    g = torch.Generator(device=dev).manual_seed(seed)
    s, st = shape, {}
    hl, per = s.num_heads // world, s.num_experts // world
    bf = lambda *d: (torch.randn(*d, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    norm = lambda n: (1 + torch.randn(n, generator=g, device=dev) * 0.02).to(torch.bfloat16)

    def fp8(key, n, k):
        q, packed, _ = fp8_prep.quantize_ue8m0(bf(n, k))
        st[key + ".weight"], st[key + ".scale"] = q, fp8_prep.packed_rows_contiguous(packed)

    def experts(key, n, k):
        w = torch.empty(per, n, k, dtype=torch.float8_e4m3fn, device=dev)
        for e in range(per):
            w[e] = (torch.randn(n, k, generator=g, device=dev) * 0.5).to(torch.float8_e4m3fn)
        st[key + ".weight"] = w
        st[key + ".scale"] = torch.rand(per, n, k // 128, generator=g, device=dev) * 0.01 + 0.001

    st["model.embed_tokens.weight"], st["model.norm.weight"] = bf(s.vocab_size, s.hidden_size), norm(s.hidden_size)
    st["lm_head.weight"] = bf(s.vocab_size, s.hidden_size)
    for i in range(s.num_layers):
        p = f"model.layers.{i}."
        a, m = p + "self_attn.", p + "mlp."
        st[p + "input_layernorm.weight"], st[p + "post_attention_layernorm.weight"] = norm(s.hidden_size), norm(s.hidden_size)
        st[a + "q_a_layernorm.weight"], st[a + "kv_a_layernorm.weight"] = norm(s.q_lora_rank), norm(D_LATENT)
        fp8(a + "q_a_proj", s.q_lora_rank, s.hidden_size)
        st[a + "q_b_absorbed.weight"] = bf(hl * D_K, s.q_lora_rank)
        st[a + "o_fused.weight"] = bf(s.hidden_size, hl * D_LATENT)
        fp8(a + "kv_a_latent", D_LATENT, s.hidden_size)
        fp8(a + "kv_a_rope", 128, s.hidden_size)
        if i < s.first_moe_layer:
            sub, width = "", s.intermediate_size // world
        else:
            sub, width = "shared_experts.", s.moe_intermediate_size // world
            st[m + "gate.weight"] = bf(s.num_experts, s.hidden_size)
            st[m + "gate.e_score_correction_bias"] = torch.randn(s.num_experts, generator=g, device=dev) * 0.1
            experts(m + "experts.w13", 2 * s.moe_intermediate_size, s.hidden_size)
            experts(m + "experts.w2", s.hidden_size, s.moe_intermediate_size)
        fp8(m + sub + "gate_proj", width, s.hidden_size)
        fp8(m + sub + "up_proj", width, s.hidden_size)
        fp8(m + sub + "down_proj", s.hidden_size, width)
    return st


def run_deepseek_slice(args):
    """BASELINE configuration 5: DeepSeek-V3-architecture 4-layer slice (1 dense + 3 MoE layers), FP8 weights, batch 32,
    context 4096; on N GPUs attention / dense MLP / shared expert tensor parallel and the routed experts 256 / N per
    GPU.  tok/s = batch / (max over ranks of the CUDA-event time of a decode iteration)."""
    import torch
    import torch.distributed as dist
    from mirage_b200.builders.deepseek_v3 import D_K, DeepSeekV3Runner, DeepSeekV3Shape
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    shape = DeepSeekV3Shape()
    B = 32 if args.batch == 1 else args.batch
    ctx = 4096 if args.context == 1024 else args.context
    K, Wm = (args.steps if args.steps != 128 else 16), max(args.warmup, 3)
    page = 64
    max_seq = (ctx + K + Wm + 16 + page - 1) // page * page
    state = synthetic_deepseek_state(shape, world, rank, dev, 1000 + 5)     # same seed on every rank: replicated tensors agree
    runner = DeepSeekV3Runner(shape, total_num_requests=B, max_seq_length=max_seq, max_num_batched_requests=B,
                              max_num_batched_tokens=B, max_num_pages=B * (max_seq // page), page_size=page,
                              world_size=world, rank=rank, device=local, prepared=state)
    g = torch.Generator().manual_seed(2005)
    runner.load_prompts([torch.randint(0, shape.vocab_size, (1,), generator=g).tolist() for _ in range(B)])
    mpk = runner.mpk

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    mpk.step(ctx)
    mpk.step(Wm)
    st = mpk.status()
    assert st.error == 0 and st.active_tokens == B, (st.error, st.active_tokens)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        e0.record()
        mpk.step(K)
        e1.record()
        sync_all()
    assert mpk.status().error == 0
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / K
    if rank == 0:
        # bytes this rank must read per iteration: its dense weights, the panels (+ float32 row scales) of its experts
        # that received a token in the last iteration, and the latent cache rows of every request
        active = [int(mpk.tensor_as_torch(m)[-1].item()) for m in runner.builder.moe_masks]
        I, H = shape.moe_intermediate_size, shape.hidden_size
        expert_bytes = sum(active) * (3 * I * H + 4 * (2 * I * (H // 128) + H * (I // 128)))
        kv_bytes = shape.num_layers * B * ctx * D_K * 2
        wbytes = mpk.graph_info()["weight_bytes_per_step"] + expert_bytes
        peak, peak_kind = measured_peak_gbs()
        achieved = (wbytes + kv_bytes) / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": f"deepseek_v3_slice_tok_per_s_bs{B}", "value": B * 1e3 / ms, "unit": "tok/s", "n_gpus": world, "steps": K,
            "warmup": Wm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8_e4m3 weights (bf16 absorbed q_b / fused o_proj / lm_head), bf16 activations", "data": "synthetic",
            "config": {"workload": f"DeepSeek-V3-shape slice, 1 dense + 3 MoE layers, batch {B}, context {ctx}, "
                                   f"TP={world} (attention, dense and shared MLP), {shape.num_experts // world} routed experts per GPU",
                       "active_local_experts_per_moe_layer": active, "l2": "bytes per iteration exceed L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind, "kernel": "mpk_megakernel<true%s>" % (", true" if world > 1 else ""),
                         "algorithmic_bytes_per_launch": wbytes + kv_bytes, "weight_bytes": wbytes, "kv_bytes": kv_bytes},
            "gpu_launches": K, "clocks": clocks.summary(), "tasks_per_launch": mpk.graph_info()["num_tasks"]}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=36, help="debug only: fewer layers (result is not a bench value)")
    ap.add_argument("--impl", default="mpk_b200")
    ap.add_argument("--sampling-seed", type=int, default=None,
                    help="side measurement: Gumbel-max sampling instead of greedy argmax (not the headline config)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-batches", action="store_true",
                    help="batch 1 only: skip the batch 16 / 64 measurements a default run adds to its line")
    ap.add_argument("--context-range", type=int, nargs=2, metavar=("LO", "HI"), default=None,
                    help="batch > 1: per-request contexts drawn uniformly from [LO, HI] (seeded) instead of --context")
    ap.add_argument("--fp8", action="store_true",
                    help="the FP8 decoder: e4m3 projection weights with 128 x 128 block scales, per-token activation "
                         "quantisation, block-scaled tcgen05 linears (quoted at --batch 64 --context 2048, 1 and 8 GPUs)")
    ap.add_argument("--shard-lm-head", action="store_true",
                    help="N > 1: split the lm_head rows over the ranks and merge the ranks' argmax inside the kernel "
                         "(default: every rank keeps the whole lm_head, as the reference does)")
    ap.add_argument("--workload", default="qwen3", choices=["qwen3", "fp8_layer", "moe_block", "mla_decode", "deepseek_slice", "moe_w13", "mla_dense"],
                    help="qwen3: the headline decode benchmark; the others time one block of the FP8 / MoE / MLA "
                         "task bodies at the shapes of the DeepSeek-V3-style parity configurations (1 GPU)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "ref_kernel":
        return run_ref_kernel(args)
    if args.workload == "deepseek_slice":
        return run_deepseek_slice(args)
    if args.workload != "qwen3":
        return run_block_workload(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    shape = dict(QWEN3_8B, num_layers=args.layers)
    weights = make_gpu_weights(shape, 1000 + 2, dev)      # identical on every rank (same seed)
    K, Wm = args.steps, max(args.warmup, 3)
    ctx_range = tuple(args.context_range) if args.context_range else None
    fp8 = None
    if args.fp8:
        fp8 = make_fp8_checkpoint(weights, shape, 3003, dev)
        for name in fp8:            # the bf16 projections are not part of the FP8 graph
            weights[name] = weights[name][:0]

    head = measure_decode(args, shape, weights, args.batch, args.context, ctx_range, K, Wm, world, rank, local, dev,
                          fp8=fp8)
    # The metric has two halves: ms/token at batch 1 and tok/s at batch 16 (and 64).  A default (batch 1) run times
    # the larger batches too, on the same weights, and carries them in the headline line.
    extra = {}
    if args.batch == 1 and not args.no_extra_batches and args.sampling_seed is None and not args.fp8:
        for b in (16, 64):
            r = measure_decode(args, shape, weights, b, args.context, ctx_range, min(K, 32), Wm, world, rank, local, dev,
                               with_e2e=False)
            extra[f"bs{b}_tok_s"] = r["value"]
            extra[f"bs{b}_ms_per_step"] = r["ms_step"]
            extra[f"bs{b}_frac"] = r["frac"]
            extra[f"bs{b}_contexts"] = r["contexts"]
    del weights

    if rank == 0:
        B, ctx = args.batch, args.context
        peak, peak_kind = measured_peak_gbs()
        bs1 = B == 1
        unit = "ms/token" if bs1 else "tok/s"
        # DRAM bytes of one launch: ncu capture of a 4-layer case (dram read + write = 1.0065 x its weight bytes),
        # scaled to this launch by the weight bytes it streams; only for the captured configuration (batch 1, TP=1)
        traffic = int(head["wbytes"] * 1.0065) if (bs1 and world == 1 and args.layers == 36) else None
        line = {
            "metric": metric_name(B, args.fp8), "value": head["value"], "unit": unit, "n_gpus": world, "steps": K,
            "warmup": Wm, "ms_per_step": head["ms_step"], "higher_is_better": not bs1, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> fp32 (bf16 activations)" if args.fp8 else "bf16",
            "data": "synthetic", "config": workload_config(args),
            "roofline": {"bound": "hbm", "achieved": head["achieved"], "peak": peak, "unit": "GB/s", "frac": head["frac"],
                         "traffic": traffic, "peak_kind": peak_kind,
                         "kernel": "mpk_megakernel<%s>" % ("true" if B > 8 or args.sampling_seed is not None else "false"),
                         "algorithmic_bytes_per_launch": head["wbytes"]},
            "e2e": {"value": head["e2e_value"], "unit": unit, "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B},
            "gpu_launches": K, "clocks": head["clocks"],
            "tasks_per_launch": head["tasks"],
        }
        line["config"]["contexts"] = head["contexts"]
        if extra:
            line["extra"] = extra
        if args.layers != 36:
            line["config"]["debug_layers"] = args.layers
        if args.sampling_seed is not None:
            line["config"]["sampling_seed"] = args.sampling_seed
        if world == 1 and not args.no_cpu_baseline and not args.fp8:
            ms_tok, sample, cores, _ = cpu_reference_ms_per_token(dict(QWEN3_8B, num_layers=args.layers), ctx, B,
                                                                  steps=3, warmup=1)
            line["cpu_baseline"] = {"value": ms_tok if bs1 else 1e3 / ms_tok, "unit": unit, "cores": cores,
                                    "kind": "port", "sample": sample}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def ragged_prompt_lengths(targets, budget):
    """Prompt lengths that leave request i with about targets[i] cached positions when the last request has finished
    its prefill.  The scheduler prefills greedily in request order under a budget of `budget` tokens per iteration
    while the requests already decoding take one token each, so request i keeps growing for as many iterations as
    the prefill of the requests after it takes; those iterations are simulated here and taken off its prompt."""
    n = len(targets)
    targets = sorted(targets, reverse=True)   # the request that waits longest for the others is the one meant to be longest
    prompts = list(targets)
    for _ in range(6):
        done_at, it, i, left = [0] * n, 0, 0, prompts[0]
        while i < n:
            room = budget - i                     # requests 0 .. i-1 decode one token each
            it += 1
            while room > 0 and i < n:
                take = min(room, left)
                left -= take
                room -= take
                if left == 0:
                    done_at[i] = it
                    i += 1
                    left = prompts[i] if i < n else 0
                else:
                    break
        prompts = [max(1, targets[k] - (it - done_at[k])) for k in range(n)]
    return prompts


def measure_decode(args, shape, weights, B, ctx, ctx_range, K, Wm, world, rank, local, dev, with_e2e=True, fp8=None):
    """Builds the decoder for a batch of B requests, brings every request to its context, and times K decode
    iterations (one launch each) with CUDA events on the launch stream, max over ranks."""
    import torch
    import torch.distributed as dist
    from mirage_b200.builders.runner import DecoderShape, Qwen3Runner

    page = 64
    g = torch.Generator().manual_seed(2002)
    if ctx_range and B > 1:
        lo, hi = ctx_range
        targets = sorted(torch.randint(lo, hi + 1, (B,), generator=g).tolist(), reverse=True)
        plens = ragged_prompt_lengths(targets, B)
        ctx_max = hi + 2 * B
    else:
        targets = [ctx] * B
        # Batch 1: a ctx-token random prompt, fed one token per launch.  Batch > 1 at a uniform context: one-token
        # prompts, and the context is built by ctx decode iterations (long prompts under a budget of B tokens would be
        # prefilled one request after the other, leaving the requests at very different lengths).
        plens = [ctx if B == 1 else 1] * B
        ctx_max = ctx
    max_seq = ctx_max + K + Wm + 2 * K + 16          # room for warm-up, the timed steps and the end-to-end pass
    max_seq = (max_seq + page - 1) // page * page
    pages = B * (max_seq // page)
    ds = DecoderShape(max_position=max(4096, max_seq), **shape)
    runner = Qwen3Runner(ds, weights, total_num_requests=B, max_seq_length=max_seq, max_num_batched_requests=B,
                         max_num_batched_tokens=B, max_num_pages=pages, page_size=page, world_size=world, rank=rank,
                         device=local, sampling_seed=args.sampling_seed, fp8_state_dict=fp8,
                         shard_lm_head=getattr(args, "shard_lm_head", False))
    prompts = [torch.randint(0, shape["vocab_size"], (n,), generator=g).tolist() for n in plens]
    runner.load_prompts(prompts)
    mpk = runner.mpk

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    if ctx_range and B > 1:
        # run until every request decodes one token per launch
        for _ in range(4 * (sum(plens) // B + B) // 64 + 2):
            mpk.step(64)
            qo = runner.meta["qo_indptr_buffer"].cpu().tolist()
            if qo[:B + 1] == list(range(B + 1)):
                break
    else:
        mpk.step(ctx)     # every request advances one position per launch (prompt token at batch 1, decoded token otherwise)
    mpk.step(Wm)
    st = mpk.status()
    assert st.error == 0 and st.active_tokens == B, (st.error, st.active_tokens)
    qo = runner.meta["qo_indptr_buffer"].cpu().tolist()
    assert qo[:B + 1] == list(range(B + 1)), f"timed region must hold {B} decoding requests of one token each: {qo}"
    steps_now = runner.meta["step"].cpu().tolist()[:B]
    contexts = {"min": int(min(steps_now)), "max": int(max(steps_now)), "mean": float(sum(steps_now)) / B}
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        e0.record()
        mpk.step(K)
        e1.record()
        sync_all()
    ms = e0.elapsed_time(e1)
    st = mpk.status()
    assert st.error == 0 and st.active_tokens == B
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / K

    e2e_ms_step = None
    if with_e2e:
        # end to end through the public API with host buffers: each step the host hands the token ids it read
        # back in the previous step to the device (pinned -> device) and reads the new ids (device -> pinned)
        host_tok = torch.zeros(B, 1, dtype=torch.int64).pin_memory()
        out_tok = runner.meta["output_tokens"]
        host_tok.copy_(out_tok)
        sync_all()
        t0 = time.perf_counter()
        for _ in range(K):
            out_tok.copy_(host_tok, non_blocking=True)
            mpk.step(1)
            host_tok.copy_(out_tok, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        sync_all()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([e2e_ms], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms_step = float(t.item()) / K
        assert mpk.status().error == 0

    peak, _ = measured_peak_gbs()
    info = mpk.graph_info()
    wbytes = info["weight_bytes_per_step"]
    achieved = wbytes / (ms_step * 1e-3) / 1e9
    to_metric = (lambda m: m / B) if B == 1 else (lambda m: B * 1e3 / m)
    res = {"value": to_metric(ms_step), "ms_step": ms_step, "achieved": achieved, "frac": achieved / peak, "wbytes": wbytes,
           "e2e_value": to_metric(e2e_ms_step) if e2e_ms_step else None, "clocks": clocks.summary(),
           "tasks": info["num_tasks"], "contexts": contexts}
    del runner, mpk
    torch.cuda.empty_cache()
    return res


if __name__ == "__main__":
    main()
