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


def cpu_reference_ms_per_token(shape, context, batch, layers_sampled=2, steps=2):
    """The CPU oracle (a port of the reference's PyTorch forward) on the host cores.

    Bounded sample: `steps` decode iterations of a `layers_sampled`-layer slice plus the lm_head at the
    benchmark's context length; the per-layer time is scaled to the full depth.  Returns
    (ms per token of the full model, description, cores)."""
    import torch
    from oracle.qwen3_decoder import Qwen3Config, Qwen3Oracle, make_weights
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = Qwen3Config(num_layers=layers_sampled, hidden_size=shape["hidden_size"], num_q_heads=shape["num_q_heads"],
                      num_kv_heads=shape["num_kv_heads"], head_dim=shape["head_dim"],
                      intermediate_size=shape["intermediate_size"], vocab_size=shape["vocab_size"])
    w = make_weights(cfg, seed=1)
    page = 64
    pages_per_req = (context + steps + page) // page
    orc = Qwen3Oracle(cfg, w, max_num_pages=pages_per_req * batch, page_size=page)
    g = torch.Generator().manual_seed(0)
    for kc in orc.k_cache + orc.v_cache:      # a random "prefilled" cache: same arithmetic, no CPU prefill
        kc.copy_(torch.randn(kc.shape, generator=g).to(torch.bfloat16))
    ids = torch.randint(0, cfg.vocab_size, (batch,), generator=g)

    def run(nl_only_head=False):
        reqs = [((b, b + 1), list(range(b * pages_per_req, (b + 1) * pages_per_req)), context + 1) for b in range(batch)]
        t0 = time.perf_counter()
        orc.forward_tokens(ids, reqs)
        return time.perf_counter() - t0

    run()                                       # warm-up
    full = min(run() for _ in range(steps))
    # time of the non-layer part (embedding + final norm + lm_head): a 0-layer oracle
    cfg0 = Qwen3Config(num_layers=0, hidden_size=cfg.hidden_size, num_q_heads=cfg.num_q_heads,
                       num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                       intermediate_size=cfg.intermediate_size, vocab_size=cfg.vocab_size)
    orc0 = Qwen3Oracle(cfg0, w, max_num_pages=1, page_size=page)
    orc0.forward_tokens(ids, [])
    t0 = time.perf_counter()
    orc0.forward_tokens(ids, [])
    head = time.perf_counter() - t0
    per_layer = max(full - head, 0.0) / layers_sampled
    total_s = head + per_layer * shape["num_layers"]
    sample = (f"{steps} decode steps of a {layers_sampled}-layer slice + lm_head at context {context}, batch {batch}; "
              f"per-layer time scaled to {shape['num_layers']} layers")
    return total_s * 1e3 / batch, sample, cores


def run_reference(args):
    """`--impl reference`: the reference's CPU path for the same metric (the CPU oracle port; the reference's
    own megakernel cannot be built in this image and its PyTorch model needs its CUDA extension)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    shape = dict(QWEN3_8B)
    ms_tok, sample, cores = cpu_reference_ms_per_token(shape, args.context, args.batch)
    bs1 = args.batch == 1
    value = ms_tok if bs1 else 1e3 / ms_tok
    unit = "ms/token" if bs1 else "tok/s"
    line = {"impl": "reference", "metric": metric_name(args.batch), "value": value, "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_tok * args.batch,
            "higher_is_better": not bs1, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(args),
            "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def metric_name(batch):
    return "qwen3_8b_decode_ms_per_token_bs1" if batch == 1 else f"qwen3_8b_decode_tok_per_s_bs{batch}"


def workload_config(args):
    return {"workload": f"Qwen3-8B-shape decoder, 36 layers, bf16, batch {args.batch}, context {args.context}, "
                        f"paged KV (page 64), greedy decode, TP={args.gpus}",
            "global_batch": args.batch, "context": args.context, "parallelism": f"tp{args.gpus}",
            "l2": "weights (15 GB) exceed L2; every step re-streams them from HBM"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=36, help="debug only: fewer layers (result is not a bench value)")
    ap.add_argument("--impl", default="mpk_b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from mirage_b200.builders.runner import DecoderShape, Qwen3Runner

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    shape = dict(QWEN3_8B, num_layers=args.layers)
    B, ctx, K, Wm = args.batch, args.context, args.steps, max(args.warmup, 3)
    page = 64
    max_seq = ctx + K + Wm + 2 * K + 16          # room for warm-up, the timed steps and the end-to-end pass
    max_seq = (max_seq + page - 1) // page * page
    pages = B * (max_seq // page)
    weights = make_gpu_weights(shape, 1000 + 2, dev)      # identical on every rank (same seed)
    ds = DecoderShape(max_position=max(4096, max_seq), **shape)
    runner = Qwen3Runner(ds, weights, total_num_requests=B, max_seq_length=max_seq, max_num_batched_requests=B,
                         max_num_batched_tokens=B, max_num_pages=pages, page_size=page, world_size=world, rank=rank,
                         device=local)
    del weights
    g = torch.Generator().manual_seed(2002)
    prompts = torch.randint(0, shape["vocab_size"], (B, ctx), generator=g).tolist()
    runner.load_prompts(prompts)
    mpk = runner.mpk

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # context: with a token budget of B per iteration every request advances one prompt token per launch
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
    ms = e0.elapsed_time(e1)
    st = mpk.status()
    assert st.error == 0 and st.active_tokens == B
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / K

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
    st = mpk.status()
    assert st.error == 0

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        info = mpk.graph_info()
        wbytes = info["weight_bytes_per_step"]
        achieved = wbytes / (ms_step * 1e-3) / 1e9
        bs1 = B == 1
        to_metric = (lambda m: m / B) if bs1 else (lambda m: B * 1e3 / m)
        unit = "ms/token" if bs1 else "tok/s"
        line = {
            "metric": metric_name(B), "value": to_metric(ms_step), "unit": unit, "n_gpus": world, "steps": K,
            "warmup": Wm, "ms_per_step": ms_step, "higher_is_better": not bs1, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind, "kernel": "mpk_megakernel",
                         "algorithmic_bytes_per_launch": wbytes},
            "e2e": {"value": to_metric(e2e_ms_step), "unit": unit, "h2d_bytes_per_step": 8 * B,
                    "d2h_bytes_per_step": 8 * B},
            "gpu_launches": K, "clocks": clocks.summary(),
            "tasks_per_launch": info["num_tasks"],
        }
        if args.layers != 36:
            line["config"]["debug_layers"] = args.layers
        if world == 1 and not args.no_cpu_baseline:
            ms_tok, sample, cores = cpu_reference_ms_per_token(dict(QWEN3_8B), ctx, B)
            line["cpu_baseline"] = {"value": ms_tok if bs1 else 1e3 / ms_tok, "unit": unit, "cores": cores,
                                    "kind": "port", "sample": sample}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
