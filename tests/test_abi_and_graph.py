"""CPU-only checks: the C-ABI library loads and exports every declared symbol, and the task-graph
compiler (run in dry-run mode, which makes no CUDA call) folds, partitions and orders the Qwen3 graph
as designed."""
import ctypes
import json
import os
import re

import pytest
import torch

from oracle.qwen3_decoder import Qwen3Config
from dry_util import dry_qwen3

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_symbol_of_the_header():
    hdr = open(os.path.join(ROOT, "include", "mpk_b200.h")).read()
    declared = set(re.findall(r"\b(mpk_[a-z_0-9]+)\s*\(", hdr))
    assert len(declared) >= 19
    from mirage_b200 import _native
    lib = ctypes.CDLL(_native._LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/mpk_b200.h but not exported"
    assert declared == set(_native.SYMBOLS), declared ^ set(_native.SYMBOLS)


def test_config_struct_matches_header_layout():
    from mirage_b200 import _native
    # 15 int32 (+1 pad) + int64 + 12 pointers + uint64, as in mpk_config
    assert ctypes.sizeof(_native.MpkConfig) == 14 * 4 + 8 + 12 * 8 + 8
    assert ctypes.sizeof(_native.MpkStatus) == 6 * 4 + 8


def test_create_rejects_bad_arguments_with_message():
    import mirage_b200 as mi
    with pytest.raises(mi.MpkError) as e:
        mi.PersistentKernel(mode="offline", world_size=9, mpi_rank=0, test_mode=True, dry_run=True)
    assert "world_size" in str(e.value)
    with pytest.raises(ValueError):
        mi.PersistentKernel(mode="bogus", dry_run=True, test_mode=True)


def test_qwen3_8b_graph_single_gpu():
    pk = dry_qwen3(Qwen3Config.qwen3_8b(36))
    info = pk.graph_info()
    g = json.loads(pk.dump_task_graph())
    # weight bytes of one decode step: 36 x 192,937,984 + 151,936 x 4096 parameters, 2 bytes each
    assert info["weight_bytes_per_step"] == (36 * 192937984 + 151936 * 4096) * 2
    assert info["num_workers"] == 148
    # every rmsnorm and silu_mul of the builder's graph is folded into its consumer: 36 * 3 + 1
    assert info["num_folded"] == 109
    types = [e["type"] for e in g["events"]]
    assert types[:3] == ["batch", "embed", "linear"]
    assert types.count("attention") == 36 and types.count("linear") == 36 * 4 + 1
    assert "rmsnorm" not in types and "silu_mul" not in types
    # a pure chain: every event has exactly one dependency, on its predecessor, counting all its tasks
    for i, e in enumerate(g["events"][1:], start=1):
        assert [d[0] for d in e["deps"]] == [i - 1]
        assert e["deps"][0][1] == g["events"][i - 1]["tasks"]
    per_layer = g["events"][2:7]
    # rmsnorm rides in the prologue of qkv and gate_up; silu_mul in the EPILOGUE of gate_up (its [gate | up] weight
    # rows are re-interleaved 2 + 2 at compile time), so the down projection stages plain activations
    assert [e.get("prologue") for e in per_layer] == ["rmsnorm", None, None, "rmsnorm", None]
    assert [e.get("epilogue") for e in per_layer] == [None, None, None, "silu_mul", None]
    assert per_layer[1]["type"] == "attention" and per_layer[1]["tasks"] == 8 * 18


@pytest.mark.parametrize("world", [2, 4, 8])
def test_qwen3_8b_graph_tensor_parallel(world):
    pk = dry_qwen3(Qwen3Config.qwen3_8b(4), world=world, rank=world - 1, mbt=4, mbr=4)
    g = json.loads(pk.dump_task_graph())
    types = [e["type"] for e in g["events"]]
    # the allreduce layers leave no task behind: pushed by the producer, gathered by the consumers
    assert "allreduce" not in types
    per_rank = (4 * 192937984 // world + 151936 * 4096) * 2
    assert pk.graph_info()["weight_bytes_per_step"] == per_rank


@pytest.mark.parametrize("world", [2, 8])
def test_qwen3_8b_graph_with_sharded_lm_head(world):
    """lm_head rows split over the ranks: each rank streams 1 / world of it, and the argmax merge becomes one exchange
    task that is a further instance of the allreduce sequence with its own area behind the partial-sum words."""
    pk = dry_qwen3(Qwen3Config.qwen3_8b(4), world=world, rank=1, mbt=4, mbr=4, shard_lm_head=True)
    g = json.loads(pk.dump_task_graph())
    types = [e["type"] for e in g["events"]]
    assert types.count("argmax_exchange") == 1 and "argmax_reduce" not in types and "allreduce" not in types
    assert pk.graph_info()["weight_bytes_per_step"] == (4 * 192937984 + 151936 * 4096) // world * 2


def test_unfoldable_allreduce_keeps_reduce_tasks():
    """An allreduce whose result feeds a non-linear layer stays a separate task group."""
    import mirage_b200 as mi
    pk = mi.PersistentKernel(mode="offline", world_size=2, mpi_rank=0, max_num_batched_tokens=2,
                             max_num_batched_requests=2, test_mode=True, dry_run=True)
    meta = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device="meta")
    x, w = pk.attach_input(meta(2, 256), "x"), pk.attach_input(meta(512, 256), "w")
    part = pk.new_tensor((2, 512), name="part", io_category="nvshmem_tensor")
    buf = pk.new_tensor((2, 2, 512), name="buf", io_category="nvshmem_tensor")
    red = pk.new_tensor((2, 512), name="red", io_category="nvshmem_tensor")
    out = pk.attach_input(meta(2, 512), "out")
    pk.linear_layer(input=x, weight=w, output=part, grid_dim=(8, 1, 1), block_dim=(128, 1, 1))
    pk.allreduce_layer(input=part, buffer=buf, output=red, grid_dim=(8, 1, 1), block_dim=(128, 1, 1))
    pk.elementwise_add_layer(input_a=red, input_b=red, output=out, grid_dim=(2, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    g = json.loads(pk.dump_task_graph())
    assert [e["type"] for e in g["events"]] == ["linear", "allreduce", "elementwise_add"]
    assert g["events"][0].get("push") is True
    # the reduce tasks wait for the pushes of both ranks
    assert g["events"][1]["deps"][0][1] == 2 * g["events"][0]["tasks"]


def test_caller_visible_intermediates_are_not_folded():
    import mirage_b200 as mi
    pk = mi.PersistentKernel(mode="offline", max_num_batched_tokens=2, max_num_batched_requests=2, test_mode=True,
                             dry_run=True)
    meta = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device="meta")
    x, gam, w = pk.attach_input(meta(2, 256), "x"), pk.attach_input(meta(256), "g"), pk.attach_input(meta(64, 256), "w")
    normed = pk.attach_input(meta(2, 256), "normed")          # attached: the caller may read it
    out = pk.attach_input(meta(2, 64), "out")
    pk.rmsnorm_layer(input=x, weight=gam, output=normed, grid_dim=(2, 1, 1), block_dim=(128, 1, 1))
    pk.linear_layer(input=normed, weight=w, output=out, grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    assert pk.graph_info()["num_folded"] == 0


def test_graph_errors_are_reported_not_fatal():
    import mirage_b200 as mi
    pk = mi.PersistentKernel(mode="offline", max_num_batched_tokens=1, test_mode=True, dry_run=True)
    meta = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device="meta")
    x, w, out = pk.attach_input(meta(1, 100), "x"), pk.attach_input(meta(64, 100), "w"), pk.attach_input(meta(1, 64), "o")
    pk.linear_layer(input=x, weight=w, output=out, grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
    with pytest.raises(mi.MpkError) as e:
        pk.compile()
    assert "multiple of 16" in str(e.value)
    with pytest.raises((mi.MpkError, AssertionError)):
        pk.step(1)      # launch before a successful compile


def test_fp8_quantize_linear_graph_compiles_and_schedules():
    """quantize -> FP8 linear (+ residual) as a dry-run graph: tasks exist, the linear waits for the quantiser."""
    import mirage_b200 as mi
    mbt, k, n = 4, 7168, 2112
    pk = mi.PersistentKernel(mode="offline", test_mode=True, num_workers=148, max_num_batched_tokens=mbt,
                             max_num_batched_requests=mbt, dry_run=True)
    meta = lambda dt, *s: torch.empty(*s, dtype=dt, device="meta")
    x = pk.attach_input(meta(torch.bfloat16, mbt, k), "x")
    wq = pk.attach_input(meta(torch.float8_e4m3fn, n, k), "wq")
    ws = pk.attach_input(meta(torch.uint32, n, (k // 128 + 3) // 4), "ws")
    res = pk.attach_input(meta(torch.bfloat16, mbt, n), "res")
    q = pk.new_tensor(dims=(mbt, k), dtype=mi.float8_e4m3, name="q", io_category="cuda_tensor")
    s = pk.new_tensor(dims=((k // 128 + 3) // 4, 4), dtype=mi.uint32, name="s", io_category="cuda_tensor")
    y = pk.new_tensor(dims=(mbt, n), dtype=mi.bfloat16, name="y", io_category="cuda_tensor")
    pk.quantize_fp8_layer(input=x, output_fp8=q, output_scale=s, grid_dim=(mbt, 1, 1), block_dim=(128, 1, 1))
    pk.linear_fp8_with_residual_layer(input_fp8=q, input_scale=s, weight_fp8=wq, weight_scale=ws, residual=res,
                                      output=y, grid_dim=(16, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    info = pk.graph_info()
    assert info["num_tasks"] >= 148 and info["num_events"] == 2
    assert info["weight_bytes_per_step"] == n * k     # one byte per weight element


def test_fp8_linear_rejects_bad_scale_shapes():
    import mirage_b200 as mi
    pk = mi.PersistentKernel(mode="offline", test_mode=True, num_workers=8, max_num_batched_tokens=1,
                             max_num_batched_requests=1, dry_run=True)
    meta = lambda dt, *s: torch.empty(*s, dtype=dt, device="meta")
    xq = pk.attach_input(meta(torch.float8_e4m3fn, 1, 1024), "xq")
    xs = pk.attach_input(meta(torch.uint32, 1, 2), "xs")
    wq = pk.attach_input(meta(torch.float8_e4m3fn, 256, 1024), "wq")
    ws = pk.attach_input(meta(torch.uint32, 256, 3), "ws")     # K/512 = 2 expected
    y = pk.attach_input(meta(torch.bfloat16, 1, 256), "y")
    pk.linear_fp8_layer(input_fp8=xq, input_scale=xs, weight_fp8=wq, weight_scale=ws, output=y, grid_dim=(2, 1, 1),
                        block_dim=(128, 1, 1))
    with pytest.raises(mi.MpkError, match="scale tensor"):
        pk.compile()


def test_moe_block_graph_deepseek_shapes_schedules():
    """Routed-expert block at DeepSeek-V3 sizes (256 experts, top-8, hidden 7168, expert width 2048, 32 tokens)
    as a dry-run graph: every worker owns rows of every expert, the expert tasks wait for the routing."""
    import mirage_b200 as mi
    b, e, topk, h, inter = 32, 256, 8, 7168, 2048
    pk = mi.PersistentKernel(mode="offline", test_mode=True, num_workers=148, max_num_batched_tokens=b,
                             max_num_batched_requests=b, dry_run=True)
    meta = lambda dt, *s: torch.empty(*s, dtype=dt, device="meta")
    nt = lambda dims, dt, name: pk.new_tensor(dims=dims, dtype=dt, name=name, io_category="cuda_tensor")
    x = pk.attach_input(meta(torch.bfloat16, b, h), "x")
    logits = pk.attach_input(meta(torch.bfloat16, b, e), "logits")
    bias = pk.attach_input(meta(torch.float32, e), "bias")
    w13 = pk.attach_input(meta(torch.float8_e4m3fn, e, 2 * inter, h), "w13")
    w13s = pk.attach_input(meta(torch.float32, e, 2 * inter, h // 128), "w13s")
    w2 = pk.attach_input(meta(torch.float8_e4m3fn, e, h, inter), "w2")
    w2s = pk.attach_input(meta(torch.float32, e, h, inter // 128), "w2s")
    t_w, t_idx, t_mask = nt((b, topk), mi.float32, "tw"), nt((e, b), mi.int32, "idx"), nt((e + 1,), mi.int32, "mask")
    xq, xs = nt((b, h), mi.float8_e4m3, "xq"), nt((b, h // 128), mi.float32, "xs")
    mid, act = nt((b, topk, 2 * inter), mi.bfloat16, "mid"), nt((b, topk, inter), mi.bfloat16, "act")
    aq, asc = nt((b, topk, inter), mi.float8_e4m3, "aq"), nt((b, topk, inter // 128), mi.float32, "as")
    down, y = nt((b, topk, h), mi.bfloat16, "down"), nt((b, h), mi.bfloat16, "y")
    pk.moe_topk_sigmoid_routing_layer(input=logits, bias=bias, output=(t_w, t_idx, t_mask), grid_dim=(1, 1, 1),
                                      block_dim=(256, 1, 1))
    pk.quantize_fp8_layer(input=x, output_fp8=xq, output_scale=xs, grid_dim=(b, 1, 1), block_dim=(128, 1, 1),
                          scale_ue8m0=False)
    pk.moe_w13_fp8_layer(input_fp8=xq, input_scale=xs, weight_fp8=w13, weight_scale=w13s, moe_routing_indices=t_idx,
                         moe_mask=t_mask, output=mid, grid_dim=(32, 1, 1), block_dim=(128, 1, 1))
    pk.moe_silu_mul_layer(input=mid, output=act, grid_dim=(b, topk, 1), block_dim=(128, 1, 1))
    pk.quantize_fp8_layer(input=act, output_fp8=aq, output_scale=asc, grid_dim=(b * topk, 1, 1), block_dim=(128, 1, 1),
                          scale_ue8m0=False)
    pk.moe_w2_fp8_layer(input_fp8=aq, input_scale=asc, weight_fp8=w2, weight_scale=w2s, moe_routing_indices=t_idx,
                        moe_mask=t_mask, output=down, grid_dim=(32, 1, 1), block_dim=(128, 1, 1))
    pk.moe_mul_sum_add_layer(input=down, weight=t_w, residual=x, output=y, grid_dim=(b, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    info = pk.graph_info()
    assert info["num_events"] == 7
    g = json.loads(pk.dump_task_graph())
    kinds = [ev["type"] for ev in g["events"]]
    assert kinds == ["moe_routing", "quantize_fp8", "moe_gemm", "moe_silu_mul", "quantize_fp8", "moe_gemm",
                     "moe_mul_sum_add"]
    gemm = [ev for ev in g["events"] if ev["type"] == "moe_gemm"]
    assert all(ev["tasks"] >= 148 for ev in gemm)            # every worker holds rows of every expert
    assert [d[0] for d in gemm[0]["deps"]] == [0, 1]           # W13 waits for the routing and the quantiser


def test_mpk_wrapper_builds_and_compiles_qwen3_dry_run():
    """MPKMetadata / MPK (the reference's python/mirage/mpk/mpk.py wrapper): missing meta tensors are allocated,
    the registered Qwen3 builder is found by model name, build + compile produce the same graph as the bare
    PersistentKernel path."""
    import mirage_b200 as mi
    from mirage_b200.builders.qwen3 import Qwen3ModelConfig
    from dry_util import meta_state_dict
    cfg = Qwen3Config.qwen3_8b(2)
    pages, page = 32, 64
    kc = torch.empty(cfg.num_layers, pages, page, cfg.num_kv_heads, cfg.head_dim, dtype=torch.bfloat16, device="meta")
    rope = torch.empty(4096, cfg.head_dim, dtype=torch.bfloat16, device="meta")
    mc = Qwen3ModelConfig(cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_q_heads, cfg.num_kv_heads,
                          cfg.head_dim, cfg.num_layers, kc, kc, (rope, rope), meta_state_dict(cfg))
    meta = mi.MPKMetadata(mode="offline", total_num_requests=2, max_seq_length=2048, max_num_batched_requests=2,
                          max_num_batched_tokens=2, max_num_pages=pages, page_size=page, model_name="Qwen/Qwen3-8B",
                          model_config=mc, dry_run=True,
                          input_tokens=torch.empty(2, 1, dtype=torch.int32, device="meta"))
    m = mi.MPK(meta)
    assert m.need_cpy_input and m.input_tokens.dtype == torch.int64        # int32 ids get an int64 shadow
    assert m.tokens.shape == (2, 2048) and m.qo_indptr_buffer.shape == (3,)
    assert "max_seq_length: 2048" in meta.info_as_string()
    m.build()
    m.compile()
    info = m.persistent_kernel.graph_info()
    assert info["num_events"] == 1 + 1 + 2 * 5 + 3 and info["num_workers"] == 148
    with pytest.raises(KeyError):
        mi.get_builder("no-such-model")


def test_profiler_trace_export(tmp_path):
    """Records in the kernel's profiler layout -> Chrome/Perfetto trace with a wait slice and a body slice per task."""
    from mirage_b200.profiler import decode_records, export_to_perfetto_trace
    buf = torch.zeros(4 * 8, dtype=torch.int64)
    base = 1_000_000
    # (worker, event, type, begin, ready, end)
    tasks = [(0, 2, 4, base, base + 500, base + 9000), (3, 2, 4, base + 100, base + 600, base + 9500),
             (3, 3, 5, base + 9600, base + 12000, base + 20000)]
    for i, (w, ev, ty, b, r, e) in enumerate(tasks):
        buf[i * 8 + 0], buf[i * 8 + 1], buf[i * 8 + 2] = b, r, e
        buf[i * 8 + 3] = (w << 40) | (ev << 8) | ty
    recs = decode_records(buf, 4)                 # the fourth record is empty: that task did not run
    assert [(r["worker"], r["event"], r["type"]) for r in recs] == [(0, 2, 4), (3, 2, 4), (3, 3, 5)]
    assert recs[0]["begin_ns"] == 0 and recs[2]["end_ns"] == 20000
    path = tmp_path / "trace.json"
    n = export_to_perfetto_trace(buf, str(path), num_tasks=4,
                                 task_graph_json=json.dumps({"events": [{"event": 3, "out": "attn_out"}]}))
    assert n == 3
    ev = json.loads(path.read_text())["traceEvents"]
    assert len(ev) == 6 and {e["tid"] for e in ev} == {0, 3}
    assert any(e["name"] == "attention#3 -> attn_out" and abs(e["dur"] - 8.0) < 1e-9 for e in ev)


def test_profiler_buffer_in_the_reference_layout():
    """The converter's output, walked the way the reference's exporter walks its buffer
    (python/mirage/mpk/profiler_persistent.py:123-171; tag bits per include/mirage/persistent_kernel/profiler.h:34-47):
    every task shows up on its block as a TASK_GET_NEXT_TASK span and a span of the mapped sm100 task id, begin before
    end, with globaltimer_lo stamps, and event numbers count per (block, id)."""
    from mirage_b200.profiler import REFERENCE_EVENT_IDS, to_reference_profiler_buffer
    buf = torch.zeros(5 * 8, dtype=torch.int64)
    base = (7 << 32) + 4_000_000_000               # stamps whose low 32 bits have the top bit set
    tasks = [(0, 2, 4, base, base + 500, base + 9000), (3, 2, 4, base + 100, base + 600, base + 9500),
             (3, 3, 5, base + 9600, base + 12000, base + 20000), (3, 4, 4, base + 20100, base + 20100, base + 30000)]
    for i, (w, ev, ty, b, r, e) in enumerate(tasks):
        buf[i * 8 + 0], buf[i * 8 + 1], buf[i * 8 + 2] = b, r, e
        buf[i * 8 + 3] = (w << 40) | (ev << 8) | ty
    out = to_reference_profiler_buffer(buf, 5, num_workers=4)
    nblocks, ngroups = (int(v) for v in out[:1].view(torch.int32))
    assert (nblocks, ngroups) == (4, 1)
    spans, open_at = [], {}
    for i in range(1, len(out)):
        if out[i] == 0:
            continue
        tag, stamp = (int(v) for v in out[i:i + 1].view(torch.uint32))
        event_no, block_group, event_id, kind = tag >> 19, (tag >> 11) & 0xFF, (tag >> 2) & 0x1FF, tag & 0x3
        block = block_group // ngroups
        assert (i - 1) % nblocks == block          # the slot a block's k-th entry must sit in
        if kind == 0:
            open_at[(block, event_id)] = (stamp, event_no)
        else:
            t0, no = open_at.pop((block, event_id))
            assert no == event_no
            spans.append((block, event_id, event_no, t0, stamp))
    assert not open_at
    lo = lambda t: t & 0xFFFFFFFF
    lin, att = REFERENCE_EVENT_IDS["linear"], REFERENCE_EVENT_IDS["attention"]
    assert (lin, att) == (253, 257)
    assert sorted(spans) == sorted([
        (0, 203, 0, lo(base), lo(base + 500)), (0, lin, 0, lo(base + 500), lo(base + 9000)),
        (3, 203, 0, lo(base + 100), lo(base + 600)), (3, lin, 0, lo(base + 600), lo(base + 9500)),
        (3, 203, 1, lo(base + 9600), lo(base + 12000)), (3, att, 0, lo(base + 12000), lo(base + 20000)),
        (3, 203, 2, lo(base + 20100), lo(base + 20100)), (3, lin, 1, lo(base + 20100), lo(base + 30000))])
    with pytest.raises(ValueError):
        to_reference_profiler_buffer(buf, 5, num_workers=300)


@pytest.mark.parametrize("world", [1, 2])
def test_deepseek_slice_graph_compiles_and_schedules(world):
    """Dry run of the DeepSeek-V3 slice builder: the graph compiles and the host simulation of the event protocol runs
    every task once; with two ranks the dense MLP and the MoE block (whose outputs come from an FP8 linear and from the
    weighted expert sum, not from a bf16 linear) get a push stage in front of their allreduce."""
    import dataclasses
    import mirage_b200 as mi
    from mirage_b200.builders.deepseek_v3 import DeepSeekV3Builder, DeepSeekV3Shape, prepare_state
    from oracle.deepseek_v3 import DeepSeekConfig, make_checkpoint
    cfg = DeepSeekConfig.tiny()
    shape = DeepSeekV3Shape(**{f.name: getattr(cfg, f.name) for f in dataclasses.fields(DeepSeekV3Shape)})
    state = {k: v.to("meta") for k, v in prepare_state(make_checkpoint(cfg, 1005), shape, world, world - 1).items()}
    mbr, mbt, pages, page, max_seq = 2, 4, 12, 16, 64
    i32 = lambda *s: torch.empty(*s, dtype=torch.int32, device="meta")
    i64 = lambda *s: torch.empty(*s, dtype=torch.int64, device="meta")
    meta = dict(step=i32(3), tokens=i64(3, max_seq), input_tokens=i64(mbt, 1), output_tokens=i64(mbt, 1),
                num_new_tokens=i32(3), prompt_lengths=i32(3), qo_indptr_buffer=i32(mbr + 1),
                paged_kv_indptr_buffer=i32(mbr + 1), paged_kv_indices_buffer=i32(pages),
                paged_kv_last_page_len_buffer=i32(mbr))
    pk = mi.PersistentKernel(mode="offline", world_size=world, mpi_rank=world - 1, num_workers=0, max_seq_length=max_seq,
                             max_num_batched_requests=mbr, max_num_batched_tokens=mbt, max_num_pages=pages,
                             page_size=page, meta_tensors=meta, dry_run=True)
    caches = [torch.empty(pages, page, 576, dtype=torch.bfloat16, device="meta") for _ in range(shape.num_layers)]
    DeepSeekV3Builder(pk, shape).build(state, caches)
    pk.compile()
    types = [e["type"] for e in json.loads(pk.dump_task_graph())["events"]]
    assert types.count("moe_routing") == 1 and types.count("moe_gemm") == 2 and types.count("mla_decode") == 2
    assert types.count("ar_push") == (2 if world == 2 else 0) and types.count("allreduce") == (4 if world == 2 else 0)
    # this rank's experts only: 8 of 16 expert panels of w13 [2 * 512, 1024] and w2 [1024, 512] at one byte per weight
    expert_bytes = 16 // world * (2 * 512 * 1024 + 1024 * 512)
    assert pk.graph_info()["weight_bytes_per_step"] > 0 and expert_bytes > 0


@pytest.mark.parametrize("tokens,x_tile,stages", [(16, 120832, 6), (32, 105472, 7), (64, 133120, 5)])
def test_fp8_linear_activation_tile_plan(tokens, x_tile, stages):
    """FP8 tcgen05 linears (K = 4096 and K = 12288): the e4m3 activation tile with its scale words may run on into the
    8 KB partial-sum area behind the tile buffer, and the buffer is sized so that at least five 16 KB weight slots
    remain -- at 64 tokens that is a k tile of 2048 columns (64 x 2048 + 5 x 2048 - 8192 = 133120 bytes), two tiles per
    K = 4096 linear instead of four."""
    import mirage_b200 as mi
    params = mi.PersistentKernel.get_default_init_parameters()
    params.update(test_mode=True, num_workers=148, max_num_batched_tokens=tokens, max_num_batched_requests=tokens, dry_run=True)
    pk = mi.PersistentKernel(**params)
    m = lambda *s, dt=torch.bfloat16: torch.empty(*s, dtype=dt, device="meta")
    nt = lambda dims, dt, name: pk.new_tensor(dims=dims, dtype=dt, name=name, io_category="cuda_tensor")
    for (k, n, name) in ((4096, 6144, "qkv"), (12288, 4096, "down")):
        q = nt((tokens, k), mi.float8_e4m3, name + "_q")
        s = nt(((k // 128 + 3) // 4, (tokens + 3) // 4 * 4), mi.uint32, name + "_s")
        pk.quantize_fp8_layer(input=pk.attach_input(m(tokens, k), name + "_x"), output_fp8=q, output_scale=s,
                              grid_dim=(tokens, 1, 1), block_dim=(128, 1, 1))
        pk.linear_fp8_layer(input_fp8=q, input_scale=s, weight_fp8=pk.attach_input(m(n, k, dt=torch.float8_e4m3fn), name + "_w"),
                            weight_scale=pk.attach_input(m(n, (k // 128 + 3) // 4, dt=torch.int32), name + "_ws"),
                            output=nt((tokens, n), mi.bfloat16, name + "_y"), grid_dim=(n // 128, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    d = json.loads(pk.dump_task_graph())
    assert (d["x_tile_bytes"], d["num_stages"], d["stage_bytes"]) == (x_tile, stages, 16384)
    # shared memory of the launch: slots + tile buffer + partial-sum area + barriers / descriptors stays within 227 KB
    assert stages * 16384 + x_tile + 8192 + 1536 <= 232448


@pytest.mark.parametrize("workload", ["moe_w13", "mla_dense", "fp8_layer"])
def test_bench_reference_kernel_arm_without_a_gpu(workload):
    """`bench.py --impl ref_kernel` on a machine that cannot load the reference's compiled kernels (no CUDA driver, or
    nothing built) prints one JSON line saying so and exits 0, as the reference arm's contract asks."""
    import subprocess
    import sys
    if torch.cuda.is_available():
        pytest.skip("needs a machine without a GPU")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "ref_kernel", "--workload", workload],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-400:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "ref_kernel" and "unavailable" in line
