"""Dependency structure of multi-branch graphs (dry run, no CUDA call): who waits for whom after folding and
transitive reduction, and that the host simulation of the event protocol runs every task exactly once."""
import json

import pytest

import mirage_b200 as mi
from graph_shapes import KINDS, build


def _compile(kind, B=8, H=512):
    params = mi.PersistentKernel.get_default_init_parameters()
    params.update(test_mode=True, num_workers=0, max_num_batched_tokens=B, max_num_batched_requests=B, dry_run=True)
    pk = mi.PersistentKernel(**params)
    build(pk, kind, B, H, "meta")
    pk.compile()                       # includes simulate_task_graph: a deadlock or a miscounted event is an error
    g = json.loads(pk.dump_task_graph())
    by_out = {e["out"]: e for e in g["events"]}
    deps = {e["out"]: sorted(g["events"][d[0]]["out"] for d in e["deps"]) for e in g["events"]}
    return g, by_out, deps


def test_fork_two_consumers_wait_for_one_producer():
    g, ev, deps = _compile("fork")
    assert deps["xa"] == [] and deps["xb"] == ["xa"] and deps["xc"] == ["xa"]
    # every task of the producer must have finished: the consumers need all its arrivals
    a = ev["xa"]
    assert all(d[1] == a["tasks"] for e in (ev["xb"], ev["xc"]) for d in e["deps"])


def test_join_consumer_waits_for_both_producers():
    g, ev, deps = _compile("join")
    assert deps["xc"] == ["xa", "xb"]


def test_diamond():
    g, ev, deps = _compile("diamond")
    # xa is only read by the two linears, but it is a caller-visible buffer: the norm is not folded away
    assert deps["xb"] == ["xa"] and deps["xc"] == ["xa"] and deps["xd"] == ["xb", "xc"]


def test_residual_shortcut_is_covered_by_the_longer_path():
    g, ev, deps = _compile("residual_shortcut")
    # C reads xa (residual) and xb; xb's producer already waited for xa: transitive reduction leaves one edge
    assert deps["xc"] == ["xb"]


@pytest.mark.parametrize("kind", ["join_and_fork_consumer", "fork_and_join_producer"])
def test_role_combinations_the_reference_refuses_are_plain_graphs_here(kind):
    g, ev, deps = _compile(kind)
    if kind == "join_and_fork_consumer":
        assert deps["xb"] == ["xa", "xe"] and deps["xc"] == ["xa"]
    else:
        assert deps["xc"] == ["xa"] and deps["xd"] == ["xa", "xe"]


@pytest.mark.parametrize("B,H", [(4, 4096), (8, 4096), (16, 4096), (8, 2048)])
def test_fork_over_batch_and_width_sweep(B, H):
    g, ev, deps = _compile("fork", B, H)
    assert ev["xa"]["tasks"] == min(B, 148) and deps["xb"] == ["xa"] and deps["xc"] == ["xa"]


def test_more_than_three_independent_producers_is_refused_with_a_message():
    """The limit of this runtime's task record (three dependency slots) is reported at compile time with a message:
    a linear whose input, residual and WEIGHT come from three different layers and whose output buffer was written by
    a fourth needs four waits."""
    import torch
    params = mi.PersistentKernel.get_default_init_parameters()
    params.update(test_mode=True, num_workers=0, max_num_batched_tokens=4, max_num_batched_requests=4, dry_run=True)
    mk = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device="meta")

    def graph(with_fourth):
        pk = mi.PersistentKernel(**params)
        x, w = pk.attach_input(mk(4, 256), "x"), pk.attach_input(mk(256), "w")
        w0, w1, wl = pk.attach_input(mk(256, 256), "w0"), pk.attach_input(mk(256, 256), "w1"), pk.attach_input(mk(256, 256), "wl")
        a, b, out = pk.attach_input(mk(4, 256), "a"), pk.attach_input(mk(4, 256), "b"), pk.attach_input(mk(4, 256), "out")
        pk.rmsnorm_layer(input=x, weight=w, output=a, grid_dim=(4, 1, 1), block_dim=(128, 1, 1))
        pk.rmsnorm_layer(input=x, weight=w, output=b, grid_dim=(4, 1, 1), block_dim=(128, 1, 1))
        pk.elementwise_add_layer(input_a=w0, input_b=w1, output=wl, grid_dim=(4, 1, 1), block_dim=(128, 1, 1))
        if with_fourth:
            pk.rmsnorm_layer(input=x, weight=w, output=out, grid_dim=(4, 1, 1), block_dim=(128, 1, 1))
        pk.linear_with_residual_layer(input=a, weight=wl, residual=b, output=out, grid_dim=(4, 1, 1), block_dim=(128, 1, 1))
        return pk

    graph(False).compile()
    with pytest.raises(mi.MpkError) as e:
        graph(True).compile()
    assert "more than 3" in str(e.value)


def test_overlapping_views_of_one_allocation_are_ordered():
    """Two attached tensors that alias without sharing a base pointer (a row-offset view of a buffer) must share a
    storage: the layer that reads the view waits for the layer that wrote the buffer."""
    import ctypes as C
    from mirage_b200 import _native as N
    cfg = N.MpkConfig()
    cfg.test_mode, cfg.dry_run, cfg.world_size, cfg.num_workers = 1, 1, 1, 8
    cfg.max_num_batched_tokens = cfg.max_num_batched_requests = 4
    h = C.c_void_p()
    N.check(h, N.lib.mpk_create(C.byref(cfg), C.byref(h)))

    def attach(name, ptr, rows, cols):
        dims = (C.c_int64 * 2)(rows, cols)
        return N.check(h, N.lib.mpk_attach_tensor(h, name.encode(), C.c_void_p(ptr), N.BF16, 2, dims, None))

    base = 0x10000000
    x = attach("x", base + 0x100000, 4, 256)
    w = attach("w", base + 0x200000, 1, 256)
    buf = attach("buf", base, 8, 256)                       # rows 0..7
    view = attach("view", base + 4 * 256 * 2, 4, 256)       # rows 4..7 of the same memory
    out = attach("out", base + 0x300000, 4, 256)
    grid = (C.c_int * 3)(4, 1, 1)
    ids = lambda *v: (C.c_int * len(v))(*v)
    N.check(h, N.lib.mpk_add_layer(h, N.OP_RMSNORM, ids(x, w, buf), 3, grid, None, 0))       # writes rows 0..3 of buf
    N.check(h, N.lib.mpk_add_layer(h, N.OP_RMSNORM, ids(view, w, out), 3, grid, None, 0))    # reads the overlapping view
    N.check(h, N.lib.mpk_compile(h))
    n = N.lib.mpk_dump_task_graph(h, None, 0)
    b = C.create_string_buffer(int(n))
    N.lib.mpk_dump_task_graph(h, b, n)
    ev = json.loads(b.value.decode())["events"]
    assert [d[0] for d in ev[1]["deps"]] == [0]
    N.lib.mpk_destroy(h)


def test_expert_projection_refuses_misaligned_scale_tensors():
    """The FP8 expert projection copies scales and rows 16 bytes at a time: tensors that do not start on a 16-byte
    boundary are refused when the graph is compiled (an error return, not a device fault)."""
    import ctypes as C
    from mirage_b200 import _native as N
    E, topk, n, k, b = 4, 2, 256, 512, 4

    def build(scale_offset):
        cfg = N.MpkConfig()
        cfg.test_mode, cfg.dry_run, cfg.world_size, cfg.num_workers = 1, 1, 1, 4
        cfg.max_num_batched_tokens = cfg.max_num_batched_requests = b
        h = C.c_void_p()
        N.check(h, N.lib.mpk_create(C.byref(cfg), C.byref(h)))

        def attach(name, ptr, dtype, *shape):
            dims = (C.c_int64 * len(shape))(*shape)
            return N.check(h, N.lib.mpk_attach_tensor(h, name.encode(), C.c_void_p(ptr), dtype, len(shape), dims, None))

        base = 0x20000000
        t = [attach("xq", base, N.F8E4M3, b, k), attach("xs", base + 0x100000, N.F32, b, k // 128),
             attach("w", base + 0x200000, N.F8E4M3, E, n, k), attach("ws", base + 0x400000 + scale_offset, N.F32, E, n, k // 128),
             attach("idx", base + 0x500000, N.I32, E, b), attach("mask", base + 0x600000, N.I32, E + 1),
             attach("out", base + 0x700000, N.BF16, b, topk, n)]
        grid = (C.c_int * 3)(4, 1, 1)
        N.check(h, N.lib.mpk_add_layer(h, N.OP_MOE_W13_FP8, (C.c_int * 7)(*t), 7, grid, None, 0))
        try:
            N.check(h, N.lib.mpk_compile(h))
        finally:
            N.lib.mpk_destroy(h)

    build(0)
    with pytest.raises(N.MpkError, match="16-byte"):
        build(4)
