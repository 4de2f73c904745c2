"""GPU parity of the mixture-of-experts task bodies against the CPU oracle and the fixture generated from the
reference tests' oracle functions.  Routing indices and the active-expert list are compared bit-exactly, routing
weights to 1e-5, bf16 GEMM outputs within max relative error 2e-2 (1e-2 against the exact-product oracle)."""
import os

import pytest
import torch

from oracle import moe_ops as M
from oracle import fp8_ops as F8
from gpu_util import rel_err, make_test_kernel

pytestmark = pytest.mark.gpu
E4 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def mi():
    import mirage_b200
    return mirage_b200


def _route(mi, logits, bias, *, topk, groups, keep, scaling=2.5):
    b, e = logits.shape
    pk = make_test_kernel(mi, b)
    lg = logits.clone().cuda()
    w = torch.zeros(b, topk, dtype=torch.float32, device="cuda")
    idx = torch.full((e, b), 7, dtype=torch.int32, device="cuda")
    mask = torch.full((e + 1,), 9, dtype=torch.int32, device="cuda")
    pk.moe_topk_sigmoid_routing_layer(input=pk.attach_input(lg, "logits"), bias=pk.attach_input(bias.cuda(), "bias"),
                                      output=(pk.attach_input(w, "w"), pk.attach_input(idx, "idx"),
                                              pk.attach_input(mask, "mask")),
                                      grid_dim=(1, 1, 1), block_dim=(256, 1, 1), num_groups=groups, topk_group=keep,
                                      routed_scaling_factor=scaling)
    pk.compile()
    pk.run_test_mode()
    return w.cpu(), idx.cpu(), mask.cpu(), lg.cpu()


def _check_route(got, ref):
    w, idx, mask, lg = got
    rw, ridx, ract, _ = ref
    assert torch.equal(idx, ridx)
    assert torch.equal(mask, ract)
    torch.testing.assert_close(w, rw, rtol=1e-5, atol=1e-6)
    assert (lg.float() == 0).all()        # the task zeroes the logits for the accumulating gate projection


def test_sigmoid_routing_golden_fixture(mi, golden_dir):
    f = torch.load(os.path.join(golden_dir, "ref_moe.pt"), weights_only=False)
    c = f["route_consts"]
    w, idx, mask, _ = _route(mi, f["logits"], f["bias"], topk=c["NUM_EXPERTS_PER_TOK"], groups=c["NUM_GROUPS"],
                             keep=c["TOPK_GROUP"], scaling=c["ROUTED_SCALING_FACTOR"])
    assert torch.equal(idx, f["routing"])
    n = int(mask[-1])
    on = torch.zeros(c["NUM_EXPERTS"], dtype=torch.int32)
    on[mask[:n].long()] = 1
    assert torch.equal(on, f["expert_active"])
    torch.testing.assert_close(w, f["weights"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("b", [1, 8, 32, 64])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_sigmoid_routing_deepseek_shape(mi, b, dtype):
    g = torch.Generator().manual_seed(42 + b)
    logits = torch.randn(b, 256, generator=g).to(dtype)
    bias = torch.randn(256, generator=g) * 0.1
    ref = M.topk_sigmoid_routing(logits, bias, topk=8, num_groups=8, topk_group=4, scaling=2.5)
    _check_route(_route(mi, logits, bias, topk=8, groups=8, keep=4), ref)


@pytest.mark.parametrize("b,e,topk", [(1, 128, 8), (32, 256, 8), (64, 64, 4)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_softmax_routing(mi, b, e, topk, dtype):
    """moe_topk_softmax_routing_layer against the oracle (the expression of the reference's test_gate_topk.py): routing
    table and active list exact, weights to fp32 rounding; the logits stay as they were."""
    g = torch.Generator().manual_seed(b + e)
    logits = torch.randn(b, e, generator=g).to(dtype)
    w_ref, r_ref, a_ref, _ = M.topk_softmax_routing(logits, topk=topk)
    pk = make_test_kernel(mi, b)
    lg = logits.clone().cuda()
    w = torch.zeros(b, topk, dtype=torch.float32, device="cuda")
    idx = torch.full((e, b), 7, dtype=torch.int32, device="cuda")
    mask = torch.full((e + 1,), 7, dtype=torch.int32, device="cuda")
    pk.moe_topk_softmax_routing_layer(input=pk.attach_input(lg, "logits"),
                                      output=(pk.attach_input(w, "w"), pk.attach_input(idx, "idx"), pk.attach_input(mask, "mask")),
                                      grid_dim=(1, 1, 1), block_dim=(256, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert torch.equal(idx.cpu(), r_ref) and torch.equal(mask.cpu(), a_ref)
    assert torch.allclose(w.cpu(), w_ref, rtol=2e-6, atol=1e-8)
    assert torch.equal(lg.cpu(), logits)


def test_sigmoid_routing_ties_take_the_lower_index(mi):
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(6, 64, generator=g).to(torch.bfloat16)
    logits[:, 8:16] = logits[:, 0:8]
    logits[3] = 0.5                       # every score equal
    bias = torch.randn(64, generator=g) * 0.1
    bias[8:16] = bias[0:8]
    bias2 = bias.clone()
    ref = M.topk_sigmoid_routing(logits, bias2, topk=4, num_groups=8, topk_group=3, scaling=1.0)
    _check_route(_route(mi, logits, bias, topk=4, groups=8, keep=3, scaling=1.0), ref)


def _random_routing(e, b, topk, seed):
    g = torch.Generator().manual_seed(seed)
    routing = torch.zeros(e, b, dtype=torch.int32)
    for tok in range(b):
        ex = torch.randperm(e, generator=g)[:topk]
        for slot, x in enumerate(ex.tolist()):
            routing[x, tok] = slot + 1
    act = (routing != 0).any(1).nonzero().reshape(-1).to(torch.int32)
    mask = torch.full((e + 1,), -1, dtype=torch.int32)
    mask[:act.numel()] = act
    mask[e] = act.numel()
    return routing, mask


def _run_moe_gemm(mi, x, xs, w, ws, routing, mask, topk, per_slot, first_expert=0):
    b = routing.shape[1]
    n = w.shape[1]
    pk = make_test_kernel(mi, b)
    out = torch.zeros(b, topk, n, dtype=torch.bfloat16, device="cuda")
    args = dict(moe_routing_indices=pk.attach_input(routing.cuda(), "routing"),
                moe_mask=pk.attach_input(mask.cuda(), "mask"), output=pk.attach_input(out, "out"),
                grid_dim=(1, 1, 1), block_dim=(128, 1, 1), first_expert=first_expert)
    if xs is None:
        fn = pk.moe_w2_linear_layer if per_slot else pk.moe_w13_linear_layer
        fn(input=pk.attach_input(x.cuda(), "x"), weight=pk.attach_input(w.cuda(), "w"), **args)
    else:
        fn = pk.moe_w2_fp8_layer if per_slot else pk.moe_w13_fp8_layer
        fn(input_fp8=pk.attach_input(x.cuda(), "x"), input_scale=pk.attach_input(xs.cuda(), "xs"),
           weight_fp8=pk.attach_input(w.cuda(), "w"), weight_scale=pk.attach_input(ws.cuda(), "ws"), **args)
    pk.compile()
    pk.run_test_mode()
    first = out.clone()
    pk.run_test_mode()
    assert torch.equal(first, out)
    return out.cpu()


def test_moe_fp8_gemm_golden_fixture(mi, golden_dir):
    f = torch.load(os.path.join(golden_dir, "ref_moe.pt"), weights_only=False)
    r = f["g_routing"]
    act = (r != 0).any(1).nonzero().reshape(-1).to(torch.int32)
    mask = torch.full((7,), -1, dtype=torch.int32)
    mask[:act.numel()] = act
    mask[6] = act.numel()
    out13 = _run_moe_gemm(mi, f["x13q"].view(E4), f["x13s"], f["w13q"].view(E4), f["w13s"], r, mask, 2, False)
    out2 = _run_moe_gemm(mi, f["x2q"].view(E4), f["x2s"], f["w2q"].view(E4), f["w2s"], r, mask, 2, True)
    assert rel_err(out13, f["out13"]) <= 2e-2
    assert rel_err(out2, f["out2"]) <= 2e-2


@pytest.mark.parametrize("b,e,topk,n,k,per_slot", [(1, 16, 4, 256, 1024, False), (16, 32, 4, 512, 7168, False),
                                                   (8, 32, 8, 1024, 2048, True), (64, 16, 2, 384, 1024, True),
                                                   (33, 8, 2, 2048, 512, False)])
def test_moe_fp8_gemm_shapes(mi, b, e, topk, n, k, per_slot):
    g = torch.Generator().manual_seed(b + e + n)
    routing, mask = _random_routing(e, b, topk, seed=b * 7 + e)
    x = torch.randn(*((b, topk, k) if per_slot else (b, k)), generator=g).to(torch.bfloat16)
    x[..., :128] *= 20.0
    w = (0.05 * torch.randn(e, n, k, generator=g)).to(torch.bfloat16)
    xq, xs = M.quantize_fp8_f32(x)
    wq, ws = M.quantize_fp8_f32(w)
    ref = M.moe_gemm_fp8(xq, xs, wq, ws, routing, topk=topk, per_slot_input=per_slot)
    out = _run_moe_gemm(mi, xq, xs, wq, ws, routing, mask, topk, per_slot)
    assert rel_err(out, ref) <= 1e-2


@pytest.mark.parametrize("b", [4, 32])
def test_moe_fp8_gemm_on_a_slice_of_the_experts(mi, b):
    """Expert parallelism: the weight tensor holds experts [8, 16) of 16; the routing table and the active list name
    only those (what the routing task writes when given that local range).  Slots of the other experts stay untouched."""
    e, topk, n, k, lo, hi = 16, 4, 512, 1024, 8, 16
    g = torch.Generator().manual_seed(31 + b)
    routing, _ = _random_routing(e, b, topk, seed=b)
    routing[:lo] = 0
    act = (routing != 0).any(1).nonzero().reshape(-1).to(torch.int32)
    mask = torch.full((e + 1,), -1, dtype=torch.int32)
    mask[:act.numel()] = act
    mask[e] = act.numel()
    x = torch.randn(b, k, generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(e, n, k, generator=g)).to(torch.bfloat16)
    xq, xs = M.quantize_fp8_f32(x)
    wq, ws = M.quantize_fp8_f32(w)
    ref = M.moe_gemm_fp8(xq, xs, wq, ws, routing, topk=topk, per_slot_input=False)
    out = _run_moe_gemm(mi, xq, xs, wq[lo:hi].contiguous(), ws[lo:hi].contiguous(), routing, mask, topk, False, first_expert=lo)
    assert rel_err(out, ref) <= 1e-2


@pytest.mark.parametrize("b,e,topk,n,k,per_slot", [(4, 8, 2, 512, 1024, False), (16, 16, 4, 256, 768, True)])
def test_moe_bf16_gemm_shapes(mi, b, e, topk, n, k, per_slot):
    g = torch.Generator().manual_seed(b + e + n + 1)
    routing, mask = _random_routing(e, b, topk, seed=b * 3 + e)
    x = torch.randn(*((b, topk, k) if per_slot else (b, k)), generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(e, n, k, generator=g)).to(torch.bfloat16)
    ref = M.moe_gemm_bf16(x, w, routing, topk=topk, per_slot_input=per_slot)
    out = _run_moe_gemm(mi, x, None, w, None, routing, mask, topk, per_slot)
    assert rel_err(out, ref) <= 2e-2


def test_moe_silu_mul_and_weighted_sum(mi):
    b, topk, i, h = 6, 4, 512, 1024
    g = torch.Generator().manual_seed(9)
    mid = torch.randn(b, topk, 2 * i, generator=g).to(torch.bfloat16)
    down = torch.randn(b, topk, h, generator=g).to(torch.bfloat16)
    wts = torch.rand(b, topk, generator=g)
    res = torch.randn(b, h, generator=g).to(torch.bfloat16)
    pk = make_test_kernel(mi, b)
    act = torch.zeros(b, topk, i, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(b, h, dtype=torch.bfloat16, device="cuda")
    pk.moe_silu_mul_layer(input=pk.attach_input(mid.cuda(), "mid"), output=pk.attach_input(act, "act"),
                          grid_dim=(b, topk, 1), block_dim=(128, 1, 1))
    pk.moe_mul_sum_add_layer(input=pk.attach_input(down.cuda(), "down"), weight=pk.attach_input(wts.cuda(), "wts"),
                             residual=pk.attach_input(res.cuda(), "res"), output=pk.attach_input(y, "y"),
                             grid_dim=(b, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert rel_err(act.cpu(), M.moe_silu_mul(mid)) <= 1e-2
    assert rel_err(y.cpu(), M.moe_mul_sum_add(down, wts, res)) <= 1e-2


def test_moe_block_in_one_graph(mi):
    """router logits -> routing -> quantize -> W13 (fp8) -> silu-mul -> quantize -> W2 (fp8) -> weighted sum +
    residual: the routed-expert half of a DeepSeek-V3 layer (python/mirage/mpk/models/deepseek_v3/builder.py:
    880-1075 of the reference), reduced sizes."""
    b, e, topk, hdim, inter = 8, 32, 4, 1024, 256
    g = torch.Generator().manual_seed(21)
    x = torch.randn(b, hdim, generator=g).to(torch.bfloat16)
    logits = torch.randn(b, e, generator=g).to(torch.bfloat16)
    bias = torch.randn(e, generator=g) * 0.1
    w13 = (0.05 * torch.randn(e, 2 * inter, hdim, generator=g)).to(torch.bfloat16)
    w2 = (0.05 * torch.randn(e, hdim, inter, generator=g)).to(torch.bfloat16)
    w13q, w13s = M.quantize_fp8_f32(w13)
    w2q, w2s = M.quantize_fp8_f32(w2)
    # oracle chain
    rw, ridx, ract, _ = M.topk_sigmoid_routing(logits, bias, topk=topk, num_groups=8, topk_group=4, scaling=2.5)
    xq, xs = F8.quantize_fp8_f32scale(x)
    mid = M.moe_gemm_fp8(xq, xs, w13q, w13s, ridx, topk=topk, per_slot_input=False)
    act = M.moe_silu_mul(mid)
    aq, asc = F8.quantize_fp8_f32scale(act.reshape(b * topk, inter))
    down = M.moe_gemm_fp8(aq.reshape(b, topk, inter), asc.reshape(b, topk, -1), w2q, w2s, ridx, topk=topk,
                          per_slot_input=True)
    ref = M.moe_mul_sum_add(down, rw, x)
    # megakernel graph
    pk = make_test_kernel(mi, b)
    nt = lambda dims, dt, name: pk.new_tensor(dims=dims, dtype=dt, name=name, io_category="cuda_tensor")
    t_x = pk.attach_input(x.cuda(), "x")
    t_w = nt((b, topk), mi.float32, "topk_w")
    t_idx = nt((e, b), mi.int32, "routing")
    t_mask = nt((e + 1,), mi.int32, "mask")
    t_xq, t_xs = nt((b, hdim), mi.float8_e4m3, "xq"), nt((b, hdim // 128), mi.float32, "xs")
    t_mid = nt((b, topk, 2 * inter), mi.bfloat16, "mid")
    t_act = nt((b, topk, inter), mi.bfloat16, "act")
    t_aq, t_as = nt((b, topk, inter), mi.float8_e4m3, "aq"), nt((b, topk, inter // 128), mi.float32, "as")
    t_down = nt((b, topk, hdim), mi.bfloat16, "down")
    y = torch.zeros(b, hdim, dtype=torch.bfloat16, device="cuda")
    pk.moe_topk_sigmoid_routing_layer(input=pk.attach_input(logits.cuda(), "logits"),
                                      bias=pk.attach_input(bias.cuda(), "bias"), output=(t_w, t_idx, t_mask),
                                      grid_dim=(1, 1, 1), block_dim=(256, 1, 1))
    pk.quantize_fp8_layer(input=t_x, output_fp8=t_xq, output_scale=t_xs, grid_dim=(b, 1, 1), block_dim=(128, 1, 1),
                          scale_ue8m0=False)
    pk.moe_w13_fp8_layer(input_fp8=t_xq, input_scale=t_xs, weight_fp8=pk.attach_input(w13q.cuda(), "w13"),
                         weight_scale=pk.attach_input(w13s.cuda(), "w13s"), moe_routing_indices=t_idx, moe_mask=t_mask,
                         output=t_mid, grid_dim=(16, 1, 1), block_dim=(128, 1, 1))
    pk.moe_silu_mul_layer(input=t_mid, output=t_act, grid_dim=(b, topk, 1), block_dim=(128, 1, 1))
    pk.quantize_fp8_layer(input=t_act, output_fp8=t_aq, output_scale=t_as, grid_dim=(b * topk, 1, 1),
                          block_dim=(128, 1, 1), scale_ue8m0=False)
    pk.moe_w2_fp8_layer(input_fp8=t_aq, input_scale=t_as, weight_fp8=pk.attach_input(w2q.cuda(), "w2"),
                        weight_scale=pk.attach_input(w2s.cuda(), "w2s"), moe_routing_indices=t_idx, moe_mask=t_mask,
                        output=t_down, grid_dim=(16, 1, 1), block_dim=(128, 1, 1))
    pk.moe_mul_sum_add_layer(input=t_down, weight=t_w, residual=t_x, output=pk.attach_input(y, "y"),
                             grid_dim=(b, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert torch.equal(pk.tensor_as_torch(t_idx).cpu(), ridx)
    assert rel_err(y.cpu(), ref) <= 2e-2
