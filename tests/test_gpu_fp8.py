"""GPU parity of the FP8 task bodies (per-token group quantisation, block-scaled e4m3 linear) against the
CPU oracle and the fixture generated from the reference's helper module.  Quantised bytes and scale
exponents are compared bit-exactly; bf16 linear outputs within max relative error 1e-2."""
import os

import numpy as np
import pytest
import torch

from oracle import fp8_ops as F
from gpu_util import rel_err, make_test_kernel

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def mi():
    import mirage_b200
    return mirage_b200


def _u32(t: torch.Tensor) -> torch.Tensor:
    """int64 tensor holding uint32 values -> torch.uint32 tensor."""
    return torch.from_numpy(t.numpy().astype(np.uint32)).view(torch.uint32)


def _acts(b, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(b, k, generator=g)
    # groups of very different magnitude, one all-zero group, one exact power of two maximum
    x[:, :128] *= 37.0
    if k >= 384:
        x[:, 128:256] *= 1e-3
        x[0, 256:384] = 0.0
    x[-1, 5] = 224.0 * 8
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("b,k", [(1, 512), (5, 7168), (16, 1536), (64, 1024)])
def test_quantize_fp8_packed_ue8m0_bit_exact(mi, b, k):
    x = _acts(b, k, seed=b * 1000 + k)
    q_ref, exps_ref, packed_ref = F.quantize_fp8_ue8m0(x)
    pk_k = (k // 128 + 3) // 4
    aligned = (b + 3) // 4 * 4
    pk = make_test_kernel(mi, b)
    q = torch.zeros(b, k, dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.zeros(pk_k, aligned, dtype=torch.int32, device="cuda").view(torch.uint32)   # column-major scales
    pk.quantize_fp8_layer(input=pk.attach_input(x.cuda(), "x"), output_fp8=pk.attach_input(q, "q"),
                          output_scale=pk.attach_input(s, "s"), grid_dim=(b, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    got = s.view(torch.int32).cpu().to(torch.int64) & 0xFFFFFFFF
    assert torch.equal(got[:, :b].T.contiguous(), packed_ref)
    assert torch.equal(F.unpack_ue8m0(got[:, :b].T.contiguous(), k // 128), exps_ref)


@pytest.mark.parametrize("shape", [(3, 2048), (4, 8, 256)])
def test_quantize_fp8_float_scale_bit_exact(mi, shape):
    k = shape[-1]
    rows = int(np.prod(shape[:-1]))
    x = _acts(rows, k, seed=7 + rows).reshape(shape)
    q_ref, s_ref = F.quantize_fp8_f32scale(x.reshape(rows, k))
    pk = make_test_kernel(mi, shape[0])
    q = torch.zeros(*shape, dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.zeros(*shape[:-1], k // 128, dtype=torch.float32, device="cuda")
    pk.quantize_fp8_layer(input=pk.attach_input(x.cuda(), "x"), output_fp8=pk.attach_input(q, "q"),
                          output_scale=pk.attach_input(s, "s"), grid_dim=(rows, 1, 1), block_dim=(128, 1, 1),
                          scale_ue8m0=False)
    pk.compile()
    pk.run_test_mode()
    assert torch.equal(q.cpu().view(torch.uint8).reshape(rows, k), q_ref.view(torch.uint8))
    assert torch.equal(s.cpu().reshape(rows, -1), s_ref)


def _run_linear_fp8(mi, xq, xs_packed, wq, ws_packed, residual, *, col_major_x_scale=True):
    b, k = xq.shape
    n = wq.shape[0]
    pk = make_test_kernel(mi, b)
    out = torch.zeros(b, n, dtype=torch.bfloat16, device="cuda")
    if col_major_x_scale:
        aligned = (b + 3) // 4 * 4
        phys = torch.zeros(xs_packed.shape[1], aligned, dtype=torch.int64)
        phys[:, :b] = xs_packed.T
        xs_dev = _u32(phys).cuda()
    else:
        xs_dev = _u32(xs_packed).cuda()
    t = dict(input_fp8=pk.attach_input(xq.cuda(), "xq"), input_scale=pk.attach_input(xs_dev, "xs"),
             weight_fp8=pk.attach_input(wq.cuda(), "wq"), weight_scale=pk.attach_input(_u32(ws_packed).cuda(), "ws"),
             output=pk.attach_input(out, "out"), grid_dim=(max(n // 128, 1), 1, 1), block_dim=(128, 1, 1))
    if residual is None:
        pk.linear_fp8_layer(**t)
    else:
        pk.linear_fp8_with_residual_layer(residual=pk.attach_input(residual.cuda(), "res"), **t)
    pk.compile()
    pk.run_test_mode()
    first = out.clone()
    pk.run_test_mode()
    assert torch.equal(first, out)
    return out.cpu()


def test_linear_fp8_golden_fixture(mi, golden_dir):
    f = torch.load(os.path.join(golden_dir, "ref_fp8.pt"), weights_only=False)
    xq = f["xq"].view(torch.float8_e4m3fn)
    wq = f["wq"].view(torch.float8_e4m3fn)
    out = _run_linear_fp8(mi, xq, f["xs"], wq, f["ws"], f["residual"], col_major_x_scale=False)
    assert rel_err(out, f["out"]) <= TOL


@pytest.mark.parametrize("b,n,k,res", [(1, 128, 768, False), (1, 2112, 7168, True), (8, 1536, 1536, False),
                                       (4, 7168, 2048, True), (16, 512, 7168, True), (33, 384, 1024, False),
                                       (64, 1024, 16384, True)])
def test_linear_fp8_shapes(mi, b, n, k, res):
    g = torch.Generator().manual_seed(n + k + b)
    x = _acts(b, k, seed=b + k)
    w = (0.05 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    w[:, 128:256] *= 30.0
    xq, xe, xp = F.quantize_fp8_ue8m0(x)
    wq, we, wp = F.quantize_fp8_ue8m0(w)
    residual = torch.randn(b, n, generator=g).to(torch.bfloat16) if res else None
    ref = F.linear_fp8(xq, xe, wq, we, residual)
    out = _run_linear_fp8(mi, xq, xp, wq, wp, residual)
    assert rel_err(out, ref) <= TOL


def test_quantize_then_linear_fp8_in_one_graph(mi):
    """bf16 activations -> quantize task -> FP8 linear with residual, as the reference's builders chain them
    (python/mirage/mpk/models/deepseek_v3/builder.py:118-207)."""
    b, n, k = 8, 2048, 7168
    g = torch.Generator().manual_seed(3)
    x = _acts(b, k, seed=11)
    w = (0.03 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    residual = torch.randn(b, n, generator=g).to(torch.bfloat16)
    wq, we, wp = F.quantize_fp8_ue8m0(w)
    xq, xe, _ = F.quantize_fp8_ue8m0(x)
    ref = F.linear_fp8(xq, xe, wq, we, residual)
    pk = make_test_kernel(mi, b)
    out = torch.zeros(b, n, dtype=torch.bfloat16, device="cuda")
    fp8_buf = pk.new_tensor(dims=(b, k), dtype=mi.float8_e4m3, name="fp8_in", io_category="cuda_tensor")
    sc_buf = pk.new_tensor(dims=((k // 128 + 3) // 4, (b + 3) // 4 * 4), dtype=mi.uint32, name="fp8_scale",
                           io_category="cuda_tensor")
    pk.quantize_fp8_layer(input=pk.attach_input(x.cuda(), "x"), output_fp8=fp8_buf, output_scale=sc_buf,
                          grid_dim=(b, 1, 1), block_dim=(128, 1, 1))
    pk.linear_fp8_with_residual_layer(input_fp8=fp8_buf, input_scale=sc_buf, weight_fp8=pk.attach_input(wq.cuda(), "wq"),
                                      weight_scale=pk.attach_input(_u32(wp).cuda(), "ws"),
                                      residual=pk.attach_input(residual.cuda(), "res"),
                                      output=pk.attach_input(out, "out"), grid_dim=(16, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert rel_err(out.cpu(), ref) <= TOL
