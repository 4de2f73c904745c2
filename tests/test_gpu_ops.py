"""GPU parity of single task bodies, run through PersistentKernel test mode (one launch of the task
graph), against the CPU oracle and the golden fixtures.  Tolerances: bf16 outputs within max relative
error 2e-2."""
import os

import pytest
import torch

from oracle import mpk_ops as ops
from gpu_util import rel_err, make_test_kernel

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def mi():
    import mirage_b200
    return mirage_b200


def _bf16(*shape, seed, scale=1.0, shift=0.0):
    g = torch.Generator().manual_seed(seed)
    return (shift + scale * torch.randn(*shape, generator=g)).to(torch.bfloat16)


def test_rmsnorm_linear_baseline_config1(mi):
    """x[8,4096] ~ N(0,1), g = 1 + N(0,0.02), W[6144,4096] ~ N(0,0.02), eps 1e-6, seed 0."""
    torch.manual_seed(0)
    x = torch.randn(8, 4096).to(torch.bfloat16)
    g = (1 + 0.02 * torch.randn(4096)).to(torch.bfloat16)
    w = (0.02 * torch.randn(6144, 4096)).to(torch.bfloat16)
    ref = ops.rmsnorm_linear(x, g, w, 1e-6)
    pk = make_test_kernel(mi, 8)
    out = torch.zeros(8, 6144, dtype=torch.bfloat16, device="cuda")
    tx, tg = pk.attach_input(x.cuda(), "x"), pk.attach_input(g.cuda(), "g")
    tw, to = pk.attach_input(w.cuda(), "w"), pk.attach_input(out, "out")
    pk.rmsnorm_linear_layer(input=tx, weight_norm=tg, weight_linear=tw, output=to, grid_dim=(96, 1, 1),
                            block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert rel_err(out.cpu(), ref) <= TOL
    # a second launch gives bit-identical results (monotonic counters, no state left behind)
    first = out.clone()
    pk.run_test_mode()
    assert torch.equal(first, out)


def test_rmsnorm_linear_golden_fixture(mi, golden_dir):
    f = torch.load(os.path.join(golden_dir, "ref_norm_linear.pt"), weights_only=False)
    x, g, w = f["x"], f["g"].reshape(-1), f["w"]
    pk = make_test_kernel(mi, x.shape[0])
    out = torch.zeros(x.shape[0], w.shape[0], dtype=torch.bfloat16, device="cuda")
    pk.rmsnorm_linear_layer(input=pk.attach_input(x.cuda(), "x"), weight_norm=pk.attach_input(g.cuda(), "g"),
                            weight_linear=pk.attach_input(w.cuda(), "w"), output=pk.attach_input(out, "o"),
                            grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert rel_err(out.cpu(), f["out_f32"]) <= TOL


@pytest.mark.parametrize("B,N,K", [(1, 4096, 4096), (1, 4096, 12288), (2, 1000, 512), (3, 6144, 4096),
                                   (4, 520, 1536), (8, 777, 2048), (1, 37, 64), (5, 300, 6144),
                                   (16, 520, 4096), (33, 300, 1536), (64, 256, 12288), (64, 777, 512),
                                   (9, 96, 256)])
def test_linear_with_residual_shapes(mi, B, N, K):
    x = _bf16(B, K, seed=1)
    w = _bf16(N, K, seed=2, scale=0.02)
    r = _bf16(B, N, seed=3)
    ref = ops.linear(x, w, r)
    ref_plain = ops.linear(x, w)
    pk = make_test_kernel(mi, B)
    o1 = torch.zeros(B, N, dtype=torch.bfloat16, device="cuda")
    o2 = torch.zeros(B, N, dtype=torch.bfloat16, device="cuda")
    o3 = r.clone().cuda()
    tx, tw = pk.attach_input(x.cuda(), "x"), pk.attach_input(w.cuda(), "w")
    pk.linear_with_residual_layer(input=tx, weight=tw, residual=pk.attach_input(r.cuda(), "r"),
                                  output=pk.attach_input(o1, "o1"), grid_dim=(64, 1, 1), block_dim=(128, 1, 1))
    pk.linear_layer(input=tx, weight=tw, output=pk.attach_input(o2, "o2"), grid_dim=(64, 1, 1), block_dim=(128, 1, 1))
    pk.splitk_linear_layer(input=tx, weight=tw, output=pk.attach_input(o3, "o3"), grid_dim=(32, 4, 1),
                           block_dim=(256, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert rel_err(o1.cpu(), ref) <= TOL
    assert rel_err(o2.cpu(), ref_plain) <= TOL
    assert rel_err(o3.cpu(), ref) <= TOL      # split-K semantics: output += x W^T


@pytest.mark.parametrize("B", [16, 40, 64])
def test_rmsnorm_linear_large_batches(mi, B):
    """More than one tile of 8 tokens: token tiles are spread over the compute warps; at 64 tokens the norm can
    no longer be folded (the activation tile does not hold whole rows) and runs as its own task."""
    x = _bf16(B, 4096, seed=21)
    g = _bf16(4096, seed=22, scale=0.02, shift=1.0)
    w = _bf16(640, 4096, seed=23, scale=0.02)
    ref = ops.rmsnorm_linear(x, g, w, 1e-6)
    pk = make_test_kernel(mi, B)
    out = torch.zeros(B, 640, dtype=torch.bfloat16, device="cuda")
    normed = pk.new_tensor((B, 4096), name="normed")
    tx, tg, tw = pk.attach_input(x.cuda(), "x"), pk.attach_input(g.cuda(), "g"), pk.attach_input(w.cuda(), "w")
    pk.rmsnorm_layer(input=tx, weight=tg, output=normed, grid_dim=(B, 1, 1), block_dim=(128, 1, 1))
    pk.linear_layer(input=normed, weight=tw, output=pk.attach_input(out, "out"), grid_dim=(10, 1, 1),
                    block_dim=(128, 1, 1))
    pk.compile()
    assert pk.graph_info()["num_folded"] == (1 if B <= 16 else 0)
    pk.run_test_mode()
    assert rel_err(out.cpu(), ref) <= TOL


def test_mlp_pipeline_golden_fixture(mi, golden_dir):
    """gate_up (interleaved) -> silu_mul -> down + residual, the graph of the reference's
    test_qwen3_mlp_testmode.py, against the fixture its reference code produced."""
    f = torch.load(os.path.join(golden_dir, "ref_mlp.pt"), weights_only=False)
    x, res = f["x"], f["residual"]
    B, H = x.shape
    I = f["w_gate"].shape[0]
    groups = 4
    for fold in (True, False):
        pk = make_test_kernel(mi, B)
        tx = pk.attach_input(x.cuda(), "x")
        wg, wu = pk.attach_input(f["w_gate"].cuda(), "wg"), pk.attach_input(f["w_up"].cuda(), "wu")
        wgu = pk.shuffle_tensors([wg, wu], 0, groups, name="wgu")
        if fold:
            mid = pk.new_tensor((B, 2 * I), name="mid")
            act = pk.new_tensor((B, I), name="act")
        else:   # caller-visible intermediates stay materialised and are produced by stand-alone tasks
            mid_t = torch.zeros(B, 2 * I, dtype=torch.bfloat16, device="cuda")
            act_t = torch.zeros(B, I, dtype=torch.bfloat16, device="cuda")
            mid, act = pk.attach_input(mid_t, "mid"), pk.attach_input(act_t, "act")
        out = torch.zeros(B, H, dtype=torch.bfloat16, device="cuda")
        pk.linear_layer(input=tx, weight=wgu, output=mid, grid_dim=(2 * groups, 1, 1), block_dim=(128, 1, 1))
        pk.silu_mul_layer(input=mid, output=act, grid_dim=(groups, 1, 1), block_dim=(128, 1, 1))
        pk.linear_with_residual_layer(input=act, weight=pk.attach_input(f["w_down"].cuda(), "wd"),
                                      residual=pk.attach_input(res.cuda(), "res"), output=pk.attach_input(out, "out"),
                                      grid_dim=(H // 64, 1, 1), block_dim=(128, 1, 1))
        pk.compile()
        assert pk.graph_info()["num_folded"] == (1 if fold else 0)
        pk.run_test_mode()
        assert rel_err(out.cpu(), f["out"]) <= TOL
        if not fold:
            mid_ref = ops.linear(x, ops.shuffle_rows([f["w_gate"], f["w_up"]], groups))
            assert rel_err(mid_t.cpu(), mid_ref) <= TOL
            assert rel_err(act_t.cpu(), ops.silu_mul(mid_ref, groups)) <= TOL


def test_rmsnorm_layer_golden_fixture(mi, golden_dir):
    f = torch.load(os.path.join(golden_dir, "ref_rmsnorm.pt"), weights_only=False)
    x, w = f["x"], f["w"]
    pk = make_test_kernel(mi, x.shape[0])
    out = torch.zeros_like(x, device="cuda")
    pk.rmsnorm_layer(input=pk.attach_input(x.cuda(), "x"), weight=pk.attach_input(w.cuda(), "w"),
                     output=pk.attach_input(out, "o"), grid_dim=(x.shape[0], 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert rel_err(out.cpu(), f["out"]) <= TOL
    assert rel_err(out.cpu(), ops.rmsnorm(x, w, 1e-6)) <= 1e-2


def test_embedding_and_argmax(mi):
    V, H, B = 1000, 256, 4
    tab = _bf16(V, H, seed=5)
    ids = torch.tensor([[3], [999], [-1], [0]], dtype=torch.int64)
    logits = _bf16(B, V, seed=6)
    logits[1, 10] = logits[1, 700] = 9.0      # tie: lowest index must win
    pk = make_test_kernel(mi, B)
    out = torch.zeros(B, H, dtype=torch.bfloat16, device="cuda")
    tok = torch.zeros(B, 1, dtype=torch.int64, device="cuda")
    pk.embed_layer(input=pk.attach_input(ids.cuda(), "ids"), weight=pk.attach_input(tab.cuda(), "tab"),
                   output=pk.attach_input(out, "out"), grid_dim=(1, 1, 1), block_dim=(128, 1, 1), input_source=1)
    nparts = 7
    pv = pk.new_tensor((B, nparts), name="pv")
    pi = pk.new_tensor((B, nparts), dtype=mi.int64, name="pi")
    pk.argmax_partial_layer(input=pk.attach_input(logits.cuda(), "logits"), output=(pv, pi),
                            grid_dim=(nparts, 1, 1), block_dim=(128, 1, 1))
    pk.argmax_reduce_layer(input=(pv, pi), output=pk.attach_input(tok, "tok"), grid_dim=(1, 1, 1),
                           block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert torch.equal(out.cpu(), ops.embedding(ids, tab))
    assert tok.cpu().reshape(-1).tolist() == ops.argmax(logits).tolist()
    assert tok[1, 0].item() == 10


@pytest.mark.parametrize("token_budget", [0, 16])
@pytest.mark.parametrize("n_new,prefix,pages", [(3, 40, [2]), (1, 200, [1, 3, 0, 2]), (1, 63, [0]), (4, 124, [3, 1])])
def test_paged_attention(mi, golden_dir, n_new, prefix, pages, token_budget):
    """Fused QK-norm + RoPE + KV append + split-KV attention for one request; the (3, 40, [2]) case is
    the reference fixture (torch_multitoken_paged_attention).  A token budget of 16 selects the instantiation of
    the megakernel that serves many requests, whose attention tasks stream the cached rows through shared memory."""
    D, G, P = 128, 4, 64
    if (n_new, prefix) == (3, 40):
        f = torch.load(os.path.join(golden_dir, "ref_paged_attention.pt"), weights_only=False)
        qkv, kc, vc = f["qkv"], f["k_cache"].clone().unsqueeze(2), f["v_cache"].clone().unsqueeze(2)
        cos, sin, qn, kn = f["cos"], f["sin"], f["q_norm"].reshape(-1), f["k_norm"].reshape(-1)
    else:
        f = None
        qkv = _bf16(n_new, (G + 2) * D, seed=11)
        kc, vc = _bf16(4, P, 1, D, seed=12), _bf16(4, P, 1, D, seed=13)
        cos, sin = ops.rope_tables(D, 512, 1e6)
        qn, kn = _bf16(D, seed=14, scale=0.1, shift=1.0), _bf16(D, seed=15, scale=0.1, shift=1.0)
    seq_len = prefix + n_new
    assert len(pages) == (seq_len + P - 1) // P
    kc_ref, vc_ref = kc.clone(), vc.clone()
    ref = ops.paged_attention_request(qkv, kc_ref, vc_ref, pages, seq_len, G, 1, qn, kn, cos, sin, 1e-6)
    dev = "cuda"
    meta = {
        "qo_indptr_buffer": torch.tensor([0, n_new], dtype=torch.int32, device=dev),
        "paged_kv_indptr_buffer": torch.tensor([0, len(pages)], dtype=torch.int32, device=dev),
        "paged_kv_indices_buffer": torch.tensor(pages + [0] * (4 - len(pages)), dtype=torch.int32, device=dev),
        "paged_kv_last_page_len_buffer": torch.tensor([(seq_len - 1) % P + 1], dtype=torch.int32, device=dev),
    }
    pk = make_test_kernel(mi, max(n_new, token_budget), max_num_batched_requests=1, max_num_pages=4, page_size=P,
                          max_seq_length=256, meta_tensors=meta)
    kc_d, vc_d = kc.cuda(), vc.cuda()
    out = torch.zeros(n_new, G * D, dtype=torch.bfloat16, device=dev)
    pk.paged_attention_layer(
        input=pk.attach_input(qkv.cuda(), "qkv"), k_cache=pk.attach_input(kc_d, "kc"), v_cache=pk.attach_input(vc_d, "vc"),
        q_norm=pk.attach_input(qn.cuda(), "qn"), k_norm=pk.attach_input(kn.cuda(), "kn"),
        cos_pos_embed=pk.attach_input(cos.cuda(), "cos"), sin_pos_embed=pk.attach_input(sin.cuda(), "sin"),
        output=pk.attach_input(out, "out"), grid_dim=(1, 1, 1), block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    assert rel_err(out.cpu(), ref) <= TOL
    assert rel_err(kc_d.cpu(), kc_ref) <= 1e-2 and torch.equal(vc_d.cpu(), vc_ref)
    if f is not None:
        assert rel_err(out.cpu().reshape(n_new * G, D), f["out"]) <= TOL


@pytest.mark.parametrize("token_budget", [0, 16])
@pytest.mark.parametrize("lens,new,hkv,max_seq", [([3000, 257], [1, 2], 2, 4096), ([4096], [1], 8, 4096),
                                                  ([700, 64, 1, 2049, 65], [1, 3, 1, 2, 1], 1, 4096)])
def test_paged_attention_long_context(mi, lens, new, hkv, max_seq, token_budget):
    """Long sequences: chunks are longer than the rows a task fetches ahead of its dependency, so the per-row loop,
    many pages per request and the merge of the maximum number of chunks are exercised; two requests of very
    different lengths share the launch in the first case."""
    D, G, P = 128, 4, 64
    R, mbt = len(lens), sum(new)
    total_pages = sum((n + P - 1) // P for n in lens) + 3
    g = torch.Generator().manual_seed(sum(lens))
    qkv = (torch.randn(mbt, hkv * (G + 2) * D, generator=g)).to(torch.bfloat16)
    kc = torch.randn(total_pages, P, hkv, D, generator=g).to(torch.bfloat16)
    vc = torch.randn(total_pages, P, hkv, D, generator=g).to(torch.bfloat16)
    cos, sin = ops.rope_tables(D, max_seq, 1e6)
    qn, kn = _bf16(D, seed=14, scale=0.1, shift=1.0), _bf16(D, seed=15, scale=0.1, shift=1.0)
    perm = torch.randperm(total_pages, generator=g).tolist()
    indptr, indices, last, qo = [0], [], [], [0]
    for n, nn in zip(lens, new):
        k = (n + P - 1) // P
        indices += perm[indptr[-1]:indptr[-1] + k]
        indptr.append(indptr[-1] + k)
        last.append((n - 1) % P + 1)
        qo.append(qo[-1] + nn)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    ref = torch.cat([ops.paged_attention_request(qkv[qo[r]:qo[r + 1]], kc_ref, vc_ref, indices[indptr[r]:indptr[r + 1]],
                                                 lens[r], hkv * G, hkv, qn, kn, cos, sin, 1e-6) for r in range(R)])
    dev = "cuda"
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    meta = {"qo_indptr_buffer": i32(qo), "paged_kv_indptr_buffer": i32(indptr),
            "paged_kv_indices_buffer": i32(indices + [0] * (total_pages - len(indices))),
            "paged_kv_last_page_len_buffer": i32(last)}
    pk = make_test_kernel(mi, max(mbt, token_budget), max_num_batched_requests=R, max_num_pages=total_pages, page_size=P,
                          max_seq_length=max_seq, meta_tensors=meta)
    kc_d, vc_d = kc.cuda(), vc.cuda()
    out = torch.zeros(mbt, hkv * G * D, dtype=torch.bfloat16, device=dev)
    pk.paged_attention_layer(
        input=pk.attach_input(qkv.cuda(), "qkv"), k_cache=pk.attach_input(kc_d, "kc"), v_cache=pk.attach_input(vc_d, "vc"),
        q_norm=pk.attach_input(qn.cuda(), "qn"), k_norm=pk.attach_input(kn.cuda(), "kn"),
        cos_pos_embed=pk.attach_input(cos.cuda(), "cos"), sin_pos_embed=pk.attach_input(sin.cuda(), "sin"),
        output=pk.attach_input(out, "out"), grid_dim=(R, hkv, 1), block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    first = out.clone()
    assert rel_err(out.cpu(), ref) <= TOL
    assert rel_err(kc_d.cpu(), kc_ref) <= 1e-2 and torch.equal(vc_d.cpu(), vc_ref)
    # a second launch appends the same rows again and must reproduce the output bit for bit
    pk.run_test_mode()
    assert torch.equal(first, out)
