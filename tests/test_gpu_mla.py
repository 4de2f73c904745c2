"""GPU parity of the MLA decode tasks (append to the paged latent cache, split decode, merge) against the CPU
oracle and the fixture generated from the reference test's `pytorch_mla_ref`.  Appended cache rows bit-exact;
outputs within 1e-2 absolute (the reference test's bar) and 2e-2 max relative error."""
import os

import pytest
import torch

from oracle import mla_ops as A
from gpu_util import rel_err, make_test_kernel

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mi():
    import mirage_b200
    return mirage_b200


def _dense_decode(mi, Q, KV, q_len, kv_len, scale):
    """Q [R, q_len, H, 576], KV [R, kv_len, 576] -> [R, q_len, H, 512] through decode + reduce layers."""
    R, _, H, _ = Q.shape
    mbt = R * q_len
    S = (kv_len + 127) // 128
    pk = make_test_kernel(mi, mbt)
    out = torch.zeros(mbt, H * 512, dtype=torch.bfloat16, device="cuda")
    po = pk.new_tensor(dims=(mbt * H * S, 512), dtype=mi.bfloat16, name="po", io_category="cuda_tensor")
    lse = pk.new_tensor(dims=(mbt * H * S,), dtype=mi.float32, name="lse", io_category="cuda_tensor")
    tq = pk.attach_input(Q.reshape(mbt, H * 576).cuda(), "q")
    tkv = pk.attach_input(KV.reshape(R * kv_len, 576).cuda(), "kv")
    pk.mla_mtp_decode_layer(tq, tkv, po, lse, q_len, kv_len, sm_scale=scale)
    pk.mla_mtp_reduce_layer(po, lse, pk.attach_input(out, "out"), q_len, kv_len)
    pk.compile()
    pk.run_test_mode()
    first = out.clone()
    pk.run_test_mode()
    assert torch.equal(first, out)
    return out.cpu().reshape(R, q_len, H, 512)


def test_mla_decode_golden_fixture(mi, golden_dir):
    f = torch.load(os.path.join(golden_dir, "ref_mla.pt"), weights_only=False)
    for case in f.values():
        Q, KV = case["Q"], case["KV"]
        out = _dense_decode(mi, Q, KV, Q.shape[1], case["kv_len"], case["scale"])
        assert (out.float() - case["out"].float()).abs().max() < 1e-2
        assert rel_err(out, case["out"]) <= 2e-2


@pytest.mark.parametrize("R,q_len,H,kv_len", [(2, 2, 32, 300), (1, 1, 128, 1000), (3, 1, 16, 129), (1, 4, 16, 64)])
def test_mla_decode_dense_cache_shapes(mi, R, q_len, H, kv_len):
    g = torch.Generator().manual_seed(R * 100 + H + kv_len)
    Q = (torch.randn(R, q_len, H, 576, generator=g) * 0.3).to(torch.bfloat16)
    KV = (torch.randn(R, kv_len, 576, generator=g) * 0.3).to(torch.bfloat16)
    scale = A.DEEPSEEK_SCALE
    out = _dense_decode(mi, Q, KV, q_len, kv_len, scale)
    for r in range(R):
        kvf = KV[r].float()
        for i in range(q_len):
            lim = kv_len - q_len + i + 1
            p = torch.softmax((Q[r, i].float() @ kvf[:lim].T) * scale, dim=-1)
            ref = (p @ kvf[:lim, :512]).to(torch.bfloat16)
            assert rel_err(out[r, i], ref) <= 2e-2


@pytest.mark.parametrize("H", [16, 128])
def test_mla_paged_append_decode_reduce(mi, H):
    """Three requests of different lengths, one of them with two new tokens: append, decode on the paged cache with
    the batch's page tables, merge -- the attention step of a DeepSeek-V3 layer as the reference builds it
    (python/mirage/mpk/models/deepseek_v3/builder.py:733-775)."""
    page, npages_total = 64, 16
    lens, new = [130, 64, 257], [1, 2, 1]            # lengths include the new tokens
    R, mbt = 3, 4
    g = torch.Generator().manual_seed(H)
    cache = (torch.randn(npages_total, page, 576, generator=g) * 0.3).to(torch.bfloat16)
    perm = torch.randperm(npages_total, generator=g).tolist()
    indptr, indices, last, qo = [0], [], [], [0]
    for L, n in zip(lens, new):
        k = (L + page - 1) // page
        indices += perm[indptr[-1]:indptr[-1] + k]
        indptr.append(indptr[-1] + k)
        last.append((L - 1) % page + 1)
        qo.append(qo[-1] + n)
    lat = (torch.randn(mbt, 512, generator=g) * 0.3).to(torch.bfloat16)
    pe = (torch.randn(mbt, 128, generator=g) * 0.3).to(torch.bfloat16)     # k_pe rows are padded to 128
    Q = (torch.randn(mbt, H, 576, generator=g) * 0.3).to(torch.bfloat16)
    # oracle
    ref_cache = cache.clone()
    ref = []
    for r in range(R):
        pages = indices[indptr[r]:indptr[r + 1]]
        A.mla_append(ref_cache, lat[qo[r]:qo[r + 1]], pe[qo[r]:qo[r + 1]], pages, lens[r])
        ref.append(A.mla_decode_request(Q[qo[r]:qo[r + 1]], ref_cache, pages, lens[r], A.DEEPSEEK_SCALE))
    ref = torch.cat(ref)
    # megakernel
    dev = "cuda"
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    meta = {"qo_indptr_buffer": i32(qo), "paged_kv_indptr_buffer": i32(indptr),
            "paged_kv_indices_buffer": i32(indices + [0] * (npages_total - len(indices))),
            "paged_kv_last_page_len_buffer": i32(last)}
    max_seq = 512
    pk = make_test_kernel(mi, mbt, max_num_batched_requests=R, max_num_pages=npages_total, page_size=page,
                          max_seq_length=max_seq, meta_tensors=meta)
    S = (max_seq + 127) // 128
    cache_d = cache.cuda()
    out = torch.zeros(mbt, H * 512, dtype=torch.bfloat16, device=dev)
    t_cache = pk.attach_input(cache_d, "cache")
    contiguous = pk.new_tensor(dims=(R * max_seq, 576), dtype=mi.bfloat16, name="contiguous_kv", io_category="cuda_tensor")
    po = pk.new_tensor(dims=(mbt * H * S, 512), dtype=mi.bfloat16, name="po", io_category="cuda_tensor")
    lse = pk.new_tensor(dims=(mbt * H * S,), dtype=mi.float32, name="lse", io_category="cuda_tensor")
    pk.mla_kv_gather_layer(c_latent_new=pk.attach_input(lat.cuda(), "lat"), k_pe_new=pk.attach_input(pe.cuda(), "pe"),
                           paged_cache=t_cache, contiguous_kv=contiguous, mla_params=(576, 512, page),
                           grid_dim=(R, 1, 1), block_dim=(128, 1, 1))
    pk.mla_mtp_decode_layer(pk.attach_input(Q.reshape(mbt, H * 576).cuda(), "q"), contiguous, po, lse, mbt, max_seq)
    pk.mla_mtp_reduce_layer(po, lse, pk.attach_input(out, "out"), mbt, max_seq)
    pk.compile()
    pk.run_test_mode()
    assert torch.equal(cache_d.cpu(), ref_cache)           # appended rows identical, nothing else touched
    got = out.cpu().reshape(mbt, H, 512)
    assert (got.float() - ref.float()).abs().max() < 1e-2
    assert rel_err(got, ref) <= 2e-2
