"""The allocation-free entry point `mpk_paged_decode_attention_noalloc`, called through the C ABI, against the
handle-based paged attention path (`paged_attention_layer` in a PersistentKernel test-mode graph) on the same
inputs -- two calls in a row, because both share the library's built-in scratch array and the second call finds
the first call's partials and tickets in it.  Collected last so that every other test has run before it.

The entry point exists for callers that may not allocate at call time (stream capture, a memory pool that owns
the device); the test also checks that oversize problems are refused with a message instead of overrunning the
4 MiB scratch."""
import pytest
import torch

from oracle import mpk_ops as ops
from gpu_util import make_test_kernel, rel_err

pytestmark = pytest.mark.gpu
TOL = 2e-2   # max relative error, the bar of the other bf16 parity tests


def _case(seed, lens, G, hkv, page, pages_total):
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    qkv = torch.randn(R, hkv * (G + 2) * 128, generator=g).to(torch.bfloat16)
    kc = torch.randn(pages_total, page, hkv, 128, generator=g).to(torch.bfloat16)
    vc = torch.randn(pages_total, page, hkv, 128, generator=g).to(torch.bfloat16)
    perm = torch.randperm(pages_total, generator=g).tolist()
    indptr, indices, last = [0], [], []
    for n in lens:                       # n = sequence length including the new token
        k = (n + page - 1) // page
        indices += perm[indptr[-1]:indptr[-1] + k]
        indptr.append(indptr[-1] + k)
        last.append((n - 1) % page + 1)
    return qkv, kc, vc, indptr, indices, last


def _handle_path(mi, qkv, kc, vc, indptr, indices, last, G, hkv, page):
    """Existing entry point: mpk_compile + mpk_launch of a one-layer paged attention graph."""
    R = qkv.shape[0]
    dev = "cuda"
    meta = {"qo_indptr_buffer": torch.arange(R + 1, dtype=torch.int32, device=dev),
            "paged_kv_indptr_buffer": torch.tensor(indptr, dtype=torch.int32, device=dev),
            "paged_kv_indices_buffer": torch.tensor(indices + [0] * (kc.shape[0] - len(indices)), dtype=torch.int32,
                                                    device=dev),
            "paged_kv_last_page_len_buffer": torch.tensor(last, dtype=torch.int32, device=dev)}
    pk = make_test_kernel(mi, R, max_num_batched_requests=R, max_num_pages=kc.shape[0], page_size=page,
                          max_seq_length=page * kc.shape[0], meta_tensors=meta)
    kcd, vcd = kc.cuda(), vc.cuda()
    out = torch.zeros(R, hkv * G * 128, dtype=torch.bfloat16, device=dev)
    pk.paged_attention_layer(input=pk.attach_input(qkv.cuda(), "qkv"), k_cache=pk.attach_input(kcd, "kc"),
                             v_cache=pk.attach_input(vcd, "vc"), q_norm=None, k_norm=None, cos_pos_embed=None,
                             sin_pos_embed=None, output=pk.attach_input(out, "out"), grid_dim=(R, hkv, 1),
                             block_dim=(128, 1, 1))
    pk.compile()
    pk.run_test_mode()
    return out.cpu(), kcd.cpu(), vcd.cpu()


def test_noalloc_attention_matches_handle_path_twice():
    import mirage_b200 as mi
    G, hkv, page = 4, 2, 16
    for call, (seed, lens) in enumerate([(31, [37, 5, 64]), (32, [16, 80, 33])]):
        qkv, kc, vc, indptr, indices, last = _case(seed, lens, G, hkv, page, pages_total=16)
        ref_out, ref_kc, ref_vc = _handle_path(mi, qkv, kc, vc, indptr, indices, last, G, hkv, page)
        kcd, vcd = kc.cuda(), vc.cuda()
        out = torch.zeros(len(lens), hkv * G * 128, dtype=torch.bfloat16, device="cuda")
        ip = torch.tensor(indptr, dtype=torch.int32, device="cuda")
        ix = torch.tensor(indices, dtype=torch.int32, device="cuda")
        lp = torch.tensor(last, dtype=torch.int32, device="cuda")
        qd = qkv.cuda()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        mi.paged_decode_attention_noalloc(qd, kcd, vcd, out, ip, ix, lp, hkv * G, hkv, num_chunks=4 + call)
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        assert rel_err(out.cpu(), ref_out) <= TOL, f"call {call}"
        assert torch.equal(kcd.cpu(), ref_kc) and torch.equal(vcd.cpu(), ref_vc)     # appended rows identical
        if call > 0:      # (the first launch may still load the kernel's code; after that the device's free
            assert free_after >= free_before     # memory must not shrink across a call: nothing was allocated)
        # and against the CPU oracle directly
        for r, n in enumerate(lens):
            kk, vv = kc.clone(), vc.clone()
            o = ops.paged_attention_request(qkv[r:r + 1], kk, vv, indices[indptr[r]:indptr[r + 1]], n, hkv * G, hkv,
                                            None, None, None, None)
            assert rel_err(out[r:r + 1].cpu(), o) <= TOL


def test_noalloc_attention_rejects_oversize_problems():
    import mirage_b200 as mi
    t = torch.zeros(1, 6 * 128, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(1, 16, 1, 128, dtype=torch.bfloat16, device="cuda")
    i32 = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(mi.MpkError) as e:
        mi.paged_decode_attention_noalloc(t, kc, kc, torch.zeros(1, 512, dtype=torch.bfloat16, device="cuda"), i32, i32,
                                          i32, 4, 1, num_chunks=5000)
    assert "scratch" in str(e.value)
