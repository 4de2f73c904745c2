"""Argument checks of the allocation-free attention entry point, on the host only: every rule that bounds the
kernel's device accesses must come back as an error (C ABI) or ValueError (Python wrapper) before anything is
launched.  No GPU is touched: the C entry validates sizes, strides and alignment before its first CUDA call, so
fake non-null addresses are enough to reach the checks."""
import ctypes as C

import pytest
import torch

from mirage_b200 import _native as N
from mirage_b200.noalloc import check_noalloc_arguments


def _call(ld_qkv=768, ld_out=512, qkv=0x1000, out=0x2000, kc=0x3000, vc=0x4000, idx=0x5000, hq=4, hkv=1, chunks=4,
          requests=1):
    err = C.create_string_buffer(256)
    rc = N.lib.mpk_paged_decode_attention_noalloc(qkv, kc, vc, out, idx, idx, idx, requests, hq, hkv, 16, ld_qkv, ld_out,
                                                  chunks, None, err, len(err))
    return rc, err.value.decode()


def test_c_entry_rejects_bad_geometry_before_any_cuda_call():
    for kw, word in [(dict(ld_qkv=767), "narrower"), (dict(ld_out=511), "narrower"), (dict(ld_qkv=770), "multiples of 4"),
                     (dict(ld_out=514), "multiples of 4"), (dict(qkv=0x1004), "8-byte"), (dict(out=0x2002), "8-byte"),
                     (dict(idx=0x5002), "4-byte"), (dict(ld_qkv=1 << 40), "narrower"), (dict(hq=3, hkv=2), "bad sizes"),
                     (dict(hq=16, hkv=1, ld_qkv=18 * 128, ld_out=16 * 128), "group size"), (dict(qkv=0), "null"),
                     (dict(chunks=5000), "scratch"), (dict(requests=5000, hq=1, hkv=1, ld_qkv=384, ld_out=128), "tickets")]:
        rc, msg = _call(**kw)
        assert rc in (-1, -3), (kw, rc, msg)
        assert word in msg, (kw, msg)


def _tensors(R=2, hkv=2, G=4, page=16, pages=4):
    bf = torch.bfloat16
    return dict(qkv=torch.zeros(R, hkv * (G + 2) * 128, dtype=bf), k_cache=torch.zeros(pages, page, hkv, 128, dtype=bf),
                v_cache=torch.zeros(pages, page, hkv, 128, dtype=bf), out=torch.zeros(R, hkv * G * 128, dtype=bf),
                kv_indptr=torch.zeros(R + 1, dtype=torch.int32), kv_indices=torch.zeros(pages, dtype=torch.int32),
                kv_last_page_len=torch.ones(R, dtype=torch.int32))


def test_wrapper_checks_every_size_that_bounds_a_device_access():
    t = _tensors()
    check_noalloc_arguments(**t, num_q_heads=8, num_kv_heads=2, require_cuda=False)      # the good case passes
    bad = [("qkv", t["qkv"][:, :-128].contiguous(), "qkv rows"), ("out", t["out"][:, :-1].contiguous(), "out rows"),
           ("v_cache", t["v_cache"][:-1], "v_cache"), ("kv_indptr", t["kv_indptr"][:-1], "kv_indptr"),
           ("kv_last_page_len", t["kv_last_page_len"][:-1], "kv_last_page_len"),
           ("kv_indices", t["kv_indices"].to(torch.int64), "int32"), ("k_cache", t["k_cache"].float(), "bfloat16"),
           ("qkv", torch.zeros(2, 2 * 6 * 128 + 2, dtype=torch.bfloat16)[:, :], "multiples of 4"),
           ("qkv", torch.zeros(2, 2 * 6 * 128 * 2, dtype=torch.bfloat16)[:, ::2], "unit inner stride"),
           ("out", torch.zeros(1, 1024, dtype=torch.bfloat16), "fewer rows")]
    for name, value, word in bad:
        args = dict(t)
        args[name] = value
        with pytest.raises(ValueError) as e:
            check_noalloc_arguments(**args, num_q_heads=8, num_kv_heads=2, require_cuda=False)
        assert word in str(e.value), (name, str(e.value))
    with pytest.raises(ValueError) as e:
        check_noalloc_arguments(**t, num_q_heads=8, num_kv_heads=2)       # CPU tensors where CUDA ones are required
    assert "CUDA tensor" in str(e.value)
