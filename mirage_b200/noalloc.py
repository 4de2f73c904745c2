"""Python wrapper of `mpk_paged_decode_attention_noalloc` (include/mpk_b200.h).

For callers that cannot allocate device memory when they call the library (a stream being captured, a memory
pool that owns the device): the split-KV scratch is a fixed 4 MiB array inside libmpk_b200.so, so this call
performs no cudaMalloc / cudaFree and creates no torch tensor.  The first call on a device must happen outside
stream capture; calls that may overlap on the GPU race on the shared scratch, so keep them on one stream.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as N


def paged_decode_attention_noalloc(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                   out: torch.Tensor, kv_indptr: torch.Tensor, kv_indices: torch.Tensor,
                                   kv_last_page_len: torch.Tensor, num_q_heads: int, num_kv_heads: int,
                                   num_chunks: int = 8, stream=None) -> None:
    """out[r] = attention of request r's new token (q/k/v packed in qkv[r]) over its paged KV sequence, after
    appending the new k/v row at the sequence's last position.  All tensors are caller-owned CUDA tensors."""
    check_noalloc_arguments(qkv, k_cache, v_cache, out, kv_indptr, kv_indices, kv_last_page_len, num_q_heads,
                            num_kv_heads)
    err = C.create_string_buffer(256)
    # the library launches on the current device and picks that device's scratch: make it the tensors' device
    with torch.cuda.device(qkv.device):
        st = torch.cuda.current_stream() if stream is None else stream
        rc = N.lib.mpk_paged_decode_attention_noalloc(
            qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), kv_indptr.data_ptr(),
            kv_indices.data_ptr(), kv_last_page_len.data_ptr(), qkv.shape[0], num_q_heads, num_kv_heads,
            k_cache.shape[1], qkv.stride(0), out.stride(0), num_chunks, int(st.cuda_stream), err, len(err))
    if rc != 0:
        raise N.MpkError(rc, err.value.decode())


def check_noalloc_arguments(qkv, k_cache, v_cache, out, kv_indptr, kv_indices, kv_last_page_len, num_q_heads,
                            num_kv_heads, require_cuda: bool = True) -> None:
    """Everything that bounds the kernel's device accesses, checked on the host: a violated rule would otherwise be
    an out-of-bounds or misaligned access on the GPU (a lost context), not an error return.  Raises ValueError.
    `require_cuda=False` lets the shape / stride rules be exercised with CPU tensors."""
    tensors = dict(qkv=qkv, k_cache=k_cache, v_cache=v_cache, out=out, kv_indptr=kv_indptr, kv_indices=kv_indices,
                   kv_last_page_len=kv_last_page_len)

    def need(cond, msg):
        if not cond:
            raise ValueError("paged_decode_attention_noalloc: " + msg)

    if require_cuda:
        for name, t in tensors.items():
            need(t.is_cuda, f"{name} must be a CUDA tensor")
            need(t.device == qkv.device, f"{name} is on {t.device}, qkv on {qkv.device}: all tensors must share one device")
    need(num_kv_heads >= 1 and num_q_heads >= 1 and num_q_heads % num_kv_heads == 0, "q heads must be a multiple of kv heads")
    group = num_q_heads // num_kv_heads
    for name in ("qkv", "k_cache", "v_cache", "out"):
        need(tensors[name].dtype == torch.bfloat16, f"{name} must be bfloat16")
    for name in ("kv_indptr", "kv_indices", "kv_last_page_len"):
        need(tensors[name].dtype == torch.int32 and tensors[name].dim() == 1 and tensors[name].is_contiguous(),
             f"{name} must be a contiguous 1-D int32 tensor")
    need(qkv.dim() == 2 and out.dim() == 2 and qkv.stride(1) == 1 and out.stride(1) == 1, "qkv and out must be 2-D with unit inner stride")
    requests = qkv.shape[0]
    need(out.shape[0] >= requests, "out has fewer rows than qkv")
    need(qkv.shape[1] >= num_kv_heads * (group + 2) * 128,
         f"qkv rows hold {qkv.shape[1]} elements; {num_kv_heads} kv heads x (G + 2) x 128 = {num_kv_heads * (group + 2) * 128} needed")
    need(out.shape[1] >= num_q_heads * 128, f"out rows hold {out.shape[1]} elements; {num_q_heads * 128} needed")
    need(k_cache.dim() == 4 and k_cache.shape[3] == 128 and k_cache.shape[2] == num_kv_heads and k_cache.is_contiguous(),
         "k_cache must be a contiguous [pages, page_size, kv_heads, 128] tensor")
    need(v_cache.shape == k_cache.shape and v_cache.is_contiguous(), "v_cache must have k_cache's shape and be contiguous")
    need(kv_indptr.numel() >= requests + 1, "kv_indptr needs requests + 1 entries")
    need(kv_last_page_len.numel() >= requests, "kv_last_page_len needs one entry per request")
    need(qkv.stride(0) % 4 == 0 and out.stride(0) % 4 == 0, "row strides of qkv and out must be multiples of 4 elements")
    for name in ("qkv", "k_cache", "v_cache", "out"):
        need(tensors[name].data_ptr() % 8 == 0, f"{name} must be 8-byte aligned")
