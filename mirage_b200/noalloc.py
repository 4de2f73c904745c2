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
    assert qkv.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert kv_indptr.dtype == kv_indices.dtype == kv_last_page_len.dtype == torch.int32
    assert k_cache.dim() == 4 and k_cache.shape[3] == 128 and k_cache.shape[2] == num_kv_heads
    assert qkv.stride(1) == 1 and out.stride(1) == 1
    st = torch.cuda.current_stream() if stream is None else stream
    err = C.create_string_buffer(256)
    rc = N.lib.mpk_paged_decode_attention_noalloc(
        qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), kv_indptr.data_ptr(),
        kv_indices.data_ptr(), kv_last_page_len.data_ptr(), qkv.shape[0], num_q_heads, num_kv_heads,
        k_cache.shape[1], qkv.stride(0), out.stride(0), num_chunks, int(st.cuda_stream), err, len(err))
    if rc != 0:
        raise N.MpkError(rc, err.value.decode())
