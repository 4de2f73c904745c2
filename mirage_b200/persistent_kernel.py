"""`PersistentKernel`: the reference's Python surface over the B200 megakernel library.

Mirrors python/mirage/mpk/persistent_kernel.py:348-2708 of mirage-project/mirage for the
decode path -- same constructor arguments, same `*_layer` method names and keyword
arguments, `compile()`, `__call__`, `run_test_mode()`, `finalize()` -- but every method
only records the layer through the C ABI (include/mpk_b200.h).  `compile()` takes
milliseconds: the megakernel is pre-built, nothing is generated or handed to nvcc.

`grid_dim` / `block_dim` are accepted on every layer as in the reference.  They are
partitioning hints: the library cuts each layer into tasks itself (one contiguous weight
panel per SM for linears, split-KV chunks for attention), except where the grid defines
data layout (interleave groups of silu_mul, number of argmax partials).

PyTorch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
import math
import json
import os
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import _native as N
from ._native import MpkError, MpkTimeoutError  # noqa: F401  (re-exported)

valid_persistent_kernel_modes = ("offline", "online", "online_notoken", "onepass", "online_multi_turn")


class dtype:
    """Element type tag, named like the constants of mirage.core (python/mirage/_cython/core.pyx)."""

    def __init__(self, name: str, code: int, torch_dtype, size: int):
        self.name, self.code, self.torch_dtype, self.size = name, code, torch_dtype, size

    def __repr__(self):
        return f"mirage_b200.{self.name}"


bfloat16 = dtype("bfloat16", N.BF16, torch.bfloat16, 2)
float16 = dtype("float16", N.F16, torch.float16, 2)
float32 = dtype("float32", N.F32, torch.float32, 4)
int32 = dtype("int32", N.I32, torch.int32, 4)
int64 = dtype("int64", N.I64, torch.int64, 8)
uint32 = dtype("uint32", N.U32, torch.uint32, 4)
uint8 = dtype("uint8", N.U8, torch.uint8, 1)
int16 = dtype("int16", N.I16, torch.int16, 2)
float8_e4m3 = dtype("float8_e4m3", N.F8E4M3, torch.float8_e4m3fn, 1)
_ALL_DTYPES = [bfloat16, float16, float32, int32, int64, uint32, uint8, int16, float8_e4m3]


def convert_torch_type_to_dtype(t) -> dtype:
    for d in _ALL_DTYPES:
        if d.torch_dtype == t:
            return d
    raise ValueError(f"unsupported torch dtype {t}")


class DTensor:
    """Handle of a tensor registered with a PersistentKernel (mirage.core.DTensor look-alike)."""

    def __init__(self, tid: int, dims, strides, dt: dtype, name: str):
        self.id, self.dims, self.strides, self.dtype, self.name = tid, tuple(dims), tuple(strides), dt, name

    @property
    def num_dims(self) -> int:
        return len(self.dims)

    def dim(self, i: int) -> int:
        return self.dims[i]

    def stride(self, i: int) -> int:
        return self.strides[i]

    def __repr__(self):
        return f"DTensor({self.name}, dims={self.dims}, dtype={self.dtype.name})"


def get_configurations_from_gpu(rank: int = 0) -> Tuple[int, int]:
    """(num_workers, num_local_schedulers) for the device, like python/mirage/utils.py:33-53.

    This runtime has no scheduler CTAs: every SM is a worker and the scheduler count is
    returned only so that code written for the reference keeps working.
    """
    sm = torch.cuda.get_device_properties(rank).multi_processor_count
    return sm, 0


def _ids(tensors: Sequence[Optional[DTensor]]):
    arr = (C.c_int * len(tensors))(*[(-1 if t is None else t.id) for t in tensors])
    return arr, len(tensors)


class _KNGraphShim:
    """`mpk.kn_graph.generate_task_graph(...)` as demo scripts call it (demo/qwen3/demo.py:749-753)."""

    def __init__(self, owner: "PersistentKernel"):
        self._o = owner

    def generate_task_graph(self, num_gpus: int = 1, my_gpu_id: int = 0) -> Dict[str, str]:
        return {"cuda_code": "// pre-built sm_100a megakernel: no code is generated",
                "json_file": self._o.dump_task_graph()}


class PersistentKernel:
    def __init__(
        self,
        mode: str = "offline",
        world_size: int = 1,
        mpi_rank: int = 0,
        num_workers: int = 0,
        num_local_schedulers: int = 0,
        num_remote_schedulers: int = 0,
        max_seq_length: int = 1,
        max_num_batched_requests: int = 1,
        max_num_batched_tokens: int = 1,
        max_num_pages: int = 1,
        page_size: int = 1,
        meta_tensors: Optional[dict] = None,
        profiler_tensor: Optional[torch.Tensor] = None,
        trace_name: str = "",
        spec_decode_config=None,
        use_cutlass_kernel: bool = False,
        eos_token_id: int = -1,
        test_mode: bool = False,
        dry_run: bool = False,
        device: Optional[int] = None,
    ):
        if mode not in valid_persistent_kernel_modes:
            raise ValueError(f"Invalid persistent kernel mode: {mode}")
        if mode not in ("offline", "online_notoken") and not test_mode:
            raise NotImplementedError(f"mode {mode!r} is not implemented by mirage_b200 (offline, online_notoken)")
        if spec_decode_config is not None:
            raise NotImplementedError("speculative decoding is outside the decode path this library implements")
        self.__finalized__ = False
        self._is_compiled = False
        self.test_mode = test_mode
        self.dry_run = dry_run
        self.mode = mode
        self.world_size, self.mpi_rank = world_size, mpi_rank
        self.num_local_schedulers, self.num_remote_schedulers = num_local_schedulers, num_remote_schedulers
        self.max_seq_length = max_seq_length
        self.max_num_batched_requests = max_num_batched_requests
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_num_pages, self.page_size = max_num_pages, page_size
        self.eos_token_id = eos_token_id
        self.meta_tensors = dict(meta_tensors or {})
        self.profiler_tensor, self.trace_name = profiler_tensor, trace_name
        self.use_nvshmem = world_size > 1
        self.spec_decode_config = None
        self.use_cutlass_kernel = use_cutlass_kernel
        self._torch_tensor_refs = []
        self._mla_paged = {}     # contiguous_kv tensor id -> (paged cache tensor, page size), set by mla_kv_gather_layer
        self._model_tensors: Dict[str, torch.Tensor] = {}
        self._tensors = []
        self.kn_graph = _KNGraphShim(self)
        if dry_run:
            self.device, self.target_cc, sm = 0, 100, 148
        else:
            if not torch.cuda.is_available():
                raise RuntimeError("mirage_b200 needs a CUDA device (sm_100a); there is no CPU path")
            self.device = torch.cuda.current_device() if device is None else device
            props = torch.cuda.get_device_properties(self.device)
            self.target_cc = props.major * 10 + props.minor
            sm = props.multi_processor_count
        self.num_workers = num_workers if num_workers and num_workers > 0 else sm

        mt = self.meta_tensors
        if not test_mode and mode == "online_notoken":
            # one forward per call on a batch the caller describes: only the description itself is needed
            for key, dt in (("input_tokens", torch.int64), ("qo_indptr_buffer", torch.int32),
                            ("paged_kv_indptr_buffer", torch.int32), ("paged_kv_indices_buffer", torch.int32),
                            ("paged_kv_last_page_len_buffer", torch.int32)):
                if key not in mt:
                    raise ValueError(f"meta_tensors[{key!r}] is required in online_notoken mode")
                assert mt[key].dtype == dt, f"{key}.dtype: {mt[key].dtype}"
            self.total_num_requests = mt["tokens"].shape[0] if "tokens" in mt else max_num_batched_requests
        elif not test_mode:
            for key, dt in (("step", torch.int32), ("tokens", torch.int64), ("input_tokens", torch.int64),
                            ("output_tokens", torch.int64), ("num_new_tokens", torch.int32),
                            ("prompt_lengths", torch.int32), ("qo_indptr_buffer", torch.int32),
                            ("paged_kv_indptr_buffer", torch.int32), ("paged_kv_indices_buffer", torch.int32),
                            ("paged_kv_last_page_len_buffer", torch.int32)):
                if key not in mt:
                    raise ValueError(f"meta_tensors[{key!r}] is required outside test mode")
                assert mt[key].dtype == dt, f"{key}.dtype: {mt[key].dtype}"
            self.total_num_requests = mt["tokens"].shape[0]
            assert self.max_seq_length == mt["tokens"].shape[1]
            assert mt["qo_indptr_buffer"].shape[0] >= max_num_batched_requests + 1
            assert mt["paged_kv_indptr_buffer"].shape[0] >= max_num_batched_requests + 1
            assert mt["paged_kv_indices_buffer"].shape[0] >= max_num_pages
            assert mt["paged_kv_last_page_len_buffer"].shape[0] >= max_num_batched_requests
            if "paged_kv_indices_snapshot" not in mt and not dry_run:
                mt["paged_kv_indices_snapshot"] = torch.empty(max_num_pages, dtype=torch.int32,
                                                              device=mt["tokens"].device)
        else:
            self.total_num_requests = 1

        def ptr(key):
            t = mt.get(key)
            return None if t is None or dry_run else t.data_ptr()

        cfg = N.MpkConfig()
        cfg.mode = N.MODE_OFFLINE if mode == "offline" else N.MODE_ONLINE_NOTOKEN
        cfg.test_mode, cfg.dry_run, cfg.device = int(test_mode), int(dry_run), self.device
        cfg.world_size, cfg.rank, cfg.num_workers = world_size, mpi_rank, self.num_workers
        cfg.max_seq_length, cfg.max_num_batched_requests = max_seq_length, max_num_batched_requests
        cfg.max_num_batched_tokens, cfg.max_num_pages, cfg.page_size = max_num_batched_tokens, max_num_pages, page_size
        cfg.total_num_requests, cfg.eos_token_id = self.total_num_requests, eos_token_id
        cfg.step, cfg.tokens = ptr("step"), ptr("tokens")
        cfg.input_tokens, cfg.output_tokens = ptr("input_tokens"), ptr("output_tokens")
        cfg.num_new_tokens, cfg.prompt_lengths = ptr("num_new_tokens"), ptr("prompt_lengths")
        cfg.qo_indptr, cfg.paged_kv_indptr = ptr("qo_indptr_buffer"), ptr("paged_kv_indptr_buffer")
        cfg.paged_kv_indices = ptr("paged_kv_indices_buffer")
        cfg.paged_kv_last_page_len = ptr("paged_kv_last_page_len_buffer")
        cfg.paged_kv_indices_snapshot = ptr("paged_kv_indices_snapshot")
        if profiler_tensor is not None:
            cfg.profiler_buffer, cfg.profiler_entries = profiler_tensor.data_ptr(), profiler_tensor.numel()
        self._cfg = cfg
        h = C.c_void_p()
        rc = N.lib.mpk_create(C.byref(cfg), C.byref(h))
        self._h = h
        N.check(self._h, rc)

    @classmethod
    def get_default_init_parameters(cls):
        return {"mode": "offline", "world_size": 1, "mpi_rank": 0, "num_workers": 1, "num_local_schedulers": 4,
                "num_remote_schedulers": 0, "max_seq_length": 1, "max_num_batched_requests": 1,
                "max_num_batched_tokens": 1, "max_num_pages": 1, "page_size": 1, "meta_tensors": dict(),
                "profiler_tensor": None, "trace_name": "test_trace", "spec_decode_config": None,
                "use_cutlass_kernel": False, "eos_token_id": -1}

    # ------------------------------------------------------------------ tensors
    def attach_input(self, torch_tensor: torch.Tensor, name: str = None) -> DTensor:
        assert name is not None
        dims, strides = tuple(torch_tensor.shape), tuple(torch_tensor.stride())
        row_major = all(strides[d] == strides[d + 1] * dims[d + 1] for d in range(len(dims) - 1))
        col_major = len(dims) == 2 and strides[0] == 1 and strides[1] >= dims[0]
        assert row_major or col_major, f"Tensor must be row-major or column-major, got dims={dims} strides={strides}"
        dt = convert_torch_type_to_dtype(torch_tensor.dtype)
        d = (C.c_int64 * len(dims))(*dims)
        s = (C.c_int64 * len(dims))(*strides)
        p = None if self.dry_run else torch_tensor.data_ptr()
        tid = N.check(self._h, N.lib.mpk_attach_tensor(self._h, name.encode(), p, dt.code, len(dims), d, s))
        self._model_tensors[name] = torch_tensor
        self._torch_tensor_refs.append(torch_tensor)
        t = DTensor(tid, dims, strides, dt, name)
        self._tensors.append(t)
        return t

    def new_tensor(self, dims: tuple, strides: tuple = None, dtype: dtype = bfloat16, name: str = None,
                   io_category: str = "cuda_tensor") -> DTensor:
        assert name is not None
        if io_category not in ("cuda_tensor", "nvshmem_tensor"):
            raise RuntimeError(f"Invalid io_category: {io_category}")
        dims = tuple(int(x) for x in dims)
        if strides is None:
            st = [1] * len(dims)
            for i in range(len(dims) - 2, -1, -1):
                st[i] = st[i + 1] * dims[i + 1]
            strides = tuple(st)
        d = (C.c_int64 * len(dims))(*dims)
        s = (C.c_int64 * len(dims))(*strides)
        cat = N.IO_SYMMETRIC if io_category == "nvshmem_tensor" else N.IO_CUDA
        tid = N.check(self._h, N.lib.mpk_new_tensor(self._h, name.encode(), dtype.code, len(dims), d, s, cat))
        t = DTensor(tid, dims, strides, dtype, name)
        self._tensors.append(t)
        return t

    def _combine(self, fn, inputs, dim, num_groups, name):
        assert dim == 0
        arr, n = _ids(inputs)
        tid = N.check(self._h, fn(self._h, (name or "fused").encode(), arr, n, num_groups))
        rows = sum(t.dim(0) for t in inputs)
        t = DTensor(tid, (rows, inputs[0].dim(1)), (inputs[0].dim(1), 1), inputs[0].dtype, name)
        self._tensors.append(t)
        return t

    def fuse_tensors(self, inputs, fused_dim: int, num_groups: int, name: str = None) -> DTensor:
        return self._combine(N.lib.mpk_fuse_tensors, inputs, fused_dim, num_groups, name)

    def shuffle_tensors(self, inputs, shuffled_dim: int, num_groups: int, name: str = None) -> DTensor:
        return self._combine(N.lib.mpk_shuffle_tensors, inputs, shuffled_dim, num_groups, name)

    def tensor_as_torch(self, t: DTensor) -> torch.Tensor:
        """A torch view of a tensor the library allocated (after compile()); for tests and debugging."""
        assert self._is_compiled and not self.dry_run
        p, nb = C.c_void_p(), C.c_uint64()
        N.check(self._h, N.lib.mpk_tensor_ptr(self._h, t.id, C.byref(p), C.byref(nb)))
        n = int(nb.value) // t.dtype.size

        class _Mem:   # __cuda_array_interface__ carrier
            pass
        m = _Mem()
        m.__cuda_array_interface__ = {"shape": (int(nb.value),), "typestr": "|u1", "data": (int(p.value), False),
                                      "version": 2}
        flat = torch.as_tensor(m, device=f"cuda:{self.device}").view(t.dtype.torch_dtype)[:n]
        return torch.as_strided(flat, t.dims, t.strides)

    # ------------------------------------------------------------------ layers
    def _layer(self, op, tensors, grid_dim, params=()):
        arr, n = _ids(tensors)
        g = tuple(grid_dim) + (1,) * (3 - len(tuple(grid_dim)))
        grid = (C.c_int * 3)(*[int(x) for x in g[:3]])
        pr = (C.c_int64 * max(len(params), 1))(*[int(x) for x in params])
        return N.check(self._h, N.lib.mpk_add_layer(self._h, op, arr, n, grid, pr, len(params)))

    def embed_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple,
                    input_source: int = 0):
        self._layer(N.OP_EMBED, [input, weight, output], grid_dim, [input_source])

    def rmsnorm_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2 and output.num_dims == 2
        self._layer(N.OP_RMSNORM, [input, weight, output], grid_dim)

    def rmsnorm_linear_layer(self, input: DTensor, weight_norm: DTensor, weight_linear: DTensor, output: DTensor,
                             grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2 and weight_linear.num_dims == 2 and output.num_dims == 2
        self._layer(N.OP_RMSNORM_LINEAR, [input, weight_norm, weight_linear, output], grid_dim)

    def linear_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2 and weight.num_dims == 2 and output.num_dims == 2
        self._layer(N.OP_LINEAR, [input, weight, output], grid_dim)

    def linear_with_residual_layer(self, input: DTensor, weight: DTensor, residual: DTensor, output: DTensor,
                                   grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2 and weight.num_dims == 2 and residual.num_dims == 2 and output.num_dims == 2
        enable_residual = 0 if (self.world_size > 1 and self.mpi_rank != 0) else 1
        self._layer(N.OP_LINEAR_RESIDUAL, [input, weight, residual, output], grid_dim, [enable_residual])

    def splitk_linear_layer(self, input: DTensor, weight: DTensor, output: DTensor, grid_dim: tuple,
                            block_dim: tuple):
        assert input.num_dims == 2 and weight.num_dims == 2 and output.num_dims == 2
        self._layer(N.OP_SPLITK_LINEAR, [input, weight, output], grid_dim)

    def _attention(self, op, input, k_cache, v_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, output,
                   grid_dim, extra):
        assert input.num_dims == 2 and output.num_dims == 2
        assert k_cache.num_dims == 4 and v_cache.num_dims == 4
        head_dim, num_kv_heads = k_cache.dim(3), k_cache.dim(2)
        num_q_heads = output.dim(1) // head_dim
        rotary = 0
        if cos_pos_embed is not None or sin_pos_embed is not None:
            assert cos_pos_embed.num_dims == 2 and sin_pos_embed.num_dims == 2
            assert cos_pos_embed.dim(1) == head_dim and sin_pos_embed.dim(1) == head_dim
            rotary = 1
        qk_norm = 0
        if q_norm is not None or k_norm is not None:
            assert q_norm.num_dims == 1 and k_norm.num_dims == 1
            assert q_norm.dim(0) == head_dim and k_norm.dim(0) == head_dim
            qk_norm = 1
        self._layer(op, [input, k_cache, v_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed, output], grid_dim,
                    [num_q_heads, num_kv_heads, qk_norm, rotary] + list(extra))

    def attention_layer(self, input: DTensor, k_cache: DTensor, v_cache: DTensor, q_norm: DTensor, k_norm: DTensor,
                        cos_pos_embed: DTensor, sin_pos_embed: DTensor, output: DTensor, grid_dim: tuple,
                        block_dim: tuple):
        self._attention(N.OP_ATTENTION, input, k_cache, v_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed,
                        output, grid_dim, [])

    def paged_attention_layer(self, input: DTensor, k_cache: DTensor, v_cache: DTensor, q_norm: DTensor,
                              k_norm: DTensor, cos_pos_embed: DTensor, sin_pos_embed: DTensor, output: DTensor,
                              grid_dim: tuple, block_dim: tuple):
        assert grid_dim[0] == self.max_num_batched_requests and grid_dim[1] == k_cache.dim(2), \
            "paged attention grid must be (max_num_batched_requests, num_kv_heads, 1)"
        self._attention(N.OP_PAGED_ATTENTION, input, k_cache, v_cache, q_norm, k_norm, cos_pos_embed,
                        sin_pos_embed, output, grid_dim, [self.max_seq_length, self.page_size])

    def paged_attention_split_kv_layer(self, input: DTensor, k_cache: DTensor, v_cache: DTensor, q_norm: DTensor,
                                       k_norm: DTensor, cos_pos_embed: DTensor, sin_pos_embed: DTensor, lse: DTensor,
                                       output: DTensor, attention_params: tuple, grid_dim: tuple, block_dim: tuple):
        """First half of the reference's long-context pair (python/mirage/mpk/persistent_kernel.py:865-950): per-chunk
        partial attention into `output` [tokens, chunks x q-per-kv x head_dim, kv_heads] with `lse`.  Here every
        paged attention layer is already split over the kv range and merged by the last chunk to finish, with its
        partials in a scratch buffer the library owns; the pair is therefore recorded and emitted as ONE paged
        attention layer when `paged_attention_split_kv_merge_layer` names the final output.  `lse` and the partial
        `output` stay untouched; `attention_params = (num_q_heads, num_kv_chunks)` -- the chunk count is a hint."""
        assert input.num_dims == 2 and k_cache.num_dims == 4 and v_cache.num_dims == 4
        assert k_cache.dim(0) == self.max_num_pages and k_cache.dim(1) == self.page_size
        assert output.num_dims == 3 and lse.num_dims == 3
        assert grid_dim[0] == self.max_num_batched_requests and grid_dim[1] == k_cache.dim(2)
        assert attention_params[0] % k_cache.dim(2) == 0
        if not hasattr(self, "_pending_split_kv"):
            self._pending_split_kv = {}
        self._pending_split_kv[(lse.id, output.id)] = (input, k_cache, v_cache, q_norm, k_norm, cos_pos_embed, sin_pos_embed,
                                                       int(attention_params[0]), grid_dim)

    def paged_attention_split_kv_merge_layer(self, lse: DTensor, output_tmp: DTensor, output: DTensor,
                                             attention_params: tuple, grid_dim: tuple, block_dim: tuple):
        """Second half (python/mirage/mpk/persistent_kernel.py:952-992): merges the chunks of the split layer that wrote
        `lse` / `output_tmp` into `output` [tokens, q_heads x head_dim].  See paged_attention_split_kv_layer."""
        assert lse.num_dims == 3 and output_tmp.num_dims == 3 and output.num_dims == 2
        pend = getattr(self, "_pending_split_kv", {}).pop((lse.id, output_tmp.id), None)
        if pend is None:
            raise ValueError("paged_attention_split_kv_merge_layer: no paged_attention_split_kv_layer wrote these lse / output_tmp")
        input, k_cache, v_cache, q_norm, k_norm, cos, sin, num_q_heads, split_grid = pend
        assert int(attention_params[0]) == num_q_heads and output.dim(1) == num_q_heads * k_cache.dim(3)
        self.paged_attention_layer(input=input, k_cache=k_cache, v_cache=v_cache, q_norm=q_norm, k_norm=k_norm,
                                   cos_pos_embed=cos, sin_pos_embed=sin, output=output, grid_dim=split_grid,
                                   block_dim=block_dim)

    def moe_topk_softmax_routing_layer(self, input: DTensor, output: tuple, grid_dim: tuple, block_dim: tuple,
                                       local_experts: tuple = None):
        """Softmax top-k routing (python/mirage/mpk/persistent_kernel.py:1385-1406, tasks/blackwell/topk_softmax_sm100.cuh):
        softmax over the experts in fp32, the k largest probabilities (ties to the lower expert), weights renormalised over
        the selected ones; routing_indices[e, b] = 1-based slot or 0, the list of active experts with its count in the last
        entry.  The logits are left untouched.  `local_experts`: as for the sigmoid routing (the reference task's
        start_expert / end_expert)."""
        assert input.num_dims == 2 and len(output) == 3
        w, idx, mask = output
        assert w.num_dims == 2 and idx.num_dims == 2 and mask.num_dims == 1
        params = [] if local_experts is None else [int(local_experts[0]), int(local_experts[1])]
        self._layer(N.OP_MOE_TOPK_SOFTMAX, [input, w, idx, mask], grid_dim, params)

    def silu_mul_layer(self, input: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2 and output.num_dims == 2
        self._layer(N.OP_SILU_MUL, [input, output], grid_dim)

    def allreduce_layer(self, input: DTensor, buffer: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 2 and buffer.num_dims == 3 and output.num_dims == 2
        self._layer(N.OP_ALLREDUCE, [input, buffer, output], grid_dim, [self.world_size, self.mpi_rank])

    def argmax_partial_layer(self, input: DTensor, output: Tuple[DTensor, DTensor], grid_dim: tuple,
                             block_dim: tuple):
        assert input.num_dims == 2 and len(output) == 2
        value, index = output
        self.argmax_partial_output_size = input.dim(1) // grid_dim[0]
        self._layer(N.OP_ARGMAX_PARTIAL, [input, value, index], grid_dim, [grid_dim[0]])

    def argmax_reduce_layer(self, input: Tuple[DTensor, DTensor], output: DTensor, grid_dim: tuple,
                            block_dim: tuple):
        assert len(input) == 2
        self._layer(N.OP_ARGMAX_REDUCE, [input[0], input[1], output], grid_dim)

    def argmax_exchange_layer(self, input: Tuple[DTensor, DTensor], output: DTensor, first_column: int):
        """Merge of argmax partials over a vocabulary that is sharded across the tensor-parallel ranks.

        No reference counterpart (the reference keeps the whole lm_head on every rank).  `input` are this rank's
        partial (value, index) tensors over ITS logits columns, `first_column` the vocabulary column of its column 0.
        Every rank pushes its best pair to all peers inside the megakernel and writes the same global winner
        (largest value, lowest column on ties) to `output`."""
        assert len(input) == 2 and self.world_size > 1
        self._layer(N.OP_ARGMAX_EXCHANGE, [input[0], input[1], output], (1, 1, 1), [int(first_column)])

    def sampling_sm100_layer(self, logits: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple,
                             seed: int = 42):
        """Gumbel-max sampling of one token id per row of `logits` (python/mirage/mpk/persistent_kernel.py:1968-1986).

        Same result as the reference task: key = bf16(logit) + bf16(gumbel noise) in bf16, largest key wins, equal
        keys go to the highest index; the noise of column j is element j % 4 of the Philox4x32-10 block with
        key `seed`, subsequence (row % rows_per_task) * V + 4 * (j // 4), offset 0 -- the same noise every
        iteration, as in the reference (its philox offset is the constant 0).  `grid_dim[0]` says how many tasks
        the reference would cut the rows into, which fixes rows_per_task; here the vocabulary is cut into one
        column range per worker and a last task merges them, as for argmax.
        """
        assert logits.num_dims == 2 and output.num_dims == 2
        rows = logits.dim(0)
        rows_per_task = max(1, rows // max(int(grid_dim[0]), 1))
        n_part = max(1, min(self.num_workers if self.num_workers > 0 else 148, logits.dim(1) // 256))
        k = self._num_sampling_layers = getattr(self, "_num_sampling_layers", 0) + 1
        key = self.new_tensor(dims=(rows, n_part), dtype=bfloat16, name=f"sampling_part_key_{k}")
        idx = self.new_tensor(dims=(rows, n_part), dtype=int64, name=f"sampling_part_index_{k}")
        self._layer(N.OP_SAMPLING_PARTIAL, [logits, key, idx], (n_part, 1, 1), [int(seed), rows_per_task])
        self._layer(N.OP_SAMPLING_REDUCE, [key, idx, output], (1, 1, 1))

    def elementwise_add_layer(self, input_a: DTensor, input_b: DTensor, output: DTensor, grid_dim: tuple,
                              block_dim: tuple):
        self._layer(N.OP_ELEMENTWISE_ADD, [input_a, input_b, output], grid_dim)

    def quantize_fp8_layer(self, input: DTensor, output_fp8: DTensor, output_scale: DTensor, grid_dim: tuple,
                           block_dim: tuple, scale_ue8m0: bool = True):
        """bf16 -> e4m3 with one scale per (token, 128 columns): packed UE8M0 uint32 (for linear_fp8_layer) or
        float32 (`scale_ue8m0=False`, for the MoE grouped GEMM)."""
        self._layer(N.OP_QUANTIZE_FP8, [input, output_fp8, output_scale], grid_dim, [1 if scale_ue8m0 else 0])

    def linear_fp8_layer(self, input_fp8: DTensor, input_scale: DTensor, weight_fp8: DTensor, weight_scale: DTensor,
                         output: DTensor, grid_dim: tuple, block_dim: tuple):
        self._layer(N.OP_LINEAR_FP8, [input_fp8, input_scale, weight_fp8, weight_scale, output], grid_dim)

    def linear_fp8_with_residual_layer(self, input_fp8: DTensor, input_scale: DTensor, weight_fp8: DTensor,
                                       weight_scale: DTensor, residual: DTensor, output: DTensor, grid_dim: tuple,
                                       block_dim: tuple):
        self._layer(N.OP_LINEAR_FP8_RESIDUAL, [input_fp8, input_scale, weight_fp8, weight_scale, residual, output],
                    grid_dim, [1])

    # ---- mixture of experts (persistent_kernel.py:1385-1704 of the reference) -------------------------------
    def moe_topk_sigmoid_routing_layer(self, input: DTensor, bias: DTensor, output: tuple, grid_dim: tuple,
                                       block_dim: tuple, num_groups: int = 8, topk_group: int = 4,
                                       routed_scaling_factor: float = 2.5, local_experts: tuple = None):
        """input [B, E] logits (zeroed by the task), bias [E] float32; output = (topk_weight [B, topk] float32,
        routing_indices [E, B] int32 holding slot + 1 or 0, mask [E + 1] int32: active experts, count last)."""
        import struct
        assert input.num_dims == 2 and bias.num_dims == 1 and len(output) == 3
        w, idx, mask = output
        assert w.num_dims == 2 and idx.num_dims == 2 and mask.num_dims == 1
        bits = struct.unpack("i", struct.pack("f", routed_scaling_factor))[0]
        # local_experts = (first, one past last): expert parallelism -- the hook the reference's task has as
        # start_expert / end_expert (tasks/blackwell/topk_sigmoid_sm100.cuh:310-323): selection and normalisation over
        # all experts, but only this rank's experts enter the routing table and the active list, and the weights of
        # the other ranks' slots are 0
        params = [num_groups, topk_group, bits]
        if local_experts is not None:
            params += [int(local_experts[0]), int(local_experts[1])]
        self._layer(N.OP_MOE_TOPK_SIGMOID, [input, bias, w, idx, mask], grid_dim, params)

    def moe_w13_linear_layer(self, input: DTensor, weight: DTensor, moe_routing_indices: DTensor, moe_mask: DTensor,
                             output: DTensor, grid_dim: tuple, block_dim: tuple, first_expert: int = 0):
        assert input.num_dims == 2 and weight.num_dims == 3 and output.num_dims == 3
        self._layer(N.OP_MOE_W13_LINEAR, [input, weight, moe_routing_indices, moe_mask, output], grid_dim, [int(first_expert)])

    def moe_w2_linear_layer(self, input: DTensor, weight: DTensor, moe_routing_indices: DTensor, moe_mask: DTensor,
                            output: DTensor, grid_dim: tuple, block_dim: tuple, first_expert: int = 0):
        assert input.num_dims == 3 and weight.num_dims == 3 and output.num_dims == 3
        self._layer(N.OP_MOE_W2_LINEAR, [input, weight, moe_routing_indices, moe_mask, output], grid_dim, [int(first_expert)])

    def moe_w13_fp8_layer(self, input_fp8: DTensor, input_scale: DTensor, weight_fp8: DTensor, weight_scale: DTensor,
                          moe_routing_indices: DTensor, moe_mask: DTensor, output: DTensor, grid_dim: tuple,
                          block_dim: tuple, first_expert: int = 0):
        assert input_fp8.num_dims == 2 and weight_fp8.num_dims == 3 and weight_scale.num_dims == 3
        self._layer(N.OP_MOE_W13_FP8, [input_fp8, input_scale, weight_fp8, weight_scale, moe_routing_indices,
                                       moe_mask, output], grid_dim, [int(first_expert)])

    def moe_w2_fp8_layer(self, input_fp8: DTensor, input_scale: DTensor, weight_fp8: DTensor, weight_scale: DTensor,
                         moe_routing_indices: DTensor, moe_mask: DTensor, output: DTensor, grid_dim: tuple,
                         block_dim: tuple, first_expert: int = 0):
        assert input_fp8.num_dims == 3 and weight_fp8.num_dims == 3 and weight_scale.num_dims == 3
        self._layer(N.OP_MOE_W2_FP8, [input_fp8, input_scale, weight_fp8, weight_scale, moe_routing_indices,
                                      moe_mask, output], grid_dim, [int(first_expert)])

    def moe_silu_mul_layer(self, input: DTensor, output: DTensor, grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 3 and output.num_dims == 3
        self._layer(N.OP_MOE_SILU_MUL, [input, output], grid_dim)

    def moe_mul_sum_add_layer(self, input: DTensor, weight: DTensor, residual: DTensor, output: DTensor,
                              grid_dim: tuple, block_dim: tuple):
        assert input.num_dims == 3 and weight.num_dims == 2 and residual.num_dims == 2 and output.num_dims == 2
        self._layer(N.OP_MOE_MUL_SUM_ADD, [input, weight, residual, output], grid_dim)

    # ---- multi-head latent attention (persistent_kernel.py:995-1363 of the reference) ------------------------
    # softmax scale the reference's generated call sites hard-code for DeepSeek-V3
    MLA_DEFAULT_SCALE = (1.0 / math.sqrt(192.0)) * (0.1 * math.log(40.0) + 1.0) ** 2

    def mla_kv_gather_layer(self, c_latent_new: DTensor, k_pe_new: DTensor, paged_cache: DTensor,
                            contiguous_kv: DTensor, mla_params: tuple, grid_dim: tuple, block_dim: tuple):
        """Appends each request's new [c_latent | k_pe] rows to the paged cache [pages, page, 576].  The decode
        layers that are handed `contiguous_kv` read the paged cache in place, so no copy of the sequence is made
        and `contiguous_kv` stays untouched."""
        d_k, d_v, page_size = mla_params
        self._mla_paged[contiguous_kv.id] = (paged_cache, int(page_size))
        self._layer(N.OP_MLA_KV_GATHER, [c_latent_new, k_pe_new, paged_cache, contiguous_kv], grid_dim,
                    [d_k, d_v, page_size])

    def _mla_decode(self, q_input, kv_input, output_partial, output_lse, q_len, kv_len, sm_scale):
        import struct
        heads = q_input.dims[-1] // 576
        scale = self.MLA_DEFAULT_SCALE if sm_scale is None else float(sm_scale)
        bits = struct.unpack("i", struct.pack("f", scale))[0]
        cache, page = self._mla_paged.get(kv_input.id, (kv_input, 0))
        splits = (kv_len + 127) // 128
        self._layer(N.OP_MLA_DECODE, [q_input, cache, output_partial, output_lse], (1, 1, 1),
                    [heads, q_len, kv_len, splits, bits, page])

    def _mla_reduce(self, input_partial, input_lse, output, kv_len):
        heads = output.dims[-1] // 512 if output.num_dims == 2 else output.dims[-2]
        self._layer(N.OP_MLA_REDUCE, [input_partial, input_lse, output], (1, 1, 1), [heads, (kv_len + 127) // 128])

    def mla_mtp_decode_layer(self, q_input: DTensor, kv_input: DTensor, output_partial: DTensor, output_lse: DTensor,
                             q_len: int, kv_len: int, sm_scale: float = None):
        """q [tokens, heads * 576]; kv: the `contiguous_kv` of a preceding mla_kv_gather_layer (the paged cache is
        then read with the batch's page tables) or a dense [requests * kv_len, 576] tensor with `q_len` tokens per
        request; partial O (bf16) and LSE (float32) buffers for `ceil(kv_len / 128)` splits."""
        self._mla_decode(q_input, kv_input, output_partial, output_lse, q_len, kv_len, sm_scale)

    def mla_mtp_reduce_layer(self, input_partial: DTensor, input_lse: DTensor, output: DTensor, q_len: int,
                             kv_len: int):
        self._mla_reduce(input_partial, input_lse, output, kv_len)

    # tensor-parallel variants: the local head count comes from the q tensor, the task bodies are the same
    mla_mtp_decode_tp2_layer = mla_mtp_decode_tp4_layer = mla_mtp_decode_tp8_layer = mla_mtp_decode_layer
    mla_mtp_decode_tp2_reduce_layer = mla_mtp_decode_tp4_reduce_layer = mla_mtp_decode_tp8_reduce_layer = \
        mla_mtp_reduce_layer

    def mla_decode_layer(self, q_input: DTensor, kv_input: DTensor, output_partial: DTensor, output_lse: DTensor,
                         mla_params: tuple, grid_dim: tuple, block_dim: tuple, q_len: int = 1, sm_scale: float = None):
        if len(mla_params) == 6:
            num_heads, d_k, d_v, num_splits, kv_len, q_len = mla_params
        else:
            num_heads, d_k, d_v, num_splits, kv_len = mla_params
        self._mla_decode(q_input, kv_input, output_partial, output_lse, q_len, kv_len, sm_scale)

    def mla_reduce_layer(self, input_partial: DTensor, input_lse: DTensor, output: DTensor, mla_params: tuple,
                         grid_dim: tuple, block_dim: tuple, q_len: int = 1):
        num_splits = mla_params[2]
        self._mla_reduce(input_partial, input_lse, output, num_splits * 128)

    def tensor_init_layer(self, input: DTensor, dummy_input: DTensor = None, dummy_output: DTensor = None,
                          grid_dim: tuple = (1, 1, 1), block_dim: tuple = (128, 1, 1)):
        self._layer(N.OP_TENSOR_INIT, [input], grid_dim)

    # ------------------------------------------------------------------ compile / run
    def compile(self, **kwargs):
        """Cut the layers into the task schedule and upload it.  `output_dir`, if given, receives the
        task-graph dump (the reference writes its generated .cu/.json there); `eos_token_id` may be
        overridden as in the reference."""
        assert not self._is_compiled, "compile() called twice"
        if "eos_token_id" in kwargs and kwargs["eos_token_id"] is not None:
            assert kwargs["eos_token_id"] == self.eos_token_id or self.eos_token_id == -1, \
                "eos_token_id must be given to the constructor"
        if getattr(self, "_pending_split_kv", None):
            raise ValueError("paged_attention_split_kv_layer without its paged_attention_split_kv_merge_layer")
        N.check(self._h, N.lib.mpk_compile(self._h))
        self._is_compiled = True
        if self.world_size > 1 and not self.dry_run and kwargs.get("link_peers", True):
            # (link_peers=False: the caller maps the peers itself, e.g. multigpu.link_local for ranks that live
            # in one process)
            from .multigpu import exchange_comm_handles
            exchange_comm_handles(self)
        out_dir = kwargs.get("output_dir")
        if out_dir:
            os.makedirs(out_dir, exist_ok=True)
            with open(os.path.join(out_dir, f"task_graph_rank{self.mpi_rank}.json"), "w") as f:
                f.write(self.dump_task_graph())

    def load_mpk_kernel(self, output_dir: str, skip_validation: bool = False):
        """The reference reloads a cached nvcc build here; this runtime has nothing to cache."""
        if not self._is_compiled:
            self.compile()

    def dump_task_graph(self) -> str:
        n = N.lib.mpk_dump_task_graph(self._h, None, 0)
        if n < 0:
            N.check(self._h, int(n))
        buf = C.create_string_buffer(int(n))
        N.lib.mpk_dump_task_graph(self._h, buf, n)
        return buf.value.decode()

    def graph_info(self) -> Dict[str, int]:
        a, b, c, d = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        N.check(self._h, N.lib.mpk_graph_info(self._h, C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
        return {"num_tasks": a.value, "num_events": b.value, "num_workers": c.value, "num_folded": d.value,
                "weight_bytes_per_step": int(N.lib.mpk_weight_bytes_per_step(self._h))}

    def _stream_ptr(self, stream) -> int:
        if self.dry_run:
            return 0
        if stream is None:
            stream = torch.cuda.current_stream()
        if hasattr(stream, "cuda_stream"):
            return int(stream.cuda_stream)
        if isinstance(stream, int):
            return stream
        raise ValueError("Invalid stream object")

    def reset(self, stream=None):
        """Back to the state a fresh offline run starts from (steps 0, empty slots, full page ring).

        With peers linked through torch.distributed this is a collective: a rank's first launch after the reset
        pushes partial sums into its peers' inboxes, so no rank may launch before every rank's clearing has
        finished (a late clearing would wipe pushes that already arrived and the peer would wait for them until
        its bounded wait expires), and no rank may clear while a peer's earlier launch is still pushing."""
        fence = getattr(self, "_dist_linked", False) and self.world_size > 1
        if fence:
            from .multigpu import rank_fence
            rank_fence(self, stream)
        N.check(self._h, N.lib.mpk_reset(self._h, self._stream_ptr(stream)))
        if fence:
            rank_fence(self, stream)

    def step(self, num_steps: int = 1, stream=None):
        """Enqueue `num_steps` decode iterations (one megakernel launch each).  Asynchronous."""
        assert self._is_compiled, "Must call compile() first"
        if getattr(self, "_timed_out", False):
            # the previous status() reported an expired device wait: clear counters and inboxes first -- through
            # reset(), which fences the ranks when peers are linked (the library refuses to do it silently then)
            self._timed_out = False
            self.reset(stream)
        N.check(self._h, N.lib.mpk_launch(self._h, self._stream_ptr(stream), int(num_steps)))

    def status(self, stream=None) -> N.MpkStatus:
        """Synchronise and return the device status; raises MpkTimeoutError if a device wait expired."""
        st = N.MpkStatus()
        try:
            N.check(self._h, N.lib.mpk_sync_status(self._h, self._stream_ptr(stream), C.byref(st)))
        except N.MpkTimeoutError:
            self._timed_out = True
            raise
        return st

    def __call__(self, **kwargs):
        """Run the whole generation like the reference's launch: iterate until no request is left
        (offline mode), or run the graph once (online_notoken / test mode)."""
        stream = kwargs.get("default_stream", None)
        if self.test_mode or self.mode == "online_notoken":
            self.step(1, stream)
            return
        self.reset(stream)
        chunk = int(kwargs.get("steps_per_poll", 32))
        max_iters = int(kwargs.get("max_iterations", self.total_num_requests * self.max_seq_length + 2))
        done = 0
        while done < max_iters:
            n = min(chunk, max_iters - done)
            self.step(n, stream)
            done += n
            if self.status(stream).all_done:
                break

    def run_test_mode(self):
        assert self.test_mode, "run_test_mode() is only available in test mode"
        assert self._is_compiled, "Must call compile() before run_test_mode()"
        self.step(1)
        self.status()

    run = run_test_mode

    def finalize(self):
        if self.__finalized__:
            return
        self.__finalized__ = True
        if getattr(self, "_h", None):
            N.lib.mpk_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.finalize()
        except Exception:
            pass
