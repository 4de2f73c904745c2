"""`MPKMetadata` / `MPK`: the caller-facing wrapper the reference puts around its persistent kernel
(python/mirage/mpk/mpk.py:15-434) -- one object that owns the meta tensors, builds the model graph through a
registered builder, compiles it and runs generations.

Kept from the reference: the metadata fields and their meaning, `compensate_meta_tensors` (any meta tensor the
caller does not bring is allocated), `clear_buffers`, `build` / `compile` / `__call__`, the per-request
re-initialisation (`init_per_request`), rank / world size taken from the environment.  Left out on purpose:
loading HuggingFace checkpoints and tokenizers (`weight_from_model=True`), which need files this library does not
read -- prompts go in as token ids (`load_new_request_ids`), text handling stays with the caller.  Extension:
`run_steps(n)` runs n iterations (one launch each) without waiting for the end of the generation, which is what an
online serving loop needs.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .persistent_kernel import PersistentKernel

_BUILDERS: Dict[str, type] = {}


def register_model_builder(*names):
    """Same contract as python/mirage/mpk/model_registry.py: a class decorator that files a graph builder."""
    def deco(cls):
        for n in names:
            _BUILDERS[n.lower()] = cls
        return cls
    return deco


def get_builder(name: str):
    key = (name or "").lower()
    for k, v in _BUILDERS.items():
        if k in key:
            return v
    raise KeyError(f"no graph builder registered for model '{name}' (known: {sorted(_BUILDERS)})")


@dataclass
class MPKMetadata:
    mode: str = "offline"
    total_num_requests: int = 1
    num_remote_schedulers: int = 0
    max_seq_length: int = 0
    max_num_batched_requests: int = 0
    max_num_batched_tokens: int = 0
    max_num_pages: int = 0
    page_size: int = 0
    max_sm_num: int = 148
    device: str = "cuda"
    weight_from_model: bool = False
    model_name: Optional[str] = None
    model_path: Optional[str] = None
    world_size: int = 1
    rank: int = 0
    num_workers: int = -1
    num_schedulers: int = -1
    step: Optional[torch.Tensor] = None
    tokens: Optional[torch.Tensor] = None
    input_tokens: Optional[torch.Tensor] = None
    output_tokens: Optional[torch.Tensor] = None
    num_new_tokens: Optional[torch.Tensor] = None
    prompt_lengths: Optional[torch.Tensor] = None
    qo_indptr_buffer: Optional[torch.Tensor] = None
    paged_kv_indptr_buffer: Optional[torch.Tensor] = None
    paged_kv_indices_buffer: Optional[torch.Tensor] = None
    paged_kv_last_page_len_buffer: Optional[torch.Tensor] = None
    model_config: Optional[object] = None       # e.g. builders.qwen3.Qwen3ModelConfig (the MirageModelConfig role)
    profiling: bool = False
    profiler_tensor: Optional[torch.Tensor] = None
    trace_name: Optional[str] = None
    spec_decode: Optional[str] = None
    spec_decode_config: Optional[object] = None
    use_cutlass_kernel: bool = True
    eos_token_id: int = -1
    dry_run: bool = False                        # build and check the task graph only (no CUDA call)

    def check_valid(self):
        if self.weight_from_model:
            raise NotImplementedError("weight_from_model=True: loading checkpoints is outside this library; pass "
                                      "model_config.state_dict")
        assert self.model_config is not None and self.model_config.state_dict is not None, \
            "state_dict is required when weight_from_model is False"
        assert self.model_config.k_cache is not None and self.model_config.v_cache is not None

    def info_as_string(self) -> str:
        shape = lambda t: tuple(t.shape) if t is not None else None
        fields = ["mode", "total_num_requests", "max_seq_length", "max_num_batched_requests", "max_num_batched_tokens",
                  "max_num_pages", "page_size", "device", "model_name", "world_size", "rank"]
        out = ["MPKMetadata info:"] + [f"{f}: {getattr(self, f)}" for f in fields]
        for f in ("step", "tokens", "input_tokens", "output_tokens", "num_new_tokens", "prompt_lengths",
                  "qo_indptr_buffer", "paged_kv_indptr_buffer", "paged_kv_indices_buffer",
                  "paged_kv_last_page_len_buffer", "profiler_tensor"):
            out.append(f"{f}: {shape(getattr(self, f))}")
        return "\n".join(out) + "\n"

    def print_info(self):
        print(self.info_as_string())


class MPK:
    META_NAMES = ("step", "tokens", "input_tokens", "output_tokens", "num_new_tokens", "prompt_lengths",
                  "qo_indptr_buffer", "paged_kv_indptr_buffer", "paged_kv_indices_buffer",
                  "paged_kv_last_page_len_buffer")

    def __init__(self, meta: MPKMetadata):
        self.metadata = meta
        # ranks come from the launcher's environment (torchrun); the reference asks MPI (mpk.py:223-238)
        self.world_size = int(os.environ.get("WORLD_SIZE", meta.world_size))
        self.rank = int(os.environ.get("RANK", meta.rank))
        self.device = "meta" if meta.dry_run else meta.device
        self.total_num_requests = meta.total_num_requests
        self.max_seq_length = meta.max_seq_length
        self.max_num_batched_requests = meta.max_num_batched_requests
        self.max_num_batched_tokens = meta.max_num_batched_tokens
        self.max_num_pages = meta.max_num_pages
        self.page_size = meta.page_size
        for n in self.META_NAMES:
            setattr(self, n, getattr(meta, n))
        self.need_cpy_input = False
        self.src_input_tokens = None
        if self.input_tokens is not None and self.input_tokens.dtype != torch.int64:
            # callers that keep int32 ids get a private int64 copy that is refreshed before every run
            self.need_cpy_input, self.src_input_tokens = True, self.input_tokens
            self.input_tokens = torch.empty_like(self.src_input_tokens, dtype=torch.int64)
        self.profiler_tensor = meta.profiler_tensor
        if meta.profiling and self.profiler_tensor is None:
            self.profiler_tensor = torch.zeros(3000 * 128, dtype=torch.int64, device=self.device)
        self.compensate_meta_tensors()
        self.model_config = meta.model_config
        self.persistent_kernel = PersistentKernel(
            mode=meta.mode, world_size=self.world_size, mpi_rank=self.rank,
            num_workers=max(meta.num_workers, 0), num_local_schedulers=max(meta.num_schedulers, 0),
            num_remote_schedulers=0, max_seq_length=self.max_seq_length,
            max_num_batched_requests=self.max_num_batched_requests, max_num_batched_tokens=self.max_num_batched_tokens,
            max_num_pages=self.max_num_pages, page_size=self.page_size,
            meta_tensors={n: getattr(self, n) for n in self.META_NAMES}, profiler_tensor=self.profiler_tensor,
            trace_name=meta.trace_name, spec_decode_config=meta.spec_decode_config,
            use_cutlass_kernel=meta.use_cutlass_kernel, eos_token_id=meta.eos_token_id, dry_run=meta.dry_run)
        self.is_built = False
        self.is_compiled = False

    # -- python/mirage/mpk/mpk.py:240-281
    def compensate_meta_tensors(self):
        dev = self.device
        R, S, T, Q, P = (self.total_num_requests, self.max_seq_length, self.max_num_batched_tokens,
                         self.max_num_batched_requests, self.max_num_pages)
        default = {
            "step": lambda: torch.zeros(R, dtype=torch.int32, device=dev),
            "tokens": lambda: torch.zeros(R, S, dtype=torch.int64, device=dev),
            "input_tokens": lambda: torch.zeros(T, 1, dtype=torch.int64, device=dev),
            "output_tokens": lambda: torch.zeros(T, 1, dtype=torch.int64, device=dev),
            "num_new_tokens": lambda: torch.ones(R, dtype=torch.int32, device=dev),
            "prompt_lengths": lambda: torch.zeros(R, dtype=torch.int32, device=dev),
            "qo_indptr_buffer": lambda: torch.zeros(Q + 1, dtype=torch.int32, device=dev),
            "paged_kv_indptr_buffer": lambda: torch.zeros(Q + 1, dtype=torch.int32, device=dev),
            "paged_kv_indices_buffer": lambda: torch.zeros(P, dtype=torch.int32, device=dev),
            "paged_kv_last_page_len_buffer": lambda: torch.zeros(Q, dtype=torch.int32, device=dev),
        }
        for n, make in default.items():
            if getattr(self, n) is None:
                setattr(self, n, make())

    # -- python/mirage/mpk/mpk.py:329-340
    def clear_buffers(self):
        for n in self.META_NAMES:
            getattr(self, n).fill_(0)

    def build(self):
        """Registers the model's layers on the persistent kernel through the builder filed for `model_name`."""
        self.metadata.check_valid()
        self.model_builder = get_builder(self.metadata.model_name or "qwen3")(self.persistent_kernel)
        self.model_builder.build_from_config(self.model_config)
        self.with_lm_head = bool(getattr(self.model_config, "with_lm_head", True))
        self.is_built = True

    def compile(self, **kwargs):
        assert self.is_built, "build() first"
        self.persistent_kernel.compile(**kwargs)
        self.is_compiled = True

    def load_new_request_ids(self, prompts: Sequence[Sequence[int]]):
        """Token-id form of load_new_request (mpk.py:302-327): one prompt per request slot."""
        assert len(prompts) <= self.total_num_requests
        self.tokens.zero_()
        self.prompt_lengths.zero_()
        for r, p in enumerate(prompts):
            assert 0 < len(p) < self.max_seq_length
            self.tokens[r, :len(p)] = torch.tensor(list(p), dtype=torch.int64)
            self.prompt_lengths[r] = len(p)

    def init_per_request(self):
        """init_request_func of the reference: scheduler state back to 'nothing started'."""
        self.persistent_kernel.reset()

    def run_steps(self, iterations: int = 1):
        """`iterations` decode iterations (one launch each), asynchronous on the current stream."""
        if self.need_cpy_input:
            self.input_tokens.copy_(self.src_input_tokens)
        self.persistent_kernel.step(iterations)

    def __call__(self, **kwargs):
        """Offline: the whole generation.  online_notoken: ONE forward over the batch the caller described in the meta
        tensors (qo_indptr / paged_kv_* / input_tokens are the caller's; no scheduling happens on the device); without
        an lm_head the final-norm output of the batched tokens is returned (python/mirage/mpk/mpk.py:417-426)."""
        if not self.is_compiled:
            self.compile()
        if self.need_cpy_input:
            self.input_tokens.copy_(self.src_input_tokens)
        self.persistent_kernel(**kwargs)
        if not self.with_lm_head and self.persistent_kernel.mode == "online_notoken":
            return self.model_builder.returned_hidden_state
        return None

    def run_ids(self, prompts: Sequence[Sequence[int]]) -> List[List[int]]:
        """mpk.run (mpk.py:372-385) on token ids: whole generation for every request, returns the id sequences."""
        self.load_new_request_ids(prompts)
        self.init_per_request()
        self()
        torch.cuda.synchronize()
        steps = self.step_tensor_host()
        return [self.tokens[r, :steps[r] + 1].tolist() for r in range(len(prompts))]

    def step_tensor_host(self) -> List[int]:
        return self.step.cpu().tolist() if isinstance(self.step, torch.Tensor) else []
