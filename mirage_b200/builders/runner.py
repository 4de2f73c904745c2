"""Convenience wrapper: allocate the meta tensors / KV cache / RoPE tables a Qwen3 decode run needs and
build the PersistentKernel for it.  Used by the benchmark, the smoke test and the GPU tests; plays the
part of the argument handling in the reference's demo/qwen3/demo.py:150-330."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..persistent_kernel import PersistentKernel
from .qwen3 import Qwen3Builder, Qwen3ModelConfig, shard_fp8_state_dict, shard_state_dict


def rope_tables(head_dim: int, max_pos: int, theta: float, device) -> tuple:
    """bf16 cos/sin tables in the half-split layout (cos/sin of position * theta^(-2i/d), repeated twice),
    computed in fp32 like demo/qwen3/models/modeling_qwen3.py:94-117."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(torch.bfloat16).to(device), emb.sin().to(torch.bfloat16).to(device)


@dataclass
class DecoderShape:
    num_layers: int
    hidden_size: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float = 1e6
    max_position: int = 4096


class Qwen3Runner:
    """Owns the device state of one rank and the compiled megakernel."""

    def __init__(self, shape: DecoderShape, state_dict: Dict[str, torch.Tensor], *, total_num_requests: int,
                 max_seq_length: int, max_num_batched_requests: int, max_num_batched_tokens: int,
                 max_num_pages: int, page_size: int, eos_token_id: int = -1, world_size: int = 1, rank: int = 0,
                 device: Optional[int] = None, num_workers: int = 0, sampling_seed: Optional[int] = None,
                 shard_lm_head: bool = False,
                 fp8_state_dict: Optional[Dict[str, tuple]] = None, link_peers: bool = True,
                 presharded: bool = False):
        """`state_dict` / `fp8_state_dict` hold the whole model and are cut for this rank here, unless `presharded`:
        then they are this rank's shard already (what `checkpoint.load_sharded_state_dict` returns)."""
        dev = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.device, self.shape = dev, shape
        mbr, mbt = max_num_batched_requests, max_num_batched_tokens
        i32 = dict(dtype=torch.int32, device=dev)
        i64 = dict(dtype=torch.int64, device=dev)
        self.meta = {
            "step": torch.zeros(total_num_requests, **i32),
            "tokens": torch.zeros(total_num_requests, max_seq_length, **i64),
            "input_tokens": torch.zeros(mbt, 1, **i64),
            "output_tokens": torch.zeros(mbt, 1, **i64),
            "num_new_tokens": torch.ones(total_num_requests, **i32),
            "prompt_lengths": torch.zeros(total_num_requests, **i32),
            "qo_indptr_buffer": torch.zeros(mbr + 1, **i32),
            "paged_kv_indptr_buffer": torch.zeros(mbr + 1, **i32),
            "paged_kv_indices_buffer": torch.zeros(max_num_pages, **i32),
            "paged_kv_last_page_len_buffer": torch.zeros(mbr, **i32),
        }
        hkv = shape.num_kv_heads // world_size
        self.k_cache = torch.zeros(shape.num_layers, max_num_pages, page_size, hkv, shape.head_dim,
                                   dtype=torch.bfloat16, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.cos, self.sin = rope_tables(shape.head_dim, shape.max_position, shape.rope_theta, dev)
        sd = state_dict if presharded else shard_state_dict(
            state_dict, world_size, rank, shape.num_q_heads, shape.num_kv_heads, shape.head_dim,
            shard_lm_head=shard_lm_head and sampling_seed is None)
        self.sd = {k: v.to(dev) for k, v in sd.items()}
        self.mpk = PersistentKernel(
            mode="offline", world_size=world_size, mpi_rank=rank, num_workers=num_workers,
            max_seq_length=max_seq_length, max_num_batched_requests=mbr, max_num_batched_tokens=mbt,
            max_num_pages=max_num_pages, page_size=page_size, meta_tensors=self.meta, eos_token_id=eos_token_id,
            device=dev.index)
        cfg = Qwen3ModelConfig(
            hidden_size=shape.hidden_size, intermediate_size=shape.intermediate_size // world_size,
            vocab_size=shape.vocab_size, local_num_q_heads=shape.num_q_heads // world_size,
            local_num_kv_heads=hkv, head_dim=shape.head_dim, num_layers=shape.num_layers,
            k_cache=self.k_cache, v_cache=self.v_cache, position_embeddings=(self.cos, self.sin),
            state_dict=self.sd, sampling_seed=sampling_seed,
            fp8_state_dict=None if fp8_state_dict is None else
            {k: (q.to(dev), s.to(dev)) for k, (q, s) in
             (fp8_state_dict if presharded else shard_fp8_state_dict(fp8_state_dict, world_size, rank)).items()})
        self.builder = Qwen3Builder(self.mpk)
        self.builder.build_from_config(cfg)
        # link_peers=False: ranks that live in one process are mapped by multigpu.link_local afterwards
        self.mpk.compile(link_peers=link_peers)
        # logits of this rank's vocabulary columns [vocab_first, vocab_first + logits.shape[1]) (all of them at TP=1)
        self.logits = self.mpk.tensor_as_torch(self.builder.logits)
        self.vocab_first = self.builder.vocab_first

    @classmethod
    def from_checkpoint(cls, path: str, *, world_size: int = 1, rank: int = 0, shard_lm_head: bool = False,
                        sampling_seed: Optional[int] = None, **kw) -> "Qwen3Runner":
        """Runner over a HuggingFace checkpoint directory (config.json + *.safetensors): every rank reads only its own
        rows / columns from disk; projections stored as float8_e4m3fn with `_scale_inv` block scales select the FP8
        graph.  The remaining keyword arguments are the constructor's."""
        from .checkpoint import load_sharded_state_dict, shape_from_config
        shard_head = shard_lm_head and sampling_seed is None
        sd, fp8 = load_sharded_state_dict(path, world_size, rank, shard_lm_head=shard_head, dtype=torch.bfloat16)
        return cls(shape_from_config(path), sd, world_size=world_size, rank=rank, shard_lm_head=shard_lm_head,
                   sampling_seed=sampling_seed, fp8_state_dict=fp8 or None, presharded=True, **kw)

    def load_prompts(self, prompts: Sequence[Sequence[int]]):
        tok = torch.zeros_like(self.meta["tokens"], device="cpu")
        plen = torch.zeros_like(self.meta["prompt_lengths"], device="cpu")
        for i, p in enumerate(prompts):
            tok[i, :len(p)] = torch.tensor(list(p), dtype=torch.int64)
            plen[i] = len(p)
        self.meta["tokens"].copy_(tok)
        self.meta["prompt_lengths"].copy_(plen)
        self.mpk.reset()

    def step(self, n: int = 1):
        self.mpk.step(n)

    def tokens(self) -> torch.Tensor:
        return self.meta["tokens"].cpu()
