"""Reads a HuggingFace checkpoint directory (`*.safetensors`, with or without `model.safetensors.index.json`) straight
into one rank's tensor-parallel shard.

The reference gets its weights by instantiating the whole PyTorch model on every rank and slicing the tensors
afterwards (demo/qwen3/demo.py:13-29 for the shard map, :150-330 for the load); here each rank reads only the rows or
columns it owns from disk (`safetensors` slices), so that a rank's host memory and read time are 1 / world of the
checkpoint for everything that is sharded.  The result is exactly `shard_state_dict(full_state_dict, ...)`
(mirage_b200/builders/qwen3.py) -- same names, same slices -- and, for an FP8 checkpoint, the `(e4m3 weight, float32
128 x 128 block scale)` pairs `shard_fp8_state_dict` would give (HF names `<w>.weight` + `<w>.weight_scale_inv`)."""
from __future__ import annotations

import contextlib
import glob
import json
import os
from typing import Dict, Iterable, Optional, Tuple

import torch

ROW_SHARDED = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate_proj.weight", "up_proj.weight")
COLUMN_SHARDED = ("o_proj.weight", "down_proj.weight")
SCALE_SUFFIX = "_scale_inv"


def checkpoint_index(path: str) -> Dict[str, str]:
    """tensor name -> file, from the index file if the directory has one, else by listing every *.safetensors."""
    from safetensors import safe_open
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            return {k: os.path.join(path, v) for k, v in json.load(f)["weight_map"].items()}
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors under {path}")
    out = {}
    for fn in files:
        with safe_open(fn, framework="pt") as f:
            for k in f.keys():
                if k in out:
                    raise ValueError(f"{k} is in both {out[k]} and {fn}")
                out[k] = fn
    return out


def _shard_range(n: int, world_size: int, rank: int, name: str, multiple: int = 1) -> Tuple[int, int]:
    if n % world_size or (n // world_size) % multiple:
        raise ValueError(f"{name}: extent {n} does not split over {world_size} ranks in multiples of {multiple}")
    m = n // world_size
    return rank * m, (rank + 1) * m


def load_sharded_state_dict(path: str, world_size: int = 1, rank: int = 0, *, shard_lm_head: bool = False,
                            names: Optional[Iterable[str]] = None, dtype: Optional[torch.dtype] = None,
                            ) -> Tuple[Dict[str, torch.Tensor], Dict[str, Tuple[torch.Tensor, torch.Tensor]]]:
    """-> (state_dict, fp8_state_dict) of this rank.

    state_dict: every tensor that is not an FP8 projection, under its checkpoint name, cut as `shard_state_dict`
    cuts it (q/k/v/gate/up by output rows, o/down by input columns, lm_head by vocabulary rows iff `shard_lm_head`,
    the rest whole), cast to `dtype` when given.  fp8_state_dict: `{name: (e4m3 [N, K], float32 [N/128, K/128])}`
    for every projection stored as float8_e4m3fn with a `<name>_scale_inv` beside it, cut on 128-row / 128-column
    block borders.  `names` restricts the read (e.g. to the layers of a pipeline stage or of a slice)."""
    from safetensors import safe_open
    index = checkpoint_index(path)
    wanted = set(index) if names is None else set(names)
    missing = wanted - set(index)
    if missing:
        raise KeyError(f"not in the checkpoint: {sorted(missing)[:4]}")
    handles = {}
    plain, fp8 = {}, {}
    with contextlib.ExitStack() as files:
        def get(name):
            fn = index[name]
            if fn not in handles:
                handles[fn] = files.enter_context(safe_open(fn, framework="pt"))
            return handles[fn].get_slice(name)

        for name in sorted(wanted):
            if name.endswith(SCALE_SUFFIX):
                if name[:-len(SCALE_SUFFIX)] not in index:
                    raise KeyError(f"{name} has no weight beside it")
                continue
            sl = get(name)
            shape = sl.get_shape()
            quantised = sl.get_dtype() == "F8_E4M3" and (name + SCALE_SUFFIX) in index
            block = 128 if quantised else 1
            if name.endswith(ROW_SHARDED) or (name == "lm_head.weight" and shard_lm_head and world_size > 1):
                lo, hi = _shard_range(shape[0], world_size, rank, name, block)
                t, cut = sl[lo:hi], (0, lo, hi)
            elif name.endswith(COLUMN_SHARDED):
                lo, hi = _shard_range(shape[1], world_size, rank, name, block)
                t, cut = sl[:, lo:hi], (1, lo, hi)
            else:
                t, cut = sl[:], None
            t = t.contiguous()
            if quantised:
                ssl = get(name + SCALE_SUFFIX)
                if cut is None:
                    sc = ssl[:]
                elif cut[0] == 0:
                    sc = ssl[cut[1] // 128:cut[2] // 128]
                else:
                    sc = ssl[:, cut[1] // 128:cut[2] // 128]
                fp8[name] = (t, sc.to(torch.float32).contiguous())
            else:
                plain[name] = t.to(dtype) if dtype is not None and t.is_floating_point() else t
    return plain, fp8


def shape_from_config(path: str):
    """DecoderShape from the directory's config.json (the fields demo/qwen3/demo.py reads from the HF config)."""
    from .runner import DecoderShape
    with open(os.path.join(path, "config.json")) as f:
        c = json.load(f)
    rope = c.get("rope_theta") or (c.get("rope_parameters") or {}).get("rope_theta", 1e6)
    return DecoderShape(num_layers=c["num_hidden_layers"], hidden_size=c["hidden_size"],
                        num_q_heads=c["num_attention_heads"], num_kv_heads=c["num_key_value_heads"],
                        head_dim=c.get("head_dim", c["hidden_size"] // c["num_attention_heads"]),
                        intermediate_size=c["intermediate_size"], vocab_size=c["vocab_size"], rope_theta=float(rope),
                        max_position=c.get("max_position_embeddings", 4096))
