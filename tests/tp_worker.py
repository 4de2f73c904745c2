"""Tensor-parallel parity worker: run under torchrun, one rank per GPU.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 tests/tp_worker.py

Every rank builds its shard of a small Qwen3-architecture decoder, all ranks step the megakernel
together, and every rank compares its logits and the chosen token ids with the CPU oracle's TP=1 result.  With
TP_SHARD_LM_HEAD=1 the lm_head is sharded: a rank holds the logits of its own vocabulary columns and the ranks
exchange their argmax results inside the kernel.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle.qwen3_decoder import Qwen3Config, make_weights  # noqa: E402
from gpu_util import lockstep_compare, shape_of  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mirage_b200.builders.runner import Qwen3Runner
    cfg = Qwen3Config(num_layers=3, hidden_size=512, num_q_heads=16, num_kv_heads=8, head_dim=128,
                      intermediate_size=2048, vocab_size=2048, max_position=256)
    w = make_weights(cfg, seed=1005)
    g = torch.Generator().manual_seed(2005)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 4, 13)]
    kw = dict(max_seq_length=40, max_num_pages=12, page_size=8)
    mbr, mbt = 2, 4
    r = Qwen3Runner(shape_of(cfg), w, total_num_requests=len(prompts), max_num_batched_requests=mbr,
                    max_num_batched_tokens=mbt, world_size=world, rank=rank, device=local,
                    shard_lm_head=os.environ.get("TP_SHARD_LM_HEAD", "0") == "1", **kw)
    worst, _ = lockstep_compare(r, cfg, w, prompts, mbr=mbr, mbt=mbt, iterations=60, **kw)
    t = torch.tensor([worst], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"TP={world} parity ok: max |logit diff| vs oracle {t.item():.4f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
