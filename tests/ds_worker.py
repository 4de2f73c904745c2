"""DeepSeek-V3 slice parity worker: run under torchrun, one rank per GPU.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 tests/ds_worker.py

Every rank builds its shard of a small DeepSeek-V3-architecture slice (attention heads, dense MLP and shared expert tensor
parallel, routed experts split by rank), all ranks step the megakernel together, and every rank compares its logits and
token ids with the CPU oracle's emulation of the same partition (tests/test_gpu_deepseek.py has the one-device form).
"""
import dataclasses
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle.deepseek_v3 import DeepSeekConfig, DeepSeekOracle, make_checkpoint  # noqa: E402
from gpu_util import lockstep_compare  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mirage_b200.builders.deepseek_v3 import DeepSeekV3Runner, DeepSeekV3Shape
    cfg = DeepSeekConfig.tiny(num_heads=16 * world)
    shape = DeepSeekV3Shape(**{f.name: getattr(cfg, f.name) for f in dataclasses.fields(DeepSeekV3Shape)})
    ckpt = make_checkpoint(cfg, seed=1005)
    g = torch.Generator().manual_seed(2005)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 4, 13)]
    kw = dict(max_seq_length=48, max_num_pages=12, page_size=16)
    mbr, mbt = 2, 4
    r = DeepSeekV3Runner(shape, ckpt, total_num_requests=len(prompts), max_num_batched_requests=mbr,
                         max_num_batched_tokens=mbt, world_size=world, rank=rank, device=local, **kw)
    factory = lambda **okw: DeepSeekOracle(cfg, ckpt, world_size=world, **okw)
    worst, _ = lockstep_compare(r, cfg, None, prompts, mbr=mbr, mbt=mbt, iterations=40, logit_tol=0.35, id_gap=0.7,
                                oracle_factory=factory, **kw)
    t = torch.tensor([worst], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"DeepSeek slice TP/EP={world} parity ok: max |logit diff| vs oracle {t.item():.4f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
