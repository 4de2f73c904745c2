"""DeepSeek-V3-architecture slice end to end: the megakernel against the composed CPU oracle, iteration by iteration.

Small shape of the same architecture (hidden 1024, 32 heads with 512-wide latent + 64 rope, 16 experts top-4 in 4
groups + shared expert, 1 dense + 1 MoE layer), FP8 projections and experts with 128 x 128 block scales.  Bars: logits
within 0.35 abs and greedy ids equal where the oracle's top-2 gap exceeds 0.7 -- the FP8 bars of
tests/test_gpu_qwen3_fp8.py (per-token activation quantisation amplifies one-ulp differences upstream into e4m3
steps; measured in tests/test_fp8_oracle.py) -- and the batching state bit-exact.  The two-rank case runs both ranks
on ONE device (64 worker CTAs each, linked with mpk_comm_link_local): heads, dense MLP and shared expert tensor
parallel, routed experts 8 per rank, allreduces after o_proj, the dense MLP and the MoE block."""
import dataclasses

import numpy as np
import pytest
import torch

from oracle.batching import BatchState
from oracle.deepseek_v3 import DeepSeekConfig, DeepSeekOracle, make_checkpoint
from gpu_util import lockstep_compare

pytestmark = pytest.mark.gpu


def _shape(cfg):
    from mirage_b200.builders.deepseek_v3 import DeepSeekV3Shape
    return DeepSeekV3Shape(**{f.name: getattr(cfg, f.name) for f in dataclasses.fields(DeepSeekV3Shape)})


def _prompts(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in lengths]


def test_slice_matches_the_oracle_on_one_gpu():
    from mirage_b200.builders.deepseek_v3 import DeepSeekV3Runner
    cfg = DeepSeekConfig.tiny()
    ckpt = make_checkpoint(cfg, seed=1005)
    prompts = _prompts(cfg, (9, 4, 13), 2005)
    kw = dict(max_seq_length=48, max_num_pages=12, page_size=16)
    mbr, mbt = 2, 4
    r = DeepSeekV3Runner(_shape(cfg), ckpt, total_num_requests=len(prompts), max_num_batched_requests=mbr,
                         max_num_batched_tokens=mbt, **kw)
    factory = lambda **okw: DeepSeekOracle(cfg, ckpt, **okw)
    worst, _ = lockstep_compare(r, cfg, None, prompts, mbr=mbr, mbt=mbt, iterations=40, logit_tol=0.35, id_gap=0.7,
                                oracle_factory=factory, **kw)
    print(f"max |logit diff| vs oracle {worst:.4f}")


def test_two_ranks_with_expert_parallelism_on_one_device():
    from mirage_b200.builders.deepseek_v3 import DeepSeekV3Runner
    from mirage_b200.multigpu import link_local
    cfg = DeepSeekConfig.tiny()
    ckpt = make_checkpoint(cfg, seed=1006)
    batch = 4
    prompts = _prompts(cfg, (5, 3, 8, 6), 2006)
    max_seq, page = 32, 16
    pages = batch * (max_seq // page)
    kw = dict(max_seq_length=max_seq, max_num_pages=pages, page_size=page)
    runners = [DeepSeekV3Runner(_shape(cfg), ckpt, total_num_requests=batch, max_num_batched_requests=batch,
                                max_num_batched_tokens=batch, world_size=2, rank=r, device=0, num_workers=64,
                                link_peers=False, **kw) for r in (0, 1)]
    link_local([r.mpk for r in runners])
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    tokens = np.zeros((batch, max_seq), np.int64)
    plen = np.zeros(batch, np.int32)
    for i, p in enumerate(prompts):
        tokens[i, :len(p)] = p
        plen[i] = len(p)
    st = BatchState(tokens, plen, max_num_batched_requests=batch, max_num_batched_tokens=batch, max_num_pages=pages,
                    page_size=page)
    orc = DeepSeekOracle(cfg, ckpt, max_num_pages=pages, page_size=page, world_size=2)
    for r in runners:
        r.load_prompts(prompts)
    torch.cuda.synchronize()
    worst = 0.0
    for it in range(20):
        more = orc.run_iteration(st)
        for r, s in zip(runners, streams):          # both launches are enqueued before either is waited for
            r.mpk.step(1, stream=s)
        stats = [r.mpk.status(stream=s) for r, s in zip(runners, streams)]
        n = st.num_active_tokens
        for r, status in zip(runners, stats):
            assert status.error == 0 and status.active_tokens == n and bool(status.all_done) == (not more)
            assert r.meta["step"].cpu().numpy().tolist() == st.step.tolist()
        if not more:
            break
        ref = orc.last_logits.float()
        top2 = ref.topk(2, dim=-1).values
        gap = (top2[:, 0] - top2[:, 1]).numpy()
        outs = []
        for rank, r in enumerate(runners):
            got = r.logits[:n].float().cpu()
            worst = max(worst, float((got - ref).abs().max()))
            assert worst <= 0.35, f"iteration {it} rank {rank}: logits differ by {worst}"
            out = r.meta["output_tokens"].cpu().numpy().reshape(-1)[:n]
            for b in range(n):
                if gap[b] > 0.7:
                    assert out[b] == st.output_tokens[b], f"iteration {it} rank {rank} token {b}"
            outs.append(out)
        # the ranks sum the same partials in the same order: identical hidden states, logits and ids
        assert outs[0].tolist() == outs[1].tolist()
        assert torch.equal(runners[0].logits[:n].cpu(), runners[1].logits[:n].cpu())
        st.output_tokens[:n] = outs[0]
    assert it >= 8
    print(f"max |logit diff| vs oracle {worst:.4f}")
