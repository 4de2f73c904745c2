"""A runner built from a checkpoint DIRECTORY (config.json + model.safetensors written here from the seeded synthetic
weights) decodes in lockstep with the CPU oracle that holds the same weights in memory -- the weight-IO path in front
of the megakernel: file -> this rank's rows / columns -> device -> graph."""
import json

import pytest
import torch
from safetensors.torch import save_file

from oracle.qwen3_decoder import Qwen3Config, make_weights
from gpu_util import lockstep_compare

pytestmark = pytest.mark.gpu


def _write(tmp_path, cfg, w):
    save_file({k: v.contiguous() for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({
        "num_hidden_layers": cfg.num_layers, "hidden_size": cfg.hidden_size, "num_attention_heads": cfg.num_q_heads,
        "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim, "intermediate_size": cfg.intermediate_size,
        "vocab_size": cfg.vocab_size, "rope_theta": cfg.rope_theta, "max_position_embeddings": cfg.max_position}))


def test_runner_from_checkpoint_directory(tmp_path):
    from mirage_b200.builders.runner import Qwen3Runner
    cfg = Qwen3Config.tiny()
    w = make_weights(cfg, seed=1011)
    _write(tmp_path, cfg, w)
    g = torch.Generator().manual_seed(2011)
    prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (5, 9, 3)]
    kw = dict(max_seq_length=48, max_num_pages=12, page_size=16)
    runner = Qwen3Runner.from_checkpoint(str(tmp_path), total_num_requests=3, max_num_batched_requests=2,
                                         max_num_batched_tokens=4, **kw)
    assert runner.shape.num_layers == cfg.num_layers and runner.shape.vocab_size == cfg.vocab_size
    lockstep_compare(runner, cfg, w, prompts, mbr=2, mbt=4, iterations=20, **kw)


def test_two_ranks_read_their_own_shards(tmp_path):
    """Both ranks of a 2-rank graph on one device, each built from the rows / columns it read from disk itself (lm_head
    cut by vocabulary): ids agree between the ranks and with a single-rank runner over the whole checkpoint wherever
    that runner's top-2 gap is clear."""
    from mirage_b200.builders.runner import Qwen3Runner
    from mirage_b200.multigpu import link_local
    cfg = Qwen3Config(num_layers=2, hidden_size=1024, num_q_heads=8, num_kv_heads=4, head_dim=128,
                      intermediate_size=2048, vocab_size=2048, max_position=128)
    w = make_weights(cfg, seed=1012)
    _write(tmp_path, cfg, w)
    kw = dict(total_num_requests=2, max_num_batched_requests=2, max_num_batched_tokens=2, max_seq_length=32,
              max_num_pages=4, page_size=16)
    whole = Qwen3Runner.from_checkpoint(str(tmp_path), num_workers=16, **kw)
    ranks = [Qwen3Runner.from_checkpoint(str(tmp_path), world_size=2, rank=r, shard_lm_head=True, device=0,
                                         num_workers=64, link_peers=False, **kw) for r in (0, 1)]
    link_local([r.mpk for r in ranks])
    for r in ranks:
        assert r.logits.shape[1] == cfg.vocab_size // 2
    g = torch.Generator().manual_seed(2012)
    prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (4, 6)]
    for r in [whole] + ranks:
        r.load_prompts(prompts)
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for it in range(12):
        whole.step(1)
        n = whole.mpk.status().active_tokens
        for r, s in zip(ranks, streams):
            r.mpk.step(1, stream=s)
        for r, s in zip(ranks, streams):
            st = r.mpk.status(stream=s)
            assert st.error == 0 and st.active_tokens == n
        ref = whole.logits[:n].float().cpu()
        top2 = ref.topk(2, dim=-1).values
        both = torch.cat([r.logits[:n].float().cpu() for r in ranks], dim=1)
        assert float((both - ref).abs().max()) <= 5e-2
        ids = [r.meta["output_tokens"].cpu().reshape(-1)[:n].tolist() for r in ranks]
        assert ids[0] == ids[1]
        want = whole.meta["output_tokens"].cpu().reshape(-1)[:n].tolist()
        for b in range(n):
            if float(top2[b, 0] - top2[b, 1]) > 0.1:
                assert ids[0][b] == want[b]
        # keep the three on one trajectory
        for r in ranks:
            r.meta["output_tokens"].copy_(whole.meta["output_tokens"])
