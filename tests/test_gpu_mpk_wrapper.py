"""The caller-facing wrapper on a GPU: `MPK(MPKMetadata)` running a whole offline generation, and the
`online_notoken` mode (python/mirage/mpk/mpk.py:15-434): one forward per call on a batch description the caller
manages, no lm_head, the final-norm hidden state handed back."""
import numpy as np
import pytest
import torch

from oracle import mpk_ops as ops
from oracle.batching import BatchState
from oracle.qwen3_decoder import Qwen3Config, Qwen3Oracle, greedy_generate, make_weights
from gpu_util import rel_err

pytestmark = pytest.mark.gpu


def _model_config(cfg, w, pages, page, dev, with_lm_head=True):
    from mirage_b200.builders.qwen3 import Qwen3ModelConfig
    from mirage_b200.builders.runner import rope_tables
    kc = torch.zeros(cfg.num_layers, pages, page, cfg.num_kv_heads, cfg.head_dim, dtype=torch.bfloat16, device=dev)
    cos, sin = rope_tables(cfg.head_dim, cfg.max_position, cfg.rope_theta, dev)
    return Qwen3ModelConfig(cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_q_heads, cfg.num_kv_heads,
                            cfg.head_dim, cfg.num_layers, kc, torch.zeros_like(kc), (cos, sin),
                            {k: v.to(dev) for k, v in w.items()}, with_lm_head=with_lm_head)


def test_mpk_offline_generation_matches_the_oracle():
    import mirage_b200 as mi
    cfg = Qwen3Config.tiny()
    w = make_weights(cfg, seed=1011)
    prompts = [[5, 9, 200, 31], [77, 3], [8, 8, 8]]
    kw = dict(max_num_batched_requests=2, max_num_batched_tokens=3, max_num_pages=8, page_size=8)
    st, _, logits = greedy_generate(cfg, w, prompts, 20, keep_logits=True, **kw)
    meta = mi.MPKMetadata(mode="offline", total_num_requests=3, max_seq_length=20, model_name="qwen3",
                          model_config=_model_config(cfg, w, 8, 8, "cuda"), **kw)
    m = mi.MPK(meta)
    m.build()
    m.compile()
    got = m.run_ids(prompts)
    gaps = [float((l.float().topk(2, -1).values[:, 0] - l.float().topk(2, -1).values[:, 1]).min()) for l in logits]
    assert m.persistent_kernel.status().all_done == 1
    for r, p in enumerate(prompts):
        assert got[r][:len(p)] == p                       # prompts are kept
        if min(gaps) > 0.1:
            assert got[r] == st.tokens[r, :len(got[r])].tolist()
        else:                                             # at least the first generated token (compared below its tie)
            assert len(got[r]) > len(p)


def test_mpk_online_notoken_returns_the_last_hidden_state():
    """The caller (here: the CPU scheduler oracle standing in for a serving engine) writes the batch description and
    the input ids before every call; the device schedules nothing and appends to the paged cache it is pointed at."""
    import mirage_b200 as mi
    cfg = Qwen3Config.tiny()
    w = make_weights(cfg, seed=1012)
    g = torch.Generator().manual_seed(2012)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (6, 2, 9)]
    mbr, mbt, pages, page, S = 3, 4, 12, 8, 24
    meta = mi.MPKMetadata(mode="online_notoken", total_num_requests=3, max_seq_length=S, max_num_batched_requests=mbr,
                          max_num_batched_tokens=mbt, max_num_pages=pages, page_size=page, model_name="qwen3",
                          model_config=_model_config(cfg, w, pages, page, "cuda", with_lm_head=False))
    m = mi.MPK(meta)
    m.build()
    m.compile()
    tokens = np.zeros((3, S), np.int64)
    plen = np.zeros(3, np.int32)
    for i, p in enumerate(prompts):
        tokens[i, :len(p)] = p
        plen[i] = len(p)
    st = BatchState(tokens, plen, max_num_batched_requests=mbr, max_num_batched_tokens=mbt, max_num_pages=pages, page_size=page)
    orc = Qwen3Oracle(cfg, w, max_num_pages=pages, page_size=page)
    dev = "cuda"
    worst = 0.0
    for it in range(14):
        if not orc.run_iteration(st):
            break
        n = st.num_active_tokens
        m.qo_indptr_buffer.copy_(torch.from_numpy(st.qo_indptr).to(dev))
        m.paged_kv_indptr_buffer.copy_(torch.from_numpy(st.paged_kv_indptr).to(dev))
        m.paged_kv_indices_buffer.copy_(torch.from_numpy(st.paged_kv_indices).to(dev))
        m.paged_kv_last_page_len_buffer.copy_(torch.from_numpy(st.paged_kv_last_page_len).to(dev))
        m.input_tokens[:n, 0] = torch.from_numpy(st.input_tokens[:n].copy()).to(dev)
        hidden = m()
        assert m.persistent_kernel.status().error == 0
        ref = ops.rmsnorm(orc.last_hidden, w["model.norm.weight"], cfg.rms_eps)
        assert hidden.shape == (mbt, cfg.hidden_size)
        worst = max(worst, rel_err(hidden[:n].cpu(), ref))
        assert worst <= 2e-2, f"call {it}: last hidden state off by {worst}"
    assert it >= 8
