"""Shared helpers for the GPU parity tests."""
import numpy as np
import torch

from oracle.batching import BatchState
from oracle.qwen3_decoder import Qwen3Config, Qwen3Oracle


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| / max |ref|  (the 'max relative error' the parity bar is stated in)."""
    return float((got.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-12))


def make_test_kernel(mi, mbt, **kw):
    params = mi.PersistentKernel.get_default_init_parameters()
    params.update(test_mode=True, num_workers=0, max_num_batched_tokens=mbt, max_num_batched_requests=mbt)
    params.update(kw)
    return mi.PersistentKernel(**params)


def shape_of(cfg: Qwen3Config):
    from mirage_b200.builders.runner import DecoderShape
    return DecoderShape(cfg.num_layers, cfg.hidden_size, cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim,
                        cfg.intermediate_size, cfg.vocab_size, cfg.rope_theta, cfg.max_position)


def lockstep_compare(runner, cfg, weights, prompts, *, max_seq_length, mbr, mbt, max_num_pages, page_size,
                     eos=-1, iterations=16, logit_tol=5e-2, world_size=1, oracle_factory=None, id_gap=0.1):
    """Run the megakernel and the CPU oracle iteration by iteration on the same batches.

    After every iteration: logits of the active tokens within `logit_tol` (abs), greedy ids equal wherever
    the oracle's top-2 gap exceeds `id_gap` (0.1), batching meta tensors bit-exact.  The oracle is then fed the
    megakernel's tokens so both stay on the same trajectory.
    """
    tokens = np.zeros((len(prompts), max_seq_length), np.int64)
    plen = np.zeros(len(prompts), np.int32)
    for i, p in enumerate(prompts):
        tokens[i, :len(p)] = p
        plen[i] = len(p)
    st = BatchState(tokens, plen, max_num_batched_requests=mbr, max_num_batched_tokens=mbt,
                    max_num_pages=max_num_pages, page_size=page_size, eos_token_id=eos)
    if oracle_factory is not None:
        orc = oracle_factory(max_num_pages=max_num_pages, page_size=page_size)
    else:
        orc = Qwen3Oracle(cfg, weights, max_num_pages=max_num_pages, page_size=page_size, world_size=world_size)
    runner.load_prompts(prompts)
    m = runner.meta
    worst = 0.0
    mismatched_ids = 0
    for it in range(iterations):
        more = orc.run_iteration(st)
        runner.step(1)
        status = runner.mpk.status()
        assert status.error == 0
        assert bool(status.all_done) == (not more), f"iteration {it}: all_done {status.all_done} vs oracle {more}"
        n = st.num_active_tokens
        assert status.active_tokens == n
        # batching meta tensors: bit-exact
        assert m["qo_indptr_buffer"].cpu().numpy()[:mbr + 1].tolist() == st.qo_indptr.tolist(), f"qo_indptr it {it}"
        assert m["paged_kv_indptr_buffer"].cpu().numpy()[:mbr + 1].tolist() == st.paged_kv_indptr.tolist()
        npg = int(st.paged_kv_indptr[mbr])
        assert m["paged_kv_indices_buffer"].cpu().numpy()[:npg].tolist() == st.paged_kv_indices[:npg].tolist()
        nreq = int((st.request_ids != -1).sum())
        assert m["paged_kv_last_page_len_buffer"].cpu().numpy()[:nreq].tolist() == \
            st.paged_kv_last_page_len[:nreq].tolist()
        assert m["step"].cpu().numpy().tolist() == st.step.tolist(), f"step it {it}"
        assert m["input_tokens"].cpu().numpy().reshape(-1)[:n].tolist() == st.input_tokens[:n].tolist()
        if not more:
            break
        got = runner.logits[:n].float().cpu()
        ref = orc.last_logits.float().cpu()
        # a tensor-parallel rank with a sharded lm_head holds the logits of its own vocabulary columns only
        first = getattr(runner, "vocab_first", 0)
        worst = max(worst, float((got - ref[:, first:first + got.shape[1]]).abs().max()))
        assert worst <= logit_tol, f"iteration {it}: logits differ by {worst}"
        out = m["output_tokens"].cpu().numpy().reshape(-1)[:n]
        top2 = ref.topk(2, dim=-1).values
        gap = (top2[:, 0] - top2[:, 1]).numpy()
        ref_ids = st.output_tokens[:n]
        for b in range(n):
            if gap[b] > id_gap:
                assert out[b] == ref_ids[b], f"iteration {it} token {b}: {out[b]} vs {ref_ids[b]} (gap {gap[b]})"
            elif out[b] != ref_ids[b]:
                mismatched_ids += 1
        assert (out < cfg.vocab_size).all()
        st.output_tokens[:n] = out          # keep both on the megakernel's trajectory
    # committed tokens agree as well
    assert m["tokens"].cpu().numpy().tolist() == st.tokens.tolist()
    return worst, mismatched_ids


def input_checksums(t, keys):
    """Order-independent 64-bit sums of the raw bytes of the named tensors (a drift check for seeded inputs that are too
    large to commit)."""
    out = {}
    for k in keys:
        raw = t[k].contiguous().view(torch.uint8).view(-1)
        out[k] = int(sum(int(c.to(torch.int64).sum().item()) for c in raw.split(1 << 28)))
    return out
