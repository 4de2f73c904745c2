"""oracle/batching.py against the reference's own scheduler step.

The fixture tests/golden/batching_traces.npz holds traces produced by the reference's `prepare_next_batch` /
`init_kernel` (include/mirage/persistent_kernel/persistent_kernel.cuh:142-368) compiled for the host
(oracle/build_ref.py, tests/golden/make_batching_golden.py).  Every array of the scheduler state must agree after
every call: integer work, bit-exact.  Where the compiled reference itself is present (oracle/_ref/
libbatching_ref.so), further random scenarios are compared live."""
import os
import sys

import numpy as np
import pytest

from oracle.batching import BatchState

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)


def _oracle_state(st):
    return dict(step=st.step, tokens=st.tokens.reshape(st.R, -1), input_tokens=st.input_tokens,
                prompt_lengths=st.prompt_lengths, qo_indptr=st.qo_indptr, paged_kv_indptr=st.paged_kv_indptr,
                paged_kv_indices=st.paged_kv_indices, paged_kv_last_page_len=st.paged_kv_last_page_len,
                request_ids=st.request_ids, page_queue=st.page_queue,
                scalars=np.array([st.page_queue_head, st.page_queue_tail, st.next_request_id], np.int32))


def _compare(ref_state, st, what):
    """Entries the reference leaves unwritten (page ids / last-page lengths / input tokens beyond the live ranges)
    are not part of the contract: compare the live ranges, everything else in full."""
    o = _oracle_state(st)
    mbr = st.mbr
    n_tok, n_pg = int(ref_state["qo_indptr"][mbr]), int(ref_state["paged_kv_indptr"][mbr])
    n_req = int((ref_state["request_ids"] != -1).sum())
    for k in ("step", "tokens", "prompt_lengths", "qo_indptr", "paged_kv_indptr", "request_ids", "scalars"):
        assert np.array_equal(ref_state[k], o[k]), f"{what}: {k}"
    assert np.array_equal(ref_state["input_tokens"][:n_tok], o["input_tokens"][:n_tok]), f"{what}: input_tokens"
    assert np.array_equal(ref_state["paged_kv_indices"][:n_pg], o["paged_kv_indices"][:n_pg]), f"{what}: page ids"
    assert np.array_equal(ref_state["paged_kv_last_page_len"][:n_req], o["paged_kv_last_page_len"][:n_req]), what
    # the page ring: only the entries between head and tail are live
    head, tail = int(ref_state["scalars"][0]), int(ref_state["scalars"][1])
    P = len(o["page_queue"])
    live = [(head + i) % P for i in range(tail - head)]
    assert np.array_equal(ref_state["page_queue"][live], o["page_queue"][live]), f"{what}: page ring"


def test_oracle_reproduces_reference_traces():
    f = np.load(os.path.join(GOLDEN, "batching_traces.npz"))
    scenarios = f["scenarios"]
    assert len(scenarios) >= 8
    total_calls = 0
    for idx, sc in enumerate(scenarios):
        seed, R, mbr, mbt, pages, page, S, eos, max_prompt, iters = (int(v) for v in sc)
        st = BatchState(f[f"s{idx}_tokens0"], f[f"s{idx}_plen"], max_num_batched_requests=mbr,
                        max_num_batched_tokens=mbt, max_num_pages=pages, page_size=page, eos_token_id=eos)
        outs, more = f[f"s{idx}_outs"], f[f"s{idx}_more"]
        for it in range(len(more)):
            st.output_tokens[:] = outs[it]
            got = st.prepare_next_batch()
            assert got == bool(more[it]), f"scenario {idx} call {it}: continue flag"
            _compare({k: f[f"s{idx}_{k}"][it] for k in ("step", "tokens", "input_tokens", "prompt_lengths", "qo_indptr",
                                                         "paged_kv_indptr", "paged_kv_indices", "paged_kv_last_page_len",
                                                         "request_ids", "page_queue", "scalars")}, st,
                     f"scenario {idx} call {it}")
            total_calls += 1
        assert not more[-1], f"scenario {idx} must run to completion"
    assert total_calls > 150


def test_oracle_against_compiled_reference_live():
    from oracle.build_ref import build_batching
    if build_batching() is None:
        pytest.skip("the compiled reference scheduler is not present here (no reference checkout); the fixture covers it")
    import make_batching_golden as mk
    lib = mk.load_reference()
    rng = np.random.default_rng(2024)
    for case in range(40):
        mbr = int(rng.integers(1, 9))
        page = int(rng.choice([1, 2, 4, 8, 16]))
        S = int(rng.integers(6, 40))
        mbt = int(rng.integers(1, 20))
        R = int(rng.integers(1, 14))
        pages = mbr * ((S + page - 1) // page) + int(rng.integers(0, 5))
        eos = int(rng.choice([-1, 4]))
        _, tokens, plen = mk.make_scenario(1000 + case, R, S, S - 1)
        ref = mk.RefScheduler(lib, tokens, plen, mbr=mbr, mbt=mbt, pages=pages, page=page, eos=eos)
        st = BatchState(tokens, plen, max_num_batched_requests=mbr, max_num_batched_tokens=mbt, max_num_pages=pages,
                        page_size=page, eos_token_id=eos)
        for it in range(1500):
            o = rng.integers(0, 9, size=mbt).astype(np.int64)       # a small alphabet: EOS comes up often
            ref.a["output_tokens"][:] = o
            st.output_tokens[:] = o
            more = ref.step()
            assert st.prepare_next_batch() == more
            _compare(ref.a, st, f"case {case} call {it}")
            if not more:
                break
        assert not more
