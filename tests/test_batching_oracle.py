"""Hand-derived traces for the offline batching oracle
(include/mirage/persistent_kernel/persistent_kernel.cuh:206-368)."""
import numpy as np

from oracle.batching import BatchState


def _state(prompts, S=16, **kw):
    tok = np.zeros((len(prompts), S), np.int64)
    pl = np.zeros(len(prompts), np.int32)
    for i, p in enumerate(prompts):
        tok[i, :len(p)] = p
        pl[i] = len(p)
    return BatchState(tok, pl, **kw)


def test_single_request_one_token_per_iteration():
    st = _state([[5, 6, 7]], max_num_batched_requests=1, max_num_batched_tokens=1,
                max_num_pages=4, page_size=2)
    # iteration 1: admits request 0 with min(prompt 3, mbt 1) = 1 token, one page
    assert st.prepare_next_batch()
    assert st.input_tokens[0] == 5 and st.qo_indptr.tolist() == [0, 1]
    assert st.paged_kv_indptr.tolist() == [0, 1] and st.paged_kv_last_page_len[0] == 1
    assert st.paged_kv_indices[0] == 0 and st.page_queue_head == 1
    st.output_tokens[0] = 99           # ignored: step+1 = 1 < prompt_len
    assert st.prepare_next_batch()
    assert st.step[0] == 1 and st.input_tokens[0] == 6 and st.tokens[0, 1] == 6
    assert st.paged_kv_last_page_len[0] == 2 and st.paged_kv_indptr[1] == 1
    st.output_tokens[0] = 98
    assert st.prepare_next_batch()     # third prompt token, second page
    assert st.step[0] == 2 and st.input_tokens[0] == 7
    assert st.paged_kv_indptr[1] == 2 and st.paged_kv_indices[:2].tolist() == [0, 1]
    assert st.paged_kv_last_page_len[0] == 1
    st.output_tokens[0] = 42           # first generated token: step+1 = 3 >= prompt_len
    assert st.prepare_next_batch()
    assert st.tokens[0, 3] == 42 and st.input_tokens[0] == 42 and st.step[0] == 3


def test_retire_on_eos_frees_pages_and_admits_next():
    st = _state([[1, 2], [3]], S=8, max_num_batched_requests=1, max_num_batched_tokens=4,
                max_num_pages=2, page_size=4, eos_token_id=9)
    assert st.prepare_next_batch()
    assert st.qo_indptr.tolist() == [0, 2] and st.request_ids[0] == 0
    st.output_tokens[:2] = [7, 9]      # token after the prompt is EOS
    assert st.prepare_next_batch()
    # request 0: step=2, tokens[0,2]=9 == eos and step >= prompt_len -> retired, page 0 freed to tail
    assert st.tokens[0, 2] == 9 and st.page_queue_tail == 3
    assert st.request_ids[0] == 1 and st.input_tokens[0] == 3
    assert st.paged_kv_indices[0] == 1   # next page in the ring
    st.output_tokens[0] = 9
    assert not st.prepare_next_batch()   # request 1 retires, nothing left
    assert st.num_active_tokens == 0


def test_retire_on_max_seq_length():
    st = _state([[1]], S=3, max_num_batched_requests=1, max_num_batched_tokens=1,
                max_num_pages=2, page_size=4)
    assert st.prepare_next_batch()
    st.output_tokens[0] = 5
    assert st.prepare_next_batch()       # step 1, 1+0+1 < 3 still running
    st.output_tokens[0] = 6
    assert not st.prepare_next_batch()   # step 2: step + 1 >= max_seq_length
    assert st.tokens[0].tolist() == [1, 5, 6]


def test_two_requests_share_token_budget():
    st = _state([[1, 2, 3], [4, 5, 6]], max_num_batched_requests=2, max_num_batched_tokens=4,
                max_num_pages=8, page_size=2)
    assert st.prepare_next_batch()
    # request 0 takes 3 tokens, request 1 the remaining 1
    assert st.qo_indptr.tolist() == [0, 3, 4]
    assert st.input_tokens.tolist() == [1, 2, 3, 4]
    assert st.paged_kv_indptr.tolist() == [0, 2, 3]
    assert st.paged_kv_last_page_len.tolist() == [1, 1]
    st.output_tokens[:] = [0, 0, 11, 0]
    assert st.prepare_next_batch()
    # request 0 decodes 1 token (11), request 1 prefills its remaining 2
    assert st.qo_indptr.tolist() == [0, 1, 3]
    assert st.input_tokens[:3].tolist() == [11, 5, 6]
    assert st.paged_kv_indptr.tolist() == [0, 2, 4]
    # compaction keeps old pages first, new pages come from the ring head
    assert st.paged_kv_indices[:4].tolist() == [0, 1, 2, 3]
