"""CPU oracle for the device-side continuous batching of the MPK megakernel.

TEST INFRASTRUCTURE ONLY (see oracle/mpk_ops.py for the rules).

Integer-exact restatement of the offline-mode scheduler step,
include/mirage/persistent_kernel/persistent_kernel.cuh:206-368
(prepare_next_batch) and of its initial state, :142-169 (init_kernel).
The state is held in numpy arrays with the reference's meta-tensor names and
dtypes (python/mirage/mpk/persistent_kernel.py:2494-2506).

Parity status: pinned.  The reference's own function is plain C behind `__device__`; oracle/build_ref.py compiles
it for the host from the reference sources (oracle/_ref/libbatching_ref.so), tests/golden/make_batching_golden.py
recorded its state after every call of eight seeded scenarios (tests/golden/batching_traces.npz), and
tests/test_batching_golden.py requires this class to reproduce them array by array -- and, where the compiled
reference is present, 40 further random scenarios live.  tests/test_batching_oracle.py keeps the hand-derived
traces (page counts, indptr arrays, retirement on EOS / max length) as readable documentation of the rules.
"""
from __future__ import annotations

import numpy as np


class BatchState:
    """Meta tensors + private scheduler state of one megakernel instance."""

    def __init__(self, tokens: np.ndarray, prompt_lengths: np.ndarray, *,
                 max_num_batched_requests: int, max_num_batched_tokens: int,
                 max_num_pages: int, page_size: int, eos_token_id: int = -1):
        self.R, self.max_seq_length = tokens.shape
        self.mbr = max_num_batched_requests
        self.mbt = max_num_batched_tokens
        self.max_num_pages = max_num_pages
        self.page_size = page_size
        self.eos = eos_token_id
        self.tokens = tokens.astype(np.int64).copy()
        self.prompt_lengths = prompt_lengths.astype(np.int32).copy()
        self.total_num_requests = self.R
        # init_kernel, persistent_kernel.cuh:149-166
        self.step = np.zeros(self.R, np.int32)
        self.next_request_id = 0
        self.request_ids = np.full(self.mbr, -1, np.int32)
        self.qo_indptr = np.zeros(self.mbr + 1, np.int32)
        self.paged_kv_indptr = np.zeros(self.mbr + 1, np.int32)
        self.paged_kv_indices = np.zeros(max_num_pages, np.int32)
        self.paged_kv_last_page_len = np.zeros(self.mbr, np.int32)
        self.page_queue = np.arange(max_num_pages, dtype=np.int32)
        self.page_queue_head = 0
        self.page_queue_tail = max_num_pages
        self.input_tokens = np.zeros(self.mbt, np.int64)
        self.output_tokens = np.zeros(self.mbt, np.int64)

    @property
    def num_active_tokens(self) -> int:
        return int(self.qo_indptr[self.mbr])

    def prepare_next_batch(self) -> bool:
        """One scheduler step; returns False when nothing is left to run."""
        P, S = self.page_size, self.max_seq_length
        head, tail = self.page_queue_head, self.page_queue_tail
        # Step 1 (:213-250): commit the previous batch's outputs, retire requests.
        for i in range(self.mbr):
            rid = int(self.request_ids[i])
            if rid == -1:
                continue
            step = int(self.step[rid])
            qo = int(self.qo_indptr[i])
            n = int(self.qo_indptr[i + 1]) - qo
            plen = int(self.prompt_lengths[rid])
            for j in range(n):
                if step + j + 1 >= plen and step + j + 1 < S:
                    self.tokens[rid, step + j + 1] = self.output_tokens[qo + j]
            self.step[rid] = step + n
            done = (step + n + 1 >= S) or (
                self.tokens[rid, step + n] == self.eos and step + n >= plen)
            if done:
                self.request_ids[i] = -1
                kv = int(self.paged_kv_indptr[i])
                for j in range(int(self.paged_kv_indptr[i + 1]) - kv):
                    self.page_queue[tail % self.max_num_pages] = self.paged_kv_indices[kv + j]
                    tail += 1
        # Step 2 (:252-257): snapshot for in-place compaction.
        snapshot = self.paged_kv_indices.copy()
        # Step 3 (:259-304): running requests keep their slot order.
        num_reqs = num_tokens = num_pages = 0
        for i in range(self.mbr):
            rid = int(self.request_ids[i])
            if rid == -1:
                continue
            kv = int(self.paged_kv_indptr[i])
            n_old = int(self.paged_kv_indptr[i + 1]) - kv
            self.request_ids[num_reqs] = rid
            self.qo_indptr[num_reqs] = num_tokens
            self.paged_kv_indptr[num_reqs] = num_pages
            step = int(self.step[rid])
            n_new = int(self.prompt_lengths[rid]) - step
            if n_new > 0:
                n_new = min(n_new, self.mbt - num_tokens)
            else:
                n_new = min(1, self.mbt - num_tokens)
            for j in range(n_new):
                self.input_tokens[num_tokens + j] = self.tokens[rid, step + j]
            n_pages = (step + n_new + P - 1) // P
            lpl = (step + n_new) % P
            self.paged_kv_last_page_len[num_reqs] = P if lpl == 0 else lpl
            for j in range(n_old):
                self.paged_kv_indices[num_pages + j] = snapshot[kv + j]
            for j in range(n_old, n_pages):
                self.paged_kv_indices[num_pages + j] = self.page_queue[head % self.max_num_pages]
                head += 1
            num_pages += n_pages
            num_tokens += n_new
            num_reqs += 1
        # admit new requests (:306-339)
        while num_reqs < self.mbr and num_tokens < self.mbt:
            nxt = self.next_request_id
            if nxt >= self.total_num_requests:
                break
            self.request_ids[num_reqs] = nxt
            self.qo_indptr[num_reqs] = num_tokens
            self.paged_kv_indptr[num_reqs] = num_pages
            n_new = min(int(self.prompt_lengths[nxt]), self.mbt - num_tokens)
            for j in range(n_new):
                self.input_tokens[num_tokens + j] = self.tokens[nxt, j]
            n_pages = (n_new + P - 1) // P
            lpl = n_new % P
            self.paged_kv_last_page_len[num_reqs] = P if lpl == 0 else lpl
            for j in range(n_pages):
                self.paged_kv_indices[num_pages + j] = self.page_queue[head % self.max_num_pages]
                head += 1
            num_tokens += n_new
            num_pages += n_pages
            num_reqs += 1
            self.next_request_id = nxt + 1
        # Step 4 (:341-348)
        self.request_ids[num_reqs:] = -1
        self.qo_indptr[num_reqs:] = num_tokens
        self.paged_kv_indptr[num_reqs:] = num_pages
        # Step 5
        self.page_queue_head, self.page_queue_tail = head, tail
        return num_tokens != 0

    # convenience views -----------------------------------------------------
    def request_view(self, slot: int):
        """(request_id, token range, page ids, seq_len incl. new tokens) of a slot."""
        rid = int(self.request_ids[slot])
        q0, q1 = int(self.qo_indptr[slot]), int(self.qo_indptr[slot + 1])
        k0, k1 = int(self.paged_kv_indptr[slot]), int(self.paged_kv_indptr[slot + 1])
        pages = [int(p) for p in self.paged_kv_indices[k0:k1]]
        seq_len = (len(pages) - 1) * self.page_size + int(self.paged_kv_last_page_len[slot])
        return rid, (q0, q1), pages, seq_len
