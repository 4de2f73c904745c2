"""Generates tests/golden/batching_traces.npz: traces of the reference's own offline scheduler step.

The reference's `prepare_next_batch` / `init_kernel` (include/mirage/persistent_kernel/persistent_kernel.cuh:142-368)
are compiled for the host by oracle/build_ref.py (oracle/_ref/libbatching_ref.so); this script drives that library
through seeded scenarios -- ragged prompts, chunked prefill under a token budget, EOS and max-length retirement, page
recycling through the ring, more requests than slots -- and stores, per scenario, the configuration, the prompts, the
scripted output tokens of every iteration and the complete scheduler state after every call.  tests/
test_batching_golden.py replays them through oracle/batching.py and requires equality, array by array.

    python tests/golden/make_batching_golden.py            (needs the reference checkout, see oracle/build_ref.py)
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

STATE_KEYS = ("step", "tokens", "input_tokens", "prompt_lengths", "qo_indptr", "paged_kv_indptr", "paged_kv_indices",
              "paged_kv_last_page_len", "request_ids", "page_queue", "scalars")

# (seed, requests, mbr, mbt, pages, page, max_seq, eos, max prompt, iterations)
SCENARIOS = [
    (1, 1, 1, 1, 8, 4, 24, -1, 5, 30),
    (2, 3, 2, 4, 16, 4, 20, 7, 9, 60),
    (3, 6, 4, 8, 24, 8, 40, 3, 30, 80),
    (4, 9, 3, 16, 12, 16, 48, 5, 40, 120),
    (5, 5, 8, 64, 40, 64, 160, 11, 150, 90),
    (6, 12, 4, 6, 28, 2, 14, 2, 10, 150),
    (7, 4, 4, 4, 64, 1, 12, -1, 3, 40),
    (8, 20, 16, 32, 128, 8, 64, 9, 50, 120),
]


class RefScheduler:
    """The reference scheduler behind ctypes: owns the meta arrays in numpy, calls the compiled reference code."""

    def __init__(self, lib, tokens, prompt_lengths, *, mbr, mbt, pages, page, eos):
        self.lib = lib
        self.R, self.S = tokens.shape
        self.cfg = (self.R, mbr, mbt, pages, page, self.S, eos)
        self.a = dict(
            step=np.full(self.R, -7, np.int32), tokens=tokens.astype(np.int64).copy(),
            input_tokens=np.zeros(mbt, np.int64), output_tokens=np.zeros(mbt, np.int64),
            prompt_lengths=prompt_lengths.astype(np.int32).copy(), qo_indptr=np.full(mbr + 1, -7, np.int32),
            paged_kv_indptr=np.full(mbr + 1, -7, np.int32), paged_kv_indices=np.zeros(pages, np.int32),
            snapshot=np.zeros(pages, np.int32), paged_kv_last_page_len=np.zeros(mbr, np.int32),
            request_ids=np.full(mbr, -7, np.int32), page_queue=np.full(pages, -7, np.int32),
            scalars=np.full(3, -7, np.int32))
        order = ("step", "tokens", "input_tokens", "output_tokens", "prompt_lengths", "qo_indptr", "paged_kv_indptr",
                 "paged_kv_indices", "snapshot", "paged_kv_last_page_len", "request_ids", "page_queue", "scalars")
        self.ptrs = (C.c_void_p * len(order))(*[self.a[k].ctypes.data for k in order])
        lib.ref_batching_init(self.ptrs, *self._args())

    def _args(self):
        R, mbr, mbt, pages, page, S, eos = self.cfg
        return C.c_int(R), C.c_int(mbr), C.c_int(mbt), C.c_int(pages), C.c_int(page), C.c_int(S), C.c_longlong(eos)

    def step(self) -> bool:
        return bool(self.lib.ref_batching_step(self.ptrs, *self._args()))


def load_reference():
    from oracle.build_ref import build_batching
    path = build_batching()
    if path is None:
        raise SystemExit("oracle/_ref/libbatching_ref.so cannot be built here: the reference checkout is absent")
    lib = C.CDLL(path)
    lib.ref_batching_step.restype = C.c_int
    return lib


def make_scenario(seed, R, S, max_prompt):
    rng = np.random.default_rng(seed)
    plen = rng.integers(1, min(max_prompt, S - 1) + 1, size=R).astype(np.int32)
    tokens = np.zeros((R, S), np.int64)
    for i in range(R):
        tokens[i, :plen[i]] = rng.integers(20, 1000, size=plen[i])
    return rng, tokens, plen


def run_reference(lib, scenario):
    seed, R, mbr, mbt, pages, page, S, eos, max_prompt, iters = scenario
    # the reference does not bound-check its page table: every slot at full length must fit
    assert pages >= mbr * ((S + page - 1) // page), "scenario would overrun paged_kv_indices in the reference itself"
    rng, tokens, plen = make_scenario(seed, R, S, max_prompt)
    ref = RefScheduler(lib, tokens, plen, mbr=mbr, mbt=mbt, pages=pages, page=page, eos=eos)
    outs, more, states = [], [], {k: [] for k in STATE_KEYS}
    for _ in range(iters):
        # what the model "generated" for the previous batch: mostly ordinary ids, now and then the EOS id
        o = rng.integers(20, 1000, size=mbt).astype(np.int64)
        if eos >= 0:
            o[rng.random(mbt) < 0.12] = eos
        ref.a["output_tokens"][:] = o
        outs.append(o)
        more.append(ref.step())
        for k in STATE_KEYS:
            states[k].append(ref.a[k].copy())
        if not more[-1]:
            break
    return tokens, plen, np.stack(outs), np.array(more), {k: np.stack(v) for k, v in states.items()}


def main():
    lib = load_reference()
    out = {"scenarios": np.array(SCENARIOS, np.int64)}
    for idx, sc in enumerate(SCENARIOS):
        tokens, plen, outs, more, states = run_reference(lib, sc)
        out[f"s{idx}_tokens0"], out[f"s{idx}_plen"], out[f"s{idx}_outs"], out[f"s{idx}_more"] = tokens, plen, outs, more
        for k, v in states.items():
            out[f"s{idx}_{k}"] = v
        print(f"scenario {idx}: {len(more)} calls, finished={not more[-1]}")
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "batching_traces.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
