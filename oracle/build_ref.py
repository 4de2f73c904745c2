"""Builds the checker's native pieces into oracle/_ref/ (test infrastructure, never shipped or timed as product).

    libcurand_pin.so    from oracle/curand_pin.cu: the real cuRAND generator the sampling oracle is pinned against.
    libbatching_ref.so  the reference's own scheduler step, compiled for the HOST from the reference sources where
                        they lie: `prepare_next_batch` and the body of `init_kernel`
                        (include/mirage/persistent_kernel/persistent_kernel.cuh:142-368) with the real
                        `RuntimeConfig` of runtime_header.h.  The two functions are plain C behind `__device__`;
                        this recipe cuts their text out of the header at build time, puts a small shim in front
                        (empty `__device__` / `__global__`, the MPK_* compile-time limits as variables, a one-thread
                        `threadIdx`) and pipes the translation unit to g++ on stdin, so no reference source is
                        written anywhere: only the .so lands in oracle/_ref/ (git-ignored).  It needs the reference
                        checkout (environment variable MIRAGE_REFERENCE, default: the directory `reference` beside the
                        repository) and is skipped where that is absent;
                        tests/golden/batching_traces.npz holds traces generated with it
                        (tests/golden/make_batching_golden.py).

Usage: python oracle/build_ref.py
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
REFERENCE = os.environ.get("MIRAGE_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
BATCHING_HEADER = os.path.join("include", "mirage", "persistent_kernel", "persistent_kernel.cuh")

_SHIM_HEAD = r"""
#include <algorithm>
#include <cassert>
#include <cstdint>
#define MIRAGE_BACKEND_USE_CUDA
#define MODE_OFFLINE
#define MPK_TARGET_CC 100
#include "runtime_header.h"
using namespace mirage::runtime;
using std::min;
#define __device__
#define __global__
#define __forceinline__ inline
// the reference fixes these limits at compile time of the generated megakernel; here they are run-time values
static int g_mbr, g_mbt, g_pages, g_page, g_seq;
#define MPK_MAX_NUM_BATCHED_REQUESTS g_mbr
#define MPK_MAX_NUM_BATCHED_TOKENS g_mbt
#define MPK_MAX_NUM_PAGES g_pages
#define MPK_PAGE_SIZE g_page
#define MPK_MAX_SEQ_LENGTH g_seq
static const struct { int x, y, z; } threadIdx = {0, 0, 0}, gridDim = {1, 1, 1};
"""

_SHIM_TAIL = r"""
extern "C" {
// meta: step, tokens, input_tokens, output_tokens, prompt_length, qo_indptr, paged_kv_indptr, paged_kv_indices,
//       paged_kv_indices_snapshot, paged_kv_last_page_len, request_ids, page_queue, {head, tail, next_request_id}
static RuntimeConfig make_config(void **m, int total, int seq, long long eos) {
  RuntimeConfig c{};
  c.step = (int *)m[0]; c.tokens = (long long *)m[1]; c.input_tokens = (long long *)m[2];
  c.output_tokens = (long long *)m[3]; c.prompt_length = (int *)m[4]; c.qo_indptr_buffer = (int *)m[5];
  c.paged_kv_indptr_buffer = (int *)m[6]; c.paged_kv_indices_buffer = (int *)m[7];
  c.paged_kv_indices_snapshot = (int *)m[8]; c.paged_kv_last_page_len_buffer = (int *)m[9];
  c.request_ids = (int *)m[10]; c.page_queue = (int *)m[11];
  int *sc = (int *)m[12];
  c.page_queue_head = sc; c.page_queue_tail = sc + 1; c.next_request_id = sc + 2;
  c.total_num_requests = total; c.max_seq_length = seq; c.eos_token_id = eos;
  return c;
}
static void set_limits(int mbr, int mbt, int pages, int page, int seq) {
  g_mbr = mbr; g_mbt = mbt; g_pages = pages; g_page = page; g_seq = seq;
}
void ref_batching_init(void **m, int total, int mbr, int mbt, int pages, int page, int seq, long long eos) {
  set_limits(mbr, mbt, pages, page, seq);
  init_kernel(make_config(m, total, seq, eos));
}
int ref_batching_step(void **m, int total, int mbr, int mbt, int pages, int page, int seq, long long eos) {
  set_limits(mbr, mbt, pages, page, seq);
  RuntimeConfig c = make_config(m, total, seq, eos);
  return prepare_next_batch(c) ? 1 : 0;
}
}
"""


def _cut_function(text: str, signature: str, first_word: str) -> str:
    """The definition that contains `signature`, from `first_word` of its declaration to the matching brace."""
    at = text.index(signature)
    start = text.rfind(first_word, 0, at + len(first_word))
    depth, i = 0, text.index("{", at)
    while True:
        depth += {"{": 1, "}": -1}.get(text[i], 0)
        i += 1
        if depth == 0:
            return text[start:i]


def build_curand(force: bool = False) -> str:
    src = os.path.join(HERE, "curand_pin.cu")
    out = os.path.join(OUT_DIR, "libcurand_pin.so")
    if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-use_fast_math", "-shared",
                    "-Xcompiler", "-fPIC", "-o", out, src, "-lcudart"], check=True)
    return out


def build_batching(force: bool = False):
    """Returns the path of libbatching_ref.so, or None where the reference checkout is absent and no earlier build
    exists (the GPU box: it uses the prebuilt file that travelled with the tree, or the committed traces)."""
    out = os.path.join(OUT_DIR, "libbatching_ref.so")
    header = os.path.join(REFERENCE, BATCHING_HEADER)
    if not os.path.exists(header):
        return out if os.path.exists(out) else None
    if not force and os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(header),
                                                                          os.path.getmtime(__file__)):
        return out
    os.makedirs(OUT_DIR, exist_ok=True)
    text = open(header).read()
    unit = (_SHIM_HEAD + _cut_function(text, "__global__ void init_kernel(RuntimeConfig config)", "__global__") + "\n" +
            _cut_function(text, "prepare_next_batch(RuntimeConfig const &config)", "__device__") + "\n" + _SHIM_TAIL)
    inc = os.path.join(REFERENCE, "include")
    subprocess.run(["g++", "-x", "c++", "-std=c++17", "-O1", "-shared", "-fPIC", "-w", "-I", inc,
                    "-I", os.path.join(inc, "mirage", "persistent_kernel"), "-I", "/usr/local/cuda/include",
                    "-", "-o", out], input=unit.encode(), check=True)
    return out


def build(force: bool = False) -> str:
    build_batching(force)
    return build_curand(force)


if __name__ == "__main__":
    print(build_curand(force=True))
    print(build_batching(force=True))
