"""Gumbel-max sampling task on the GPU: the oracle's random stream is pinned against the real cuRAND generator, the
task's ids are compared with the oracle (bit-exact keys, ties to the highest column), and a whole decoder samples
the token the oracle picks from the same logits.

Exact comparisons take the noise from oracle/_ref/libcurand_pin.so (real cuRAND plus the reference's transform
compiled with the reference's -use_fast_math); keys, the bf16 roundings and the tie rule are the CPU oracle's.  With
the oracle's own float64 log2 the noise can differ by one bf16 step near u = 1, so that comparison accepts an id
whose oracle key is within two bf16 steps of the oracle's largest key."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import sampling_ops as so
from gpu_util import make_test_kernel, shape_of

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def mi():
    import mirage_b200
    return mirage_b200


@pytest.fixture(scope="module")
def pin():
    path = os.path.join(ROOT, "oracle", "_ref", "libcurand_pin.so")
    if not os.path.exists(path):
        from oracle import build_ref
        path = build_ref.build()
    lib = ctypes.CDLL(path)
    lib.curand_pin_fill.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_void_p,
                                    ctypes.c_void_p]
    lib.curand_pin_fill.restype = ctypes.c_int
    return lib


@pytest.mark.parametrize("seed", [0, 42, 2**31 - 1, 0x1234_5678_9ABC_DEF0])
@pytest.mark.parametrize("first", [0, 3 * 151936, 2**32 + 8])
def test_oracle_stream_equals_curand(pin, seed, first):
    groups = 4096
    u = torch.zeros(groups * 4, dtype=torch.float32, device="cuda")
    g = torch.zeros_like(u)
    assert pin.curand_pin_fill(seed, first, groups, u.data_ptr(), g.data_ptr()) == 0
    want_u = so.uniforms(seed, first, groups)
    assert np.array_equal(u.cpu().numpy().view(np.uint32), want_u.view(np.uint32)), "uniforms differ from cuRAND"
    # Gumbel values: the device takes log2 with lg2.approx (absolute error up to 2^-22 near 1), which is felt where
    # u is close to 1 and -log2(u) is tiny; elsewhere the two agree closely
    want_g, got_g = so.gumbel_from_uniform(want_u), g.cpu().numpy()
    far = want_u < 0.99
    np.testing.assert_allclose(got_g[far], want_g[far], rtol=1e-4, atol=1e-4)
    assert np.abs(got_g - want_g).max() < 0.1


def _pin_noise(pin):
    def fn(seed, local_row, V):
        groups = (V + 3) // 4
        u = torch.zeros(groups * 4, dtype=torch.float32, device="cuda")
        g = torch.zeros_like(u)
        assert pin.curand_pin_fill(seed, (local_row * V) & 0xFFFFFFFF, groups, u.data_ptr(), g.data_ptr()) == 0
        return g.cpu()[:V].to(torch.bfloat16)
    return fn


def _check(pin, ids, logits, seed, rows_per_task):
    """Exact against the oracle fed with the device-side noise; within two bf16 steps against the pure CPU oracle."""
    want = so.sampling_from_logits(logits, seed, rows_per_task, _pin_noise(pin))
    assert ids.tolist() == want.tolist()
    keys = so.sampling_keys(logits, seed, rows_per_task).float()
    for b in range(logits.shape[0]):
        top = float(keys[b].max())
        step = 2.0 ** (np.floor(np.log2(max(abs(top), 1e-30))) - 7)     # one bf16 step at the top key
        i = int(ids[b])
        assert float(keys[b, i]) >= top - 2 * step, f"row {b}: id {i} has key {float(keys[b, i])}, best {top}"


def _run(mi, logits, seed, grid_rows):
    B = logits.shape[0]
    pk = make_test_kernel(mi, B)
    out = torch.full((B, 1), -7, dtype=torch.int64, device="cuda")
    tl, to = pk.attach_input(logits.cuda(), "logits"), pk.attach_input(out, "ids")
    pk.sampling_sm100_layer(logits=tl, output=to, grid_dim=(grid_rows, 1, 1), block_dim=(256, 1, 1), seed=seed)
    pk.compile()
    pk.run_test_mode()
    first = out.clone()
    pk.run_test_mode()
    assert torch.equal(first, out)          # the reference's philox offset is constant: same draw every launch
    return out.cpu().reshape(-1)


@pytest.mark.parametrize("B,V,seed", [(8, 151936, 42), (1, 151936, 7), (5, 1000, 123456789), (3, 1003, 2**31 - 1),
                                      (16, 4096, 0)])
def test_sampling_ids_match_oracle(mi, pin, B, V, seed):
    g = torch.Generator().manual_seed(seed % 1000)
    logits = (2.0 * torch.randn(B, V, generator=g)).to(torch.bfloat16)
    ids = _run(mi, logits, seed, B)
    _check(pin, ids, logits, seed, 1)


def test_rows_of_one_reference_task_get_different_noise(mi, pin):
    """grid (1,1,1): one reference task sees all rows, row b uses subsequences b * V + ...; grid (B,1,1): every row is
    row 0 of its own task.  Flat logits make the id a function of the noise alone."""
    B, V, seed = 4, 8192, 99
    logits = torch.zeros(B, V, dtype=torch.bfloat16)
    same = _run(mi, logits, seed, B)
    assert len(set(same.tolist())) == 1
    _check(pin, same, logits, seed, 1)
    diff = _run(mi, logits, seed, 1)
    _check(pin, diff, logits, seed, B)
    assert len(set(diff.tolist())) > 1


def test_equal_keys_go_to_the_highest_column(mi):
    """At 32768 a bf16 step is 128 below and 256 above, far wider than any Gumbel value: every boosted column has the
    same key and the last one must win."""
    V, seed = 4096, 5
    logits = torch.zeros(2, V, dtype=torch.bfloat16)
    logits[0, [17, 900, 3001]] = 32768.0
    logits[1, [4095, 0]] = 32768.0
    keys = so.sampling_keys(logits, seed, 1).float()
    assert float(keys[0, 17]) == float(keys[0, 900]) == float(keys[0, 3001])      # the premise of the case
    ids = _run(mi, logits, seed, 2)
    assert ids.tolist() == [3001, 4095] == so.sampling_from_logits(logits, seed, 1).tolist()


def test_decoder_samples_what_the_oracle_picks_from_its_logits(mi, pin):
    from mirage_b200.builders.runner import Qwen3Runner
    from oracle.qwen3_decoder import Qwen3Config, make_weights
    cfg = Qwen3Config.tiny()
    w = make_weights(cfg, seed=11)
    kw = dict(max_num_batched_requests=2, max_num_batched_tokens=2, max_num_pages=8, page_size=16)
    seed = 31337
    r = Qwen3Runner(shape_of(cfg), w, total_num_requests=2, max_seq_length=40, device=0, sampling_seed=seed, **kw)
    prompts = [[5, 9, 2], [7]]
    r.load_prompts(prompts)
    rows = 0
    for it in range(12):
        r.step(1)
        st = r.mpk.status()
        assert st.error == 0
        n = st.active_tokens
        logits = r.logits[:n].cpu()
        ids = r.meta["output_tokens"][:n, 0].cpu()
        _check(pin, ids, logits, seed, 1)
        rows += n
    assert rows > 0
    # sampled tokens were fed back: past its prompt, a request's tokens are drawn ids, not all equal to the argmax run
    toks = r.tokens()
    assert int(toks[1, 1:8].abs().sum()) > 0
