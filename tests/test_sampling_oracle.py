"""CPU checks of the Gumbel-max sampling oracle and of the sampling layer's place in the task graph (no GPU)."""
import json

import numpy as np
import torch

from oracle import sampling_ops as so


def test_uniforms_are_in_range_and_look_uniform():
    u = so.uniforms(seed=42, first_subsequence=0, groups=50000)
    assert u.dtype == np.float32 and u.min() > 0.0 and u.max() <= 1.0
    assert abs(float(u.mean()) - 0.5) < 5e-3 and abs(float(u.var()) - 1.0 / 12.0) < 2e-3
    hist = np.histogram(u, bins=16, range=(0.0, 1.0))[0]
    expect = u.size / 16
    assert float(((hist - expect) ** 2 / expect).sum()) < 50.0       # chi-square, 15 degrees of freedom
    # counter-based: a block depends on (seed, subsequence) only
    again = so.uniforms(seed=42, first_subsequence=4 * 100, groups=10)
    assert np.array_equal(again, u[400:440])
    assert not np.array_equal(so.uniforms(seed=43, first_subsequence=0, groups=10), u[:40])


def test_gumbel_max_draws_follow_softmax():
    """Over many seeds the sampled id is distributed as softmax(logits): the property the task exists for."""
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5, 1.5, -2.0, 0.25]], dtype=torch.bfloat16)
    n = 4000
    counts = np.zeros(8)
    for seed in range(n):
        counts[int(so.sampling_from_logits(logits, seed)[0])] += 1
    p = torch.softmax(logits.float()[0], dim=0).numpy()
    chi2 = float(((counts - n * p) ** 2 / (n * p)).sum())
    assert chi2 < 40.0, (chi2, counts, n * p)      # 7 degrees of freedom; bf16 rounding of noise and key adds a little


def test_equal_keys_go_to_the_highest_column_and_rows_per_task():
    logits = torch.zeros(3, 64, dtype=torch.bfloat16)
    logits[:, [5, 40]] = 32768.0
    assert so.sampling_from_logits(logits, 1).tolist() == [40, 40, 40]
    flat = torch.zeros(4, 4096, dtype=torch.bfloat16)
    same = so.sampling_from_logits(flat, 9, rows_per_task=1)
    assert len(set(same.tolist())) == 1
    diff = so.sampling_from_logits(flat, 9, rows_per_task=4)
    assert diff[0] == same[0] and len(set(diff.tolist())) > 1


def test_sampling_layer_schedules_partials_and_a_merge():
    import mirage_b200 as mi
    mbt, V = 4, 151936
    pk = mi.PersistentKernel(mode="offline", test_mode=True, num_workers=148, max_num_batched_tokens=mbt,
                             max_num_batched_requests=mbt, dry_run=True)
    logits = pk.attach_input(torch.empty(mbt, V, dtype=torch.bfloat16, device="meta"), "logits")
    out = pk.attach_input(torch.empty(mbt, 1, dtype=torch.int64, device="meta"), "ids")
    pk.sampling_sm100_layer(logits=logits, output=out, grid_dim=(mbt, 1, 1), block_dim=(256, 1, 1), seed=2**31 - 1)
    pk.compile()
    g = json.loads(pk.dump_task_graph())
    ev = [e for e in g["events"] if e["type"].startswith("sampling")]
    assert [e["type"] for e in ev] == ["sampling_partial", "sampling_reduce"]
    assert ev[0]["tasks"] == 148 and ev[1]["tasks"] == 1
    assert ev[1]["deps"] and ev[1]["deps"][0][1] == 148          # the merge waits for every column range


def test_qwen3_builder_with_sampling_seed_dry_run():
    """sampling_seed on the model config swaps the argmax pair for the sampling pair (demo/qwen3/demo_sampling.py)."""
    import mirage_b200 as mi
    from mirage_b200.builders.qwen3 import Qwen3ModelConfig
    from oracle.qwen3_decoder import Qwen3Config
    from dry_util import meta_state_dict
    cfg = Qwen3Config.qwen3_8b(1)
    pages, page = 32, 64
    kc = torch.empty(cfg.num_layers, pages, page, cfg.num_kv_heads, cfg.head_dim, dtype=torch.bfloat16, device="meta")
    rope = torch.empty(4096, cfg.head_dim, dtype=torch.bfloat16, device="meta")
    mc = Qwen3ModelConfig(cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_q_heads, cfg.num_kv_heads,
                          cfg.head_dim, cfg.num_layers, kc, kc, (rope, rope), meta_state_dict(cfg), sampling_seed=5)
    meta = mi.MPKMetadata(mode="offline", total_num_requests=1, max_seq_length=2048, max_num_batched_requests=1,
                          max_num_batched_tokens=1, max_num_pages=pages, page_size=page, model_name="Qwen/Qwen3-8B",
                          model_config=mc, dry_run=True)
    m = mi.MPK(meta)
    m.build()
    m.compile()
    g = json.loads(m.persistent_kernel.dump_task_graph())
    assert [e["type"] for e in g["events"] if e["type"].startswith("sampling")] == ["sampling_partial", "sampling_reduce"]
    assert not any(e["type"].startswith("argmax") for e in g["events"])
