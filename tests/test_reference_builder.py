"""The reference's OWN Qwen3 graph builder, loaded unmodified from its source tree, run against this repo's
`PersistentKernel` (dry run: no CUDA call): every call it makes -- attach_input, new_tensor, shuffle_tensors,
rmsnorm_layer / linear_layer / paged_attention_layer / linear_with_residual_layer / silu_mul_layer / argmax layers with the
reference's own keyword arguments -- is accepted, and the graph compiles and passes the host simulation.

The builder file is python/mirage/mpk/models/qwen3/builder.py of the reference; it is imported under the package names
it expects (`mirage.core`, `mirage.mpk.persistent_kernel`, `mirage.mpk.model_registry` are this repo's modules,
`mirage.mpk.models.{utils,graph_builder}` the reference's own files).  The builder allocates its intermediates with
device="cuda" and asks for the device's compute capability; on this CPU-only run those two are redirected (meta
tensors, capability 10.0).  Skipped where the reference tree is not present (it does not travel to the GPU box)."""
import importlib.util
import json
import os
import sys
import types

import pytest
import torch

from oracle.qwen3_decoder import Qwen3Config
from dry_util import meta_state_dict

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("MIRAGE_REFERENCE", os.path.join(ROOT, "..", "reference"))
REF_PY = os.path.join(REF, "python", "mirage")


@pytest.mark.skipif(not os.path.isfile(os.path.join(REF_PY, "mpk", "models", "qwen3", "builder.py")),
                    reason="reference source tree not present")
def test_reference_qwen3_builder_runs_unmodified(monkeypatch):
    import mirage_b200 as mi
    from mirage_b200 import persistent_kernel as pkmod

    def package(name):
        m = types.ModuleType(name)
        m.__path__ = []
        monkeypatch.setitem(sys.modules, name, m)

    for name in ("mirage", "mirage.mpk", "mirage.mpk.models", "mirage.mpk.models.qwen3"):
        package(name)
    core = types.ModuleType("mirage.core")
    for n in ("bfloat16", "int64", "float32", "int32", "float16", "uint32", "float8_e4m3"):
        setattr(core, n, getattr(pkmod, n))
    monkeypatch.setitem(sys.modules, "mirage.core", core)
    monkeypatch.setitem(sys.modules, "mirage.mpk.persistent_kernel", pkmod)
    registry = types.ModuleType("mirage.mpk.model_registry")
    registered = {}

    def register_model_builder(*names):      # same contract; a registry of this test's own, so that this repo's stays as it is
        def deco(cls):
            registered.update({n: cls for n in names})
            return cls
        return deco

    registry.register_model_builder = register_model_builder
    monkeypatch.setitem(sys.modules, "mirage.mpk.model_registry", registry)

    def load(name, *path):
        spec = importlib.util.spec_from_file_location(name, os.path.join(REF_PY, *path))
        m = importlib.util.module_from_spec(spec)
        monkeypatch.setitem(sys.modules, name, m)
        spec.loader.exec_module(m)
        return m

    load("mirage.mpk.models.utils", "mpk", "models", "utils.py")
    gb = load("mirage.mpk.models.graph_builder", "mpk", "models", "graph_builder.py")
    ref = load("mirage.mpk.models.qwen3.builder", "mpk", "models", "qwen3", "builder.py")

    def to_meta(f):
        def g(*a, **k):
            if str(k.get("device")) == "cuda":
                k["device"] = "meta"
            return f(*a, **k)
        return g

    for n in ("zeros", "empty", "full", "ones"):
        monkeypatch.setattr(torch, n, to_meta(getattr(torch, n)))

    class Props:
        major, minor = 10, 0

    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda *a, **k: Props())

    cfg = Qwen3Config.qwen3_8b(2)
    mbr = mbt = 1
    pages, page, max_seq = 32, 64, 2048
    i32 = lambda *s: torch.empty(*s, dtype=torch.int32, device="meta")
    i64 = lambda *s: torch.empty(*s, dtype=torch.int64, device="meta")
    meta = dict(step=i32(mbr), tokens=i64(mbr, max_seq), input_tokens=i64(mbt, 1), output_tokens=i64(mbt, 1),
                num_new_tokens=i32(mbr), prompt_lengths=i32(mbr), qo_indptr_buffer=i32(mbr + 1),
                paged_kv_indptr_buffer=i32(mbr + 1), paged_kv_indices_buffer=i32(pages),
                paged_kv_last_page_len_buffer=i32(mbr))
    params = mi.PersistentKernel.get_default_init_parameters()
    params.update(mode="offline", world_size=1, mpi_rank=0, num_workers=148, max_seq_length=max_seq,
                  max_num_batched_requests=mbr, max_num_batched_tokens=mbt, max_num_pages=pages, page_size=page,
                  meta_tensors=meta, dry_run=True)
    pk = mi.PersistentKernel(**params)
    kc = torch.empty(cfg.num_layers, pages, page, cfg.num_kv_heads, cfg.head_dim, dtype=torch.bfloat16, device="meta")
    rope = torch.empty(1, 8192, cfg.head_dim, dtype=torch.bfloat16, device="meta")      # the HF rotary module's shape
    mc = gb.MirageModelConfig(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                              vocab_size=cfg.vocab_size, local_num_q_heads=cfg.num_q_heads,
                              local_num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, num_layers=cfg.num_layers,
                              k_cache=kc, v_cache=kc, position_embeddings=(rope, rope), state_dict=meta_state_dict(cfg),
                              with_lm_head=True)
    assert registered["Qwen3"] is ref.Qwen3Builder
    ref.Qwen3Builder(pk).build_from_config(mc)
    pk.compile()
    g = json.loads(pk.dump_task_graph())
    types_ = [e["type"] for e in g["events"]]
    # the same five task groups per layer as this repo's own builder (norms and silu folded into the linears)
    assert types_[:7] == ["batch", "embed", "linear", "attention", "linear", "linear", "linear"]
    assert types_.count("attention") == 2 and types_[-2:] == ["argmax_partial", "argmax_reduce"]
    # two layers + the reference's lm_head padded to 153,600 rows
    assert pk.graph_info()["weight_bytes_per_step"] == (2 * 192937984 + 153600 * 4096) * 2
