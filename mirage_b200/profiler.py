"""Trace export for the megakernel's in-kernel profiler.

Plays the part of python/mirage/mpk/profiler_persistent.py:110-171 (`export_to_perfetto_trace`): the reference
writes (tag, timestamp) pairs per event and converts them with `tg4perfetto`; this kernel writes one 8 x u64 record
per task -- [wait begin, dependencies satisfied, body end, worker << 40 | event << 8 | task type, then up to four
phase stamps] in globaltimer nanoseconds -- and the export is a Chrome / Perfetto JSON trace ("traceEvents") with one
track per worker CTA and two slices per task: the dependency wait and the body.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional

import torch

TASK_NAMES = ["nop", "batch", "embed", "rmsnorm", "linear", "attention", "silu_mul", "argmax_partial", "argmax_reduce",
              "allreduce", "elementwise_add", "tensor_init", "quantize_fp8", "moe_routing", "moe_gemm", "moe_silu_mul",
              "moe_mul_sum_add", "mla_append", "mla_decode", "mla_reduce", "sampling_partial", "sampling_reduce", "argmax_exchange", "ar_push"]


def decode_records(profiler_buffer: torch.Tensor, num_tasks: int) -> List[Dict[str, int]]:
    """-> one dict per task that ran: worker, event, type, begin_ns, ready_ns, end_ns (relative to the earliest)."""
    rec = profiler_buffer.detach().cpu().view(torch.int64)[: num_tasks * 8].reshape(num_tasks, 8)
    rows = [r.tolist() for r in rec if int(r[0]) > 0 and int(r[2]) > 0]
    if not rows:
        return []
    t0 = min(r[0] for r in rows)
    out = []
    for r in rows:
        tag = r[3] & 0xFFFFFFFFFFFFFFFF
        out.append({"worker": int(tag >> 40), "event": int((tag >> 8) & 0xFFFFFFFF), "type": int(tag & 0xFF),
                    "begin_ns": r[0] - t0, "ready_ns": max(r[1], r[0]) - t0, "end_ns": r[2] - t0})
    return out


def export_to_perfetto_trace(profiler_buffer: torch.Tensor, file_name: str, num_tasks: Optional[int] = None,
                             task_graph_json: Optional[str] = None) -> int:
    """Writes `file_name` (open with ui.perfetto.dev or chrome://tracing); returns the number of tasks exported."""
    n = num_tasks if num_tasks is not None else profiler_buffer.numel() // 8
    layer_of_event = {}
    if task_graph_json:
        for ev in json.loads(task_graph_json).get("events", []):
            layer_of_event[ev["event"]] = ev.get("out", "")
    events = []
    for r in decode_records(profiler_buffer, n):
        name = TASK_NAMES[r["type"]] if r["type"] < len(TASK_NAMES) else f"task_{r['type']}"
        label = f"{name}#{r['event']}" + (f" -> {layer_of_event[r['event']]}" if layer_of_event.get(r["event"]) else "")
        common = {"pid": 0, "tid": r["worker"], "cat": name}
        if r["ready_ns"] > r["begin_ns"]:
            events.append(dict(common, name="wait " + label, ph="X", ts=r["begin_ns"] / 1e3,
                               dur=(r["ready_ns"] - r["begin_ns"]) / 1e3))
        events.append(dict(common, name=label, ph="X", ts=r["ready_ns"] / 1e3,
                           dur=max(r["end_ns"] - r["ready_ns"], 0) / 1e3))
    with open(file_name, "w") as f:
        json.dump({"displayTimeUnit": "ns", "traceEvents": events}, f)
    return len({(e["tid"], e["ts"]) for e in events if not e["name"].startswith("wait ")})


# Event-type ids of the reference's exporter (python/mirage/mpk/profiler_persistent.py:11-103, `event_name_list`) for
# this kernel's task types: the sm100 task of the same job where the reference has one.
REFERENCE_EVENT_IDS = {
    "batch": 10,              # TASK_BEGIN_TASK_GRAPH
    "embed": 101,             # TASK_EMBEDDING
    "rmsnorm": 119,           # TASK_RMS_NORM
    "linear": 253,            # TASK_LINEAR_SM100
    "attention": 257,         # TASK_ATTN_SM100
    "silu_mul": 118,          # TASK_SILU_MUL
    "argmax_partial": 259,    # TASK_ARGMAX_PARTIAL_SM100
    "argmax_reduce": 258,     # TASK_ARGMAX_REDUCE_SM100
    "allreduce": 106,         # TASK_ALLREDUCE
    "elementwise_add": 281,   # TASK_ELEMENTWISE_ADD_SM100
    "tensor_init": 262,       # TASK_TENSOR_INIT
    "quantize_fp8": 275,      # TASK_QUANTIZE_FP8_SM100
    "moe_routing": 280,       # TASK_MOE_TOPK_SIGMOID_SM100
    "moe_gemm": 248,          # TASK_MOE_W13_FP8_SM100
    "moe_silu_mul": 118,      # TASK_SILU_MUL
    "moe_mul_sum_add": 261,   # TASK_MOE_MUL_SUM_ADD_SM100
    "mla_append": 278,        # TASK_MLA_KV_GATHER_SM100
    "mla_decode": 266,        # TASK_MLA_DECODE_SM100
    "mla_reduce": 267,        # TASK_MLA_REDUCE_SM100
    "sampling_partial": 265,  # TASK_SAMPLING_SM100
    "sampling_reduce": 265,
    "argmax_exchange": 107,   # TASK_REDUCE
    "ar_push": 302,           # TASK_NVSHMEM_TILE_ALLREDUCE
}
REFERENCE_WAIT_EVENT_ID = 203  # TASK_GET_NEXT_TASK: the span a worker spends waiting for a task's dependencies


def to_reference_profiler_buffer(profiler_buffer: torch.Tensor, num_tasks: int, num_workers: int) -> torch.Tensor:
    """Re-encodes this kernel's per-task records as the reference's profiler buffer, so that the reference's own
    `export_to_perfetto_trace` (python/mirage/mpk/profiler_persistent.py:123-171) reads them unchanged.

    Layout written (include/mirage/persistent_kernel/profiler.h:34-47, 92-135): int64 entries; entry 0 holds
    {nblocks, ngroups = 1} as two uint32; every other entry is {tag, globaltimer_lo} with tag = event_no << 19 |
    block << 11 | event id << 2 | {0 begin, 1 end}; the k-th entry a block wrote sits at 1 + block + k * nblocks.
    Each task becomes four entries on its worker's block: a TASK_GET_NEXT_TASK begin/end pair over the dependency
    wait and a begin/end pair of the mapped task id over the body; event_no counts the events of one id on one block
    (13 bits, wrapping as the reference's does).  Entries a block did not write stay 0, which the exporter skips.
    The tag has 8 bits for the block, so at most 256 worker CTAs can be represented."""
    if num_workers > 256:
        raise ValueError("the reference's tag holds 8 bits of block index")
    rec = profiler_buffer.detach().cpu().view(torch.int64)[: num_tasks * 8].reshape(num_tasks, 8)
    per_block: Dict[int, List] = {}
    for r in rec.tolist():
        if r[0] <= 0 or r[2] <= 0:
            continue
        tag = r[3] & 0xFFFFFFFFFFFFFFFF
        worker, ttype = int(tag >> 40), int(tag & 0xFF)
        if worker >= num_workers:
            raise ValueError(f"record of worker {worker} but num_workers = {num_workers}")
        name = TASK_NAMES[ttype] if ttype < len(TASK_NAMES) else "nop"
        per_block.setdefault(worker, []).append((r[0], max(r[1], r[0]), r[2], REFERENCE_EVENT_IDS.get(name, 121)))
    depth = max((len(v) for v in per_block.values()), default=0) * 4
    out = torch.zeros(1 + depth * num_workers, dtype=torch.int64)
    out[0] = num_workers | (1 << 32)
    for block, tasks in per_block.items():
        tasks.sort()
        counts: Dict[int, int] = {}
        k = 0
        for begin, ready, end, eid in tasks:
            for event_id, t0, t1 in ((REFERENCE_WAIT_EVENT_ID, begin, ready), (eid, ready, end)):
                no = counts.get(event_id, 0)
                counts[event_id] = no + 1
                base = ((no & 0x1FFF) << 19) | (block << 11) | (event_id << 2)
                for kind, t in ((0, t0), (1, t1)):
                    word = (base | kind) | ((t & 0xFFFFFFFF) << 32)
                    out[1 + block + k * num_workers] = word - (1 << 64) if word >= (1 << 63) else word
                    k += 1
    return out
