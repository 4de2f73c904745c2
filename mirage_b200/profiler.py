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
