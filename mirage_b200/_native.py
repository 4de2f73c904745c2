"""ctypes binding of libmpk_b200.so (see include/mpk_b200.h).

The library is the product: if it is missing or fails to load, importing this
module raises -- there is no Python or CPU fallback behind it.
"""
from __future__ import annotations

import ctypes as C
import os

# MPK_B200_LIBRARY names another build of the same library (e.g. to compare two builds on one machine)
_LIB_PATH = os.environ.get("MPK_B200_LIBRARY") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib",
                                                               "libmpk_b200.so")

MPK_OK = 0
ERRORS = {-1: "invalid argument", -2: "CUDA error", -3: "unsupported", -4: "device wait timed out",
          -5: "bad call order", -6: "task graph deadlock"}

# mpk_dtype
BF16, F16, F32, I32, I64, F8E4M3, U32, U8, U64, I16 = range(10)
# mpk_op
OP_EMBED, OP_RMSNORM, OP_RMSNORM_LINEAR, OP_LINEAR, OP_LINEAR_RESIDUAL, OP_SPLITK_LINEAR = 1, 2, 3, 4, 5, 6
OP_ATTENTION, OP_PAGED_ATTENTION, OP_SILU_MUL, OP_ALLREDUCE = 7, 8, 9, 10
OP_ARGMAX_PARTIAL, OP_ARGMAX_REDUCE, OP_ELEMENTWISE_ADD, OP_TENSOR_INIT = 11, 12, 13, 14
OP_QUANTIZE_FP8, OP_LINEAR_FP8, OP_LINEAR_FP8_RESIDUAL = 15, 16, 17
OP_MOE_TOPK_SIGMOID, OP_MOE_W13_LINEAR, OP_MOE_W2_LINEAR, OP_MOE_W13_FP8, OP_MOE_W2_FP8 = 18, 19, 20, 21, 22
OP_MOE_SILU_MUL, OP_MOE_MUL_SUM_ADD = 23, 24
OP_MLA_KV_GATHER, OP_MLA_DECODE, OP_MLA_REDUCE = 25, 26, 27
OP_SAMPLING_PARTIAL, OP_SAMPLING_REDUCE = 28, 29
OP_ARGMAX_EXCHANGE = 30
OP_MOE_TOPK_SOFTMAX = 31
IO_CUDA, IO_SYMMETRIC = 0, 1
MODE_OFFLINE, MODE_ONLINE_NOTOKEN = 0, 1


class MpkConfig(C.Structure):
    _fields_ = [
        ("mode", C.c_int32), ("test_mode", C.c_int32), ("dry_run", C.c_int32), ("device", C.c_int32),
        ("world_size", C.c_int32), ("rank", C.c_int32), ("num_workers", C.c_int32),
        ("max_seq_length", C.c_int32), ("max_num_batched_requests", C.c_int32),
        ("max_num_batched_tokens", C.c_int32), ("max_num_pages", C.c_int32), ("page_size", C.c_int32),
        ("total_num_requests", C.c_int32), ("reserved0", C.c_int32), ("eos_token_id", C.c_int64),
        ("step", C.c_void_p), ("tokens", C.c_void_p), ("input_tokens", C.c_void_p),
        ("output_tokens", C.c_void_p), ("num_new_tokens", C.c_void_p), ("prompt_lengths", C.c_void_p),
        ("qo_indptr", C.c_void_p), ("paged_kv_indptr", C.c_void_p), ("paged_kv_indices", C.c_void_p),
        ("paged_kv_last_page_len", C.c_void_p), ("paged_kv_indices_snapshot", C.c_void_p),
        ("profiler_buffer", C.c_void_p), ("profiler_entries", C.c_uint64),
    ]


class MpkStatus(C.Structure):
    _fields_ = [("error", C.c_int32), ("where", C.c_int32), ("worker", C.c_int32), ("task", C.c_int32),
                ("all_done", C.c_int32), ("active_tokens", C.c_int32), ("iteration", C.c_uint64)]


class MpkError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libmpk_b200: {ERRORS.get(code, code)}: {message}")
        self.code = code


class MpkTimeoutError(MpkError):
    """A bounded device-side wait expired; the handle must be reset before the next launch."""


SYMBOLS = {
    "mpk_create": (C.c_int, [C.POINTER(MpkConfig), C.POINTER(C.c_void_p)]),
    "mpk_destroy": (C.c_int, [C.c_void_p]),
    "mpk_last_error": (C.c_char_p, [C.c_void_p]),
    "mpk_attach_tensor": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int, C.c_int,
                                    C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "mpk_new_tensor": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_int64),
                                 C.POINTER(C.c_int64), C.c_int]),
    "mpk_shuffle_tensors": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_int), C.c_int, C.c_int]),
    "mpk_fuse_tensors": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_int), C.c_int, C.c_int]),
    "mpk_add_layer": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int),
                                C.POINTER(C.c_int64), C.c_int]),
    "mpk_compile": (C.c_int, [C.c_void_p]),
    "mpk_comm_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mpk_comm_import": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "mpk_comm_link_local": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "mpk_reset": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mpk_launch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "mpk_sync_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(MpkStatus)]),
    "mpk_tensor_ptr": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]),
    "mpk_graph_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                 C.POINTER(C.c_int)]),
    "mpk_dump_task_graph": (C.c_int64, [C.c_void_p, C.c_char_p, C.c_int64]),
    "mpk_weight_bytes_per_step": (C.c_int64, [C.c_void_p]),
    "mpk_paged_decode_attention_noalloc": (C.c_int, [C.c_void_p] * 7 + [C.c_int] * 4 + [C.c_int64] * 2 +
                                           [C.c_int, C.c_void_p, C.c_char_p, C.c_size_t]),
}


def load_library(path: str = _LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise ImportError(
            f"{path} not found: build it with `python mirage_b200/build.py` (needs nvcc, sm_100a). "
            "mirage_b200 has no fallback path without its CUDA library.")
    lib = C.CDLL(path)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)      # AttributeError if the library does not export the symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load_library()


def check(handle, rc: int) -> int:
    if rc >= 0:
        return rc
    msg = lib.mpk_last_error(handle).decode() if handle else ""
    raise (MpkTimeoutError if rc == -4 else MpkError)(rc, msg)
