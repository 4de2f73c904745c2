"""mirage_b200: a B200 (sm_100a) decode megakernel behind Mirage's `PersistentKernel` API.

    import mirage_b200 as mi
    mpk = mi.PersistentKernel(**params)
    x = mpk.attach_input(tensor, name="x"); ...; mpk.linear_layer(...); mpk.compile(); mpk()

Importing the package loads mirage_b200/lib/libmpk_b200.so (build: `python mirage_b200/build.py`);
there is no fallback when it is absent.
"""
from .persistent_kernel import (  # noqa: F401
    DTensor, MpkError, MpkTimeoutError, PersistentKernel, bfloat16, convert_torch_type_to_dtype, dtype, float16,
    float32, float8_e4m3, get_configurations_from_gpu, int16, int32, int64, uint8, uint32,
    valid_persistent_kernel_modes,
)

from .noalloc import paged_decode_attention_noalloc  # noqa: F401,E402
from .mpk import MPK, MPKMetadata, get_builder, register_model_builder  # noqa: F401,E402
from .builders import qwen3 as _qwen3_builder  # noqa: F401,E402  (files the Qwen3 graph builder)

__all__ = ["paged_decode_attention_noalloc", "MPK", "MPKMetadata", "get_builder", "register_model_builder", "PersistentKernel", "DTensor", "MpkError", "MpkTimeoutError", "get_configurations_from_gpu",
           "bfloat16", "float16", "float32", "int32", "int64", "uint32", "uint8", "int16", "float8_e4m3"]
