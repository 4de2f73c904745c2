"""Builds the reference's stand-alone sm100 kernel wrappers ("the kernels to beat") from the reference's own sources,
unmodified and where they lie, into the git-ignored `baseline/_ref/`.

    python baseline/build_ref_kernels.py <reference checkout> [name ...]

Built (each a torch extension the reference's own tests import under the same name):
  runtime_kernel_fp8_moe   tests/runtime_python/blackwell/sm100_fp8_moe/runtime_kernel_wrapper.cu -- the FP8 grouped
                           expert GEMM of the DeepSeek-V3 shapes (256 experts, top-8, W13 [256, 4096, 7168], 16
                           tokens) on a 2-D grid, with the `fp8_moe_gemm_bench_*` entry points the reference's own
                           bench_fp8_moe_gemm.py times.
The include paths are the ones the wrapper's setup.py names (tests/runtime_python/blackwell/sm100_fp8_moe/setup.py:24-41)
with the reference's empty `deps/cutlass` submodule replaced by the CUTLASS header tree inside the flashinfer wheel.
  ref_mla_tp8              baseline/ref_mla_tp8_ext.cu (this repo's host wrapper) around the reference's device functions
                           `mla_mtp_tp8_main` / `mla_mtp_tp8_reduce` of
                           include/mirage/persistent_kernel/tasks/blackwell/mla_mtp_decode_tp8_sm100.cuh: absorbed MLA
                           decode for 16 local heads on a dense [requests, kv_len, 576] cache.
  runtime_kernel_blackwell_quantize_fp8
                           tests/runtime_python/blackwell/sm100_quantize_fp8/runtime_kernel_wrapper_sm100.cu: per-token
                           x 128 quantisation to e4m3 with packed UE8M0 scales (per_token_group_quantize_fp8.cuh).
  runtime_kernel_moe_sigmoid
                           tests/runtime_python/blackwell/sm100_moe_sigmoid/runtime_kernel_wrapper_sm100.cu: grouped
                           sigmoid top-k routing and softmax top-k routing (topk_sigmoid_sm100.cuh, topk_softmax_sm100.cuh).
  runtime_kernel           tests/runtime_python/runtime_kernel_wrapper.cu: the generic task wrappers, of which
                           `multitoken_paged_attention` (tasks/ampere/multitoken_paged_attention.cuh: 4 query heads, 1
                           kv head, q/k RMSNorm, RoPE, append, causal attention over one request's pages) is used.
Not built: the tile wrapper of the tcgen05 bf16 linear (sm100_linear) and the 128-head MLA decode wrapper
(sm100_mla/runtime_kernel_wrapper_mla_decode.cu) -- a process that ran those two one after the other on a B200 did not
return within ten minutes (which of the two stalled is not known); they are not run again.
`bench.py --impl ref_kernel` (one GPU) and the fixture generator tests/golden/make_ref_kernel_golden.py load the
results; nothing else in the repo does."""
import os
import sys

WRAPPERS = {
    "runtime_kernel_fp8_moe": "tests/runtime_python/blackwell/sm100_fp8_moe/runtime_kernel_wrapper.cu",
    "ref_mla_tp8": os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_mla_tp8_ext.cu"),
    "runtime_kernel_blackwell_quantize_fp8": "tests/runtime_python/blackwell/sm100_quantize_fp8/runtime_kernel_wrapper_sm100.cu",
    "runtime_kernel_moe_sigmoid": "tests/runtime_python/blackwell/sm100_moe_sigmoid/runtime_kernel_wrapper_sm100.cu",
    "runtime_kernel": "tests/runtime_python/runtime_kernel_wrapper.cu",
}
# wrappers that are built with their own macro set (tests/runtime_python/setup.py:38-46) instead of the Blackwell one
OWN_FLAGS = {
    "runtime_kernel": ["-O3", "-gencode=arch=compute_100a,code=sm_100a", "-DMIRAGE_UNIT_TEST", "-DMIRAGE_GRACE_HOPPER",
                       "-DMIRAGE_BACKEND_USE_CUDA", "-DMIRAGE_FINGERPRINT_USE_CUDA", "--expt-relaxed-constexpr"],
}


def build(reference: str, names=None) -> None:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    import flashinfer
    from torch.utils.cpp_extension import load
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    cutlass = os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass")
    inc = [os.path.join(reference, p) for p in ("include/mirage", "include/mirage/persistent_kernel",
                                                "include/mirage/persistent_kernel/tasks", "include")]
    inc += [os.path.join(cutlass, "include"), os.path.join(cutlass, "tools", "util", "include"),
            os.path.join(reference, "include/mirage/persistent_kernel/speculative_decoding")]
    flags = ["-O3", "-gencode=arch=compute_100a,code=sm_100a", "-DMIRAGE_GRACE_BLACKWELL", "-DMPK_ENABLE_TMA",
             "-DCUTE_ARCH_TCGEN05_TMEM_ENABLED", "-DCUTE_ARCH_TCGEN05_MXF8F6F4_MMA_ENABLED",
             "-DMIRAGE_BACKEND_USE_CUDA", "-DMIRAGE_FINGERPRINT_USE_CUDA", "--expt-relaxed-constexpr"]
    for name in names or WRAPPERS:
        bdir = os.path.join(out, name)
        os.makedirs(bdir, exist_ok=True)
        try:
            load(name=name, sources=[os.path.join(reference, WRAPPERS[name])], extra_include_paths=inc,
                 extra_cflags=["-DMIRAGE_GRACE_BLACKWELL", "-DMIRAGE_BACKEND_USE_CUDA"],
                 extra_cuda_cflags=OWN_FLAGS.get(name, flags),
                 extra_ldflags=["-lcuda", "-L/usr/local/cuda/lib64/stubs"], build_directory=bdir, verbose=True)
        except ImportError as e:          # no driver on the build machine: the library is built, loading it is not possible here
            print(f"{name}: built, not loadable here ({e})")
        if not os.path.exists(os.path.join(bdir, name + ".so")):
            raise RuntimeError(f"{name}: no library produced")
        print(f"{name}: {os.path.join(bdir, name + '.so')}")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    build(sys.argv[1], sys.argv[2:] or None)
