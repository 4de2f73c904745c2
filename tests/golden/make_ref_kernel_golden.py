"""Writes tests/golden/ref_kernel_outputs.pt: outputs of the REFERENCE'S OWN compiled sm100 kernels on seeded inputs.

    python baseline/build_ref_kernels.py <reference checkout>      # once, where the reference sources are
    python tests/golden/make_ref_kernel_golden.py <output.pt>       # on a B200

The two kernels are the ones `bench.py --impl ref_kernel` times: the FP8 expert GEMM of the DeepSeek-V3 W13 shape
(tests/runtime_python/blackwell/sm100_fp8_moe/runtime_kernel_wrapper.cu, entry `fp8_moe_gemm_2d`, grid 8 x 16) and the
16-head absorbed-MLA decode + merge (mla_mtp_decode_tp8_sm100.cuh behind baseline/ref_mla_tp8_ext.cu).  The inputs are
too large to commit (7.5 GB of expert weights) and are regenerated from their seeds by `bench.moe_w13_inputs` /
`bench.mla_dense_inputs` (torch's counter-based CUDA generator); the fixture stores the kernels' outputs, the small
routing tensors, and checksums of the inputs so that a test can tell a generator that drifted from a kernel that did."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import bench  # noqa: E402
from gpu_util import input_checksums  # noqa: E402


def main(path):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    fixture = {}
    rk = bench.load_ref_extension("runtime_kernel_fp8_moe")
    assert rk is not None, "baseline/_ref/runtime_kernel_fp8_moe is not built"
    t = bench.moe_w13_inputs(dev)
    out = torch.zeros(t["B"], t["topk"], t["N"], dtype=torch.bfloat16, device=dev)
    rk.fp8_moe_gemm_2d(t["xq"], t["xs"], t["w"], t["ws"], t["routing"], t["mask"], out, 8, 16)
    torch.cuda.synchronize()
    fixture["moe_w13"] = {"out": out.cpu(), "routing": t["routing"].cpu(), "mask": t["mask"].cpu(),
                          "checksums": input_checksums(t, ("w", "ws", "xq", "xs"))}
    del t, out
    torch.cuda.empty_cache()
    mla = bench.load_ref_extension("ref_mla_tp8")
    assert mla is not None, "baseline/_ref/ref_mla_tp8 is not built"
    t = bench.mla_dense_inputs(dev)
    qpad = torch.zeros(t["B"], 2, 16, 576, dtype=torch.bfloat16, device=dev)
    qpad[:, 0] = t["q"][:, 0]
    out = torch.zeros(t["B"], 2, 16, 512, dtype=torch.bfloat16, device=dev)
    mla.init(qpad, t["kv"], 1, t["scale"])
    mla.run(out)
    torch.cuda.synchronize()
    fixture["mla_dense"] = {"out": out[:, 0].reshape(t["B"], 16 * 512).cpu(), "scale": t["scale"],
                            "checksums": input_checksums(t, ("q", "kv"))}
    torch.save(fixture, path)
    print("wrote", path, {k: tuple(v["out"].shape) for k, v in fixture.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
