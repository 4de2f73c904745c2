"""Tensor-parallel parity on real GPUs: spawns tests/tp_worker.py under torchrun on every GPU count the box
offers (2, 4, 8).  Skipped on a single-GPU box."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("shard_lm_head", [False, True])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_parity(world, shard_lm_head):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TP_SHARD_LM_HEAD="1" if shard_lm_head else "0")
    port = 29700 + world + (20 if shard_lm_head else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert f"TP={world} parity ok" in out.stdout


@pytest.mark.parametrize("world", [2, 4])
def test_deepseek_slice_tensor_and_expert_parallel(world):
    """The DeepSeek-V3 slice with heads / MLP columns tensor parallel and the routed experts split by rank."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29750 + world), os.path.join(ROOT, "tests", "ds_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert f"TP/EP={world} parity ok" in out.stdout
