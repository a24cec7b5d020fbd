"""Expert-parallel block on 1, 2 and (where present) 4 GPUs, as child processes
(one per GPU) so that a failure cannot take the test process with it."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def run_workers(world, extra=(), port=29541):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "ep_worker.py"),
           *extra]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("EP_OK") == world, r.stdout[-3000:]


@pytest.mark.parametrize("flags", [0, 4, 8])   # default; unfused return; one-CTA GEMM kernel
def test_ep_world_1(cuda_device, flags):
    run_workers(1, ["--tokens", "1000", "--experts", "8", "--topk", "2", "--flags", str(flags)],
                port=29541)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_multi_gpu(cuda_device, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_workers(world, ["--tokens", "4096", "--experts", "16", "--topk", "4"], port=29542 + world)
    run_workers(world, ["--tokens", "2048", "--experts", "64", "--topk", "4", "--dmodel", "512", "--dff", "704",
                        "--placement", "lpt"], port=29552 + world)
    # the three most popular experts copied to every rank
    run_workers(world, ["--tokens", "4096", "--experts", "16", "--topk", "4", "--replicate", "3"],
                port=29562 + world)
