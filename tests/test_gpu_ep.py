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


C4_SHAPE = ["--experts", "64", "--topk", "4", "--dmodel", "2048", "--dff", "1408", "--replicate", "16",
            "--check-tokens", "1024"]


def test_ep_world_1(cuda_device):
    run_workers(1, ["--tokens", "1000", "--experts", "8", "--topk", "2"], port=29541)


def test_ep_world_1_with_lora_branches(cuda_device):
    """fine_tuning=True through the expert-parallel module (model.py:175-179,185-189)."""
    run_workers(1, ["--tokens", "1024", "--experts", "8", "--topk", "2", "--lora"], port=29539)


def test_ep_world_1_at_the_benchmarked_shape(cuda_device):
    """The expert-parallel workload's own shape (d 2048, f 1408: 11 GEGLU tiles, not a multiple of
    256; 64 experts, top-4, Zipf popularity, the 16 hottest experts copied) with one rank's
    share of the tokens, through the expert-parallel entry point on one GPU."""
    run_workers(1, ["--tokens", "8192", *C4_SHAPE], port=29540)


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
    run_workers(world, ["--tokens", "2048", "--experts", "16", "--topk", "4", "--lora"], port=29582 + world)
    # the configuration bench.py --gpus N times: real d/f/E/k, 8192 tokens per rank, 16 copies
    run_workers(world, ["--tokens", str(8192 * world), *C4_SHAPE], port=29572 + world)


def test_missing_peer_ends_in_timeout_status(cuda_device):
    """Failure detection without any GPU fault: rank 0 of a 2-rank configuration runs
    alone (the "peer" buffer is a second local allocation that nobody drives), so the
    flags it waits for are never set. Every wait is bounded: the call must come back
    with MOE_B200_DEV_TIMEOUT in the status word, and the context must stay usable."""
    import ctypes as C
    import helpers
    from gemmallm_b200 import _cabi, synthetic
    from gemmallm_b200._cabi import lib, check
    dev = cuda_device
    N, d, f, E, k, world = 256, 128, 256, 8, 2, 2
    dt = torch.bfloat16
    params = synthetic.make_params(d, E, f, seed=0)
    owner = [e % world for e in range(E)]
    local = [e for e in range(E) if owner[e] == 0]
    dp = helpers.device_params(params, dt, dev)
    plan = helpers.Plan(dp["w1"][local].contiguous(), dp["b1"][local].contiguous(),
                        dp["w2"][local].contiguous(), dp["b2"][local].contiguous())
    sbytes = lib.moe_b200_ep_symm_bytes(N, d, E, k, world)
    bufs = [torch.zeros(sbytes + 1024, dtype=torch.uint8, device=dev) for _ in range(world)]
    bases = (C.c_void_p * world)(*[(b.data_ptr() + 1023) & ~1023 for b in bufs])
    wbytes = lib.moe_b200_ep_workspace_bytes(N, d, f, E, k, world)
    ws = torch.zeros(wbytes + 1024, dtype=torch.uint8, device=dev)
    ws_base = (ws.data_ptr() + 1023) & ~1023
    lay = _cabi.ep_workspace_layout(N, d, f, E, k, world)
    x = synthetic.make_input(N, d, seed=1).to(dt).to(dev)
    out = torch.empty_like(x)
    vmap = (C.c_int32 * (E * world))(*[e for e in range(E) for _ in range(world)])
    check(lib.moe_b200_ep_setup((C.c_int32 * E)(*owner), vmap, N, d, f, E, k, world, E, ws_base, wbytes,
                                helpers.stream(dev)), "ep_setup")
    torch.cuda.synchronize()
    check(lib.moe_b200_ep_forward(x.data_ptr(), dp["gate_w"].data_ptr(), dp["gate_b"].data_ptr(),
                                  plan.ptr, None, N, d, f, E, k, _cabi.BF16, 0, 0, world, E,
                                  len(local), bases, ws_base, wbytes,
                                  out.data_ptr(), None, helpers.stream(dev)), "ep_forward")
    torch.cuda.synchronize()                      # returns: no wait is unbounded
    status = _cabi.read_status(ws_base + lay["status"], helpers.stream(dev))
    assert status[0] == _cabi.DEV_TIMEOUT
    # the context is intact: an ordinary call still works afterwards
    logits, idx, w, _ = helpers.router(x, dp["gate_w"], dp["gate_b"], k)
    torch.cuda.synchronize()
    assert int(idx.min()) >= 0
