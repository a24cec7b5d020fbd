"""moe_b200_dispatch_static: the dispatch entry point for callers that cannot
allocate device memory where they call from (a hook under a frozen memory pool,
a serving loop with a locked allocator, a binding that only sees the op's own
tensors). Its scratch is a fixed array inside the library, so its results must
equal those of moe_b200_dispatch with a caller-provided scratch buffer, also
when the array still holds a previous call's counters.

Collected last on purpose (file name): a run that stops at the first failure
has then already run every other test.
"""
import pytest
import torch

import helpers
from gemmallm_b200 import _cabi
from gemmallm_b200._cabi import lib, check


def dispatch_static(x, idx, E, psum_part, check_no_alloc=False):
    N, d = x.shape
    k = idx.shape[1]
    dev = x.device
    out = {
        "cnt_slot": torch.empty(k, E, dtype=torch.int32, device=dev),
        "offsets": torch.empty(E + 1, dtype=torch.int32, device=dev),
        "row_of": torch.empty(N, k, dtype=torch.int32, device=dev),
        "perm": torch.empty(N * k, d, dtype=x.dtype, device=dev),
        "psum": torch.empty(E, dtype=torch.float32, device=dev),
        "aux": torch.zeros(1, dtype=torch.float32, device=dev),
        "status": torch.zeros(16, dtype=torch.int32, device=dev),
    }
    if check_no_alloc:
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
    check(lib.moe_b200_dispatch_static(
        x.data_ptr(), idx.data_ptr(), N, d, E, k, helpers.CODE[x.dtype], out["cnt_slot"].data_ptr(),
        out["offsets"].data_ptr(), out["row_of"].data_ptr(), out["perm"].data_ptr(),
        None if psum_part is None else psum_part.data_ptr(), out["psum"].data_ptr(),
        out["aux"].data_ptr(), out["status"].data_ptr(), helpers.stream(dev)), "dispatch_static")
    if check_no_alloc:
        # the call itself took no device memory: the driver reports the same free bytes
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before
    return out


def make_case(N, d, E, k, dtype, seed, dev):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, d, generator=g).to(dtype).to(dev)
    idx = (torch.rand(N, E, generator=g) + torch.linspace(0.7, 0, E)).topk(k, dim=1).indices
    psum_part = torch.rand(max(1, lib.moe_b200_router_blocks(N)), E, generator=g).to(dev)
    return x, idx.to(torch.int32).to(dev), psum_part


@pytest.mark.gpu
def test_static_scratch_matches_caller_scratch_twice_in_a_row(cuda_device):
    # two calls in a row with different shapes: the second one finds the first
    # one's counters in the shared array and must not be affected by them
    for call, (N, d, E, k, dtype, seed) in enumerate(((5000, 256, 8, 2, torch.bfloat16, 1),
                                                     (1234, 128, 64, 4, torch.float32, 2))):
        x, idx, psum_part = make_case(N, d, E, k, dtype, seed, cuda_device)
        ref = helpers.dispatch(x, idx, E, psum_part)
        # the first call on a device looks the array's address up; from the second call on the
        # free device memory must not move
        got = dispatch_static(x, idx, E, psum_part, check_no_alloc=call > 0)
        torch.cuda.synchronize()
        assert int(got["status"][0]) == 0
        # integer and byte results: bit-exact, as in the other dispatch tests
        for name in ("cnt_slot", "offsets", "row_of", "perm"):
            assert torch.equal(got[name], ref[name]), name
        # same kernel, same fixed reduction order: the tolerance the dispatch tests use
        assert torch.allclose(got["psum"], ref["psum"], rtol=1e-5)
        assert abs(float(got["aux"][0]) - float(ref["aux"][0])) <= 1e-5 * abs(float(ref["aux"][0])) + 1e-7


@pytest.mark.gpu
def test_static_scratch_without_loss_sums_and_with_no_tokens(cuda_device):
    # psum_part = NULL: counts, offsets and rows only; N = 0: empty layout
    x, idx, _ = make_case(777, 64, 16, 2, torch.bfloat16, 3, cuda_device)
    ref = helpers.dispatch(x, idx, 16, None)
    got = dispatch_static(x, idx, 16, None, check_no_alloc=True)
    torch.cuda.synchronize()
    for name in ("cnt_slot", "offsets", "row_of", "perm"):
        assert torch.equal(got[name], ref[name]), name
    empty = dispatch_static(x[:0], idx[:0], 16, None)
    torch.cuda.synchronize()
    assert empty["offsets"].cpu().tolist() == [0] * 17
    assert int(empty["cnt_slot"].abs().sum()) == 0


@pytest.mark.gpu
def test_static_scratch_at_its_limit_after_a_smaller_call(cuda_device):
    # a shape whose counters fill the 1 MiB array to the last word, right after a call that
    # left its own counters at the front of it; one more chunk of tokens no longer fits
    E, k, d = 32, 1, 8
    N = 7599 * 64
    assert lib.moe_b200_dispatch_scratch_bytes(N, E, k) == 1 << 20
    assert lib.moe_b200_dispatch_scratch_bytes(N + 1, E, k) > 1 << 20
    xs, idxs, ps = make_case(300, 64, 8, 2, torch.bfloat16, 4, cuda_device)
    dispatch_static(xs, idxs, 8, ps)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(N, d, generator=g).to(cuda_device)
    idx = torch.randint(0, E, (N, k), generator=g).to(torch.int32).to(cuda_device)
    ref = helpers.dispatch(x, idx, E, None)
    got = dispatch_static(x, idx, E, None, check_no_alloc=True)
    torch.cuda.synchronize()
    assert int(got["status"][0]) == 0
    for name in ("cnt_slot", "offsets", "row_of", "perm"):
        assert torch.equal(got[name], ref[name]), name
    x1 = torch.zeros(N + 1, d, device=cuda_device)
    idx1 = torch.zeros(N + 1, k, dtype=torch.int32, device=cuda_device)
    buf = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    rc = lib.moe_b200_dispatch_static(x1.data_ptr(), idx1.data_ptr(), N + 1, d, E, k, _cabi.F32,
                                      buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(),
                                      None, None, None, buf.data_ptr(), helpers.stream(cuda_device))
    assert rc == -5


@pytest.mark.gpu
def test_static_scratch_rejects_shapes_beyond_its_array(cuda_device):
    x = torch.zeros(64, 64, device=cuda_device)
    idx = torch.zeros(64, 8, dtype=torch.int32, device=cuda_device)
    assert lib.moe_b200_dispatch_scratch_bytes(64, 256, 8) > (1 << 20)
    buf = torch.zeros(4096, dtype=torch.int32, device=cuda_device)
    rc = lib.moe_b200_dispatch_static(x.data_ptr(), idx.data_ptr(), 64, 64, 256, 8, _cabi.F32,
                                      buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(),
                                      None, None, None, buf.data_ptr(), helpers.stream(cuda_device))
    assert rc == -5
    assert b"scratch words" in lib.moe_b200_last_error_string()
