"""Parity of each C-ABI stage with the CPU oracle on the same seeded inputs:
routing indices and counts bit-exact, floating point within stated tolerances."""
import pytest
import torch
import torch.nn.functional as F

import helpers
from gemmallm_b200 import _cabi, synthetic
from oracle import moe_oracle
from gemmallm_b200._cabi import lib, check  # noqa: E402

pytestmark = pytest.mark.gpu

ROUTER_CASES = [
    # N, d, E, k, dtype
    (1, 64, 8, 2, torch.float32), (2, 64, 8, 2, torch.float32), (3, 64, 8, 2, torch.float32),
    (31, 64, 8, 2, torch.float32), (32, 64, 8, 2, torch.float32), (33, 64, 8, 2, torch.float32),
    (127, 64, 8, 2, torch.bfloat16), (128, 64, 8, 2, torch.bfloat16), (129, 64, 8, 2, torch.bfloat16),
    (512, 512, 8, 2, torch.float32), (1000, 256, 64, 4, torch.bfloat16),
    (300, 128, 256, 8, torch.bfloat16), (77, 72, 5, 3, torch.float32), (50, 40, 1, 1, torch.float32),
    (4096, 2048, 64, 4, torch.bfloat16), (20000, 264, 32, 4, torch.bfloat16), (9000, 1024, 24, 2, torch.bfloat16),
    (5, 72, 40, 3, torch.bfloat16), (129, 64, 17, 1, torch.bfloat16), (40000, 512, 64, 8, torch.bfloat16),
]


def make_gate(N, d, E, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    gate_w = synthetic.round_to(torch.randn(E, d, generator=g) * 0.05, dtype)
    gate_b = synthetic.round_to(torch.randn(E, generator=g) * 0.3, dtype)
    x = synthetic.round_to(torch.randn(N, d, generator=g), dtype)
    return x, gate_w, gate_b


@pytest.mark.parametrize("N,d,E,k,dtype", ROUTER_CASES)
def test_router_matches_oracle(cuda_device, N, d, E, k, dtype):
    x, gw, gb = make_gate(N, d, E, dtype, seed=N + d + E)
    logits, idx, w, psum_part = helpers.router(x.to(dtype).to(cuda_device), gw.to(dtype).to(cuda_device),
                                               gb.to(dtype).to(cuda_device), k)
    torch.cuda.synchronize()
    logits, idx, w, psum_part = logits.cpu(), idx.cpu(), w.cpu(), psum_part.cpu()
    ref_logits = F.linear(x, gw, gb)
    assert (logits - ref_logits).abs().max() <= 2e-5 * max(1.0, float(ref_logits.abs().max()))
    # bit-exact routing given the kernel's own fp32 logits
    r = moe_oracle.route_from_logits(logits, k)
    ties = moe_oracle.tie_rows(r["probs"], k)
    ok = ~ties
    assert torch.equal(idx[ok].long(), r["idx"][ok]), "routing indices differ from topk(softmax(logits))"
    assert torch.allclose(w[ok], r["w"][ok], atol=2e-6, rtol=0)
    assert torch.allclose(psum_part.sum(0), r["probs"].sum(0), rtol=1e-5, atol=1e-5)
    assert ((idx >= 0) & (idx < E)).all()
    # no expert twice for one token
    assert (idx.sort(dim=1).values.diff(dim=1) > 0).all() if k > 1 else True


@pytest.mark.parametrize("N,d,E,k", [(1, 1024, 8, 2), (8, 1024, 8, 2), (17, 256, 16, 4), (64, 1024, 8, 2),
                                     (100, 72, 5, 2), (128, 128, 32, 2), (33, 64, 24, 7),
                                     (129, 256, 8, 2), (300, 1024, 8, 2), (512, 512, 32, 2), (200, 128, 16, 5),
                                     (1000, 256, 8, 2), (2048, 128, 16, 4)])
@pytest.mark.parametrize("split", [False, True])
def test_front_small_equals_router_plus_dispatch(cuda_device, N, d, E, k, split):
    """The single-launch front end gives what the two general kernels give, whether every block
    repeats the routing or (beyond 128 tokens) the blocks share it and meet at a counter."""
    if N > 512 and not split:
        pytest.skip("every block repeating the routing is limited to 512 tokens")
    dt = torch.bfloat16
    x, gw, gb = make_gate(N, d, E, dt, seed=N + E)
    xd, gwd, gbd = x.to(dt).to(cuda_device), gw.to(dt).to(cuda_device), gb.to(dt).to(cuda_device)
    logits, idx, w, psum_part = helpers.router(xd, gwd, gbd, k)
    ref = helpers.dispatch(xd, idx, E, psum_part)
    dev = cuda_device
    got = {"logits": torch.empty(N, E, dtype=torch.float32, device=dev),
           "idx": torch.empty(N, k, dtype=torch.int32, device=dev),
           "w": torch.empty(N, k, dtype=torch.float32, device=dev),
           "cnt_slot": torch.empty(k, E, dtype=torch.int32, device=dev),
           "offsets": torch.empty(E + 1, dtype=torch.int32, device=dev),
           "row_of": torch.empty(N, k, dtype=torch.int32, device=dev),
           "perm": torch.empty(N * k, d, dtype=dt, device=dev),
           "psum": torch.empty(E, dtype=torch.float32, device=dev),
           "aux": torch.zeros(1, dtype=torch.float32, device=dev)}
    outs = [got[n].data_ptr() for n in ("logits", "idx", "w", "cnt_slot", "offsets", "row_of", "perm",
                                        "psum", "aux")]
    if split:
        xch = torch.full((helpers.lib.moe_b200_front_exchange_ints(N, E, k),), 0x5A5A5A5A,
                         dtype=torch.int32, device=dev)
        counter = torch.full((1,), 77, dtype=torch.int32, device=dev)    # the call zeroes it
        status = torch.zeros(16, dtype=torch.int32, device=dev)
        for _ in range(2):       # twice: the counter has to be back at zero after a call
            helpers.check(helpers.lib.moe_b200_front_small_split(
                xd.data_ptr(), gwd.data_ptr(), gbd.data_ptr(), N, d, E, k, _cabi.BF16, *outs,
                xch.data_ptr(), counter.data_ptr(), status.data_ptr(), helpers.stream(dev)),
                "front_small_split")
            torch.cuda.synchronize()
            assert status.cpu().tolist()[0] == 0 and int(counter.item()) == 0
    else:
        helpers.check(helpers.lib.moe_b200_front_small(
            xd.data_ptr(), gwd.data_ptr(), gbd.data_ptr(), N, d, E, k, _cabi.BF16, *outs,
            helpers.stream(dev)), "front_small")
    torch.cuda.synchronize()
    assert (got["logits"] - logits).abs().max() <= 2e-5 * max(1.0, float(logits.abs().max()))
    r = moe_oracle.route_from_logits(got["logits"].cpu(), k)
    ok = ~moe_oracle.tie_rows(r["probs"], k)
    assert torch.equal(got["idx"].cpu()[ok].long(), r["idx"][ok])
    assert torch.allclose(got["w"].cpu()[ok], r["w"][ok], atol=2e-6, rtol=0)
    if torch.equal(got["idx"], idx):     # same routing (always, unless a near-tie flips): same layout
        for name in ("cnt_slot", "offsets", "row_of", "perm"):
            assert torch.equal(got[name], ref[name]), name
        assert torch.allclose(got["psum"], ref["psum"], rtol=1e-5, atol=1e-6)
        assert abs(float(got["aux"]) - float(ref["aux"])) <= 1e-5 * abs(float(ref["aux"])) + 1e-7
    else:
        assert torch.equal(got["cnt_slot"].cpu().long(), r["cnt_slot"])


DISPATCH_CASES = [(1, 64, 8, 2), (2, 64, 8, 2), (63, 64, 8, 2), (64, 64, 8, 2), (65, 64, 8, 2),
                  (129, 128, 8, 2), (1000, 256, 64, 4), (5000, 512, 8, 2), (333, 72, 5, 3),
                  (4097, 64, 256, 8), (40000, 64, 8, 2)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N,d,E,k", DISPATCH_CASES)
def test_dispatch_is_a_stable_counting_sort(cuda_device, N, d, E, k, dtype):
    g = torch.Generator().manual_seed(N * 7 + E)
    x = torch.randn(N, d, generator=g).to(dtype)
    # k distinct experts per token, skewed popularity
    score = torch.rand(N, E, generator=g) + torch.linspace(0.5, 0, E)
    idx = score.topk(k, dim=1).indices.to(torch.int32)
    psum_part = torch.rand(max(1, _cabi.lib.moe_b200_router_blocks(N)), E, generator=g)
    out = helpers.dispatch(x.to(cuda_device), idx.to(cuda_device), E, psum_part.to(cuda_device))
    torch.cuda.synchronize()
    cnt_slot, offsets, row_of, perm = (out[n].cpu() for n in ("cnt_slot", "offsets", "row_of", "perm"))
    assert int(out["status"][0]) == 0
    ref_cnt = torch.stack([torch.bincount(idx[:, j].long(), minlength=E) for j in range(k)])
    assert torch.equal(cnt_slot.long(), ref_cnt)
    total = ref_cnt.sum(0)
    assert torch.equal(offsets.long(), torch.cat([torch.zeros(1, dtype=torch.long), total.cumsum(0)]))
    flat = row_of.long().flatten()
    assert torch.equal(flat.sort().values, torch.arange(N * k))          # a permutation
    e_of_row = torch.bucketize(flat, offsets.long()[1:], right=True)
    assert torch.equal(e_of_row, idx.long().flatten())                  # rows land in their expert
    assert torch.equal(perm[flat].view(N, k, d), x[:, None, :].expand(N, k, d))  # rows are copies
    # stable: inside one expert, rows follow token order
    tok_of_row = torch.empty(N * k, dtype=torch.long)
    tok_of_row[flat] = torch.arange(N).repeat_interleave(k)
    for e in range(E):
        seg = tok_of_row[offsets[e]:offsets[e + 1]]
        assert (seg.diff() > 0).all()
    # load-balancing loss from the partial sums, fixed-order reduction
    psum = psum_part.sum(0)
    aux = (psum / N * (ref_cnt[0].float() / N)).mean() * float(E * E)
    assert torch.allclose(out["psum"].cpu(), psum, rtol=1e-5)
    assert abs(float(out["aux"][0]) - float(aux)) <= 1e-5 * abs(float(aux)) + 1e-7


def test_dispatch_reports_bad_index(cuda_device):
    x = torch.randn(10, 64, device=cuda_device)
    idx = torch.zeros(10, 2, dtype=torch.int32, device=cuda_device)
    idx[:, 1] = 1
    idx[4, 1] = 99
    out = helpers.dispatch(x, idx, 8)
    torch.cuda.synchronize()
    assert int(out["status"][0]) == _cabi.DEV_BAD_INDEX
    assert int(out["row_of"][4, 1]) == -1
    assert int(out["offsets"][-1]) == 19


EXPERT_CASES = [
    # rows per expert, d, f
    ([5, 0, 130, 1], 64, 128), ([128, 128], 128, 256), ([127, 129, 0, 0, 300], 256, 384),
    ([1], 64, 64), ([0, 0, 7], 72, 88), ([700, 3, 0, 513, 64, 1, 255, 256], 512, 1024),
]


def expert_inputs(rows, d, f, dtype, seed):
    E = len(rows)
    params = synthetic.make_params(d, E, f, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    params["b1"] = torch.randn(E, 2 * f, generator=g) * 0.05
    params["b2"] = torch.randn(E, d, generator=g) * 0.05
    params["w1"] *= 3.0
    params["w2"] *= 3.0
    params = helpers.rounded_params(params, dtype)
    M = sum(rows)
    x = synthetic.round_to(torch.randn(M, d, generator=g), dtype)
    offsets = torch.tensor([0] + rows).cumsum(0).to(torch.int32)
    return params, x, offsets


def oracle_experts(params, x, offsets):
    hs, ys = [], []
    for e in range(len(offsets) - 1):
        seg = x[offsets[e]:offsets[e + 1]]
        gu = F.linear(seg, params["w1"][e], params["b1"][e])
        gate, up = gu.chunk(2, dim=-1)
        hs.append(F.gelu(gate, approximate="tanh") * up)
        ys.append(moe_oracle.expert_ffn(seg, params["w1"][e], params["b1"][e], params["w2"][e],
                                        params["b2"][e]))
    return torch.cat(hs), torch.cat(ys)


@pytest.mark.parametrize("rows,d,f", EXPERT_CASES)
def test_experts_fp32(cuda_device, rows, d, f):
    params, x, offsets = expert_inputs(rows, d, f, torch.float32, seed=len(rows) + d)
    dp = helpers.device_params(params, torch.float32, cuda_device)
    plan = helpers.Plan(dp["w1"], dp["b1"], dp["w2"], dp["b2"])
    h, y, status = helpers.experts(x.to(cuda_device), offsets.to(cuda_device), plan)
    torch.cuda.synchronize()
    h_ref, y_ref = oracle_experts(params, x, offsets)
    assert (h.cpu() - h_ref).abs().max() <= 1e-4     # fp32 tolerance of the block: max-abs 1e-4
    assert (y.cpu() - y_ref).abs().max() <= 1e-4


@pytest.mark.parametrize("rows,d,f", EXPERT_CASES)
def test_experts_bf16(cuda_device, rows, d, f):
    params, x, offsets = expert_inputs(rows, d, f, torch.bfloat16, seed=len(rows) + d)
    dp = helpers.device_params(params, torch.bfloat16, cuda_device)
    plan = helpers.Plan(dp["w1"], dp["b1"], dp["w2"], dp["b2"])
    h, y, status = helpers.experts(x.to(torch.bfloat16).to(cuda_device), offsets.to(cuda_device),
                                   plan)
    torch.cuda.synchronize()
    assert status.cpu().tolist()[0] == 0, f"device status {status.cpu().tolist()[:4]}"
    h_ref, y_ref = oracle_experts(params, x, offsets)
    # bf16 tolerance of the block: relative error 2e-2 (max-abs over the largest reference value)
    assert (h.float().cpu() - h_ref).abs().max() <= 2e-2 * h_ref.abs().max()
    assert (y.float().cpu() - y_ref).abs().max() <= 2e-2 * y_ref.abs().max()
    assert (y.float().cpu() - y_ref).norm() <= 2e-2 * y_ref.norm()


DECODE_CASES = [
    ([1, 1], 64, 128), ([0, 2, 0, 5, 1], 72, 264), ([16, 0, 17, 15, 20, 30, 2, 28], 1024, 4096),
    ([1, 0, 0, 0, 0, 1, 0, 0], 1024, 4096), ([200, 56], 256, 1408), ([130], 128, 512),
]


@pytest.mark.parametrize("rows,d,f", DECODE_CASES)
def test_experts_decode_path_bf16(cuda_device, rows, d, f):
    """Small-N path: narrow tiles, split-K partial sums; h and sum(part)+bias
    against the oracle at the bf16 tolerance, and against the large-N kernels."""
    params, x, offsets = expert_inputs(rows, d, f, torch.bfloat16, seed=len(rows) + f)
    dp = helpers.device_params(params, torch.bfloat16, cuda_device)
    plan = helpers.Plan(dp["w1"], dp["b1"], dp["w2"], dp["b2"])
    xd, od = x.to(torch.bfloat16).to(cuda_device), offsets.to(cuda_device)
    h, part, status = helpers.experts_decode_fused(xd, od, plan)
    h2, y2, _ = helpers.experts(xd, od, plan)
    torch.cuda.synchronize()
    assert status.cpu().tolist()[0] == 0
    assert not torch.isnan(part).any()
    # same products and fp32 accumulation; the MMA operand roles are swapped, so allow an ulp
    assert (h.float() - h2.float()).abs().max() <= 1e-2 * h2.float().abs().max()
    M = sum(rows)
    e_of_row = torch.bucketize(torch.arange(M), offsets.long()[1:], right=True)
    y = part.sum(0).cpu() + params["b2"][e_of_row]
    h_ref, y_ref = oracle_experts(params, x, offsets)
    assert (h.float().cpu() - h_ref).abs().max() <= 2e-2 * h_ref.abs().max()
    assert (y - y_ref).abs().max() <= 2e-2 * y_ref.abs().max()
    assert (y - y2.float().cpu()).abs().max() <= 1e-2 * y_ref.abs().max()
    # combine_decode == fixed-order sum of the partials, bias, bf16 rounding, weights
    k = 2 if (M % 2 == 0 and len(rows) >= 2) else 1
    N = M // k
    g = torch.Generator().manual_seed(M)
    row_of = torch.randperm(M, generator=g).view(N, k).to(torch.int32)
    idx = e_of_row[row_of.long()].to(torch.int32)
    w = torch.rand(N, k, generator=g)
    res = torch.randn(N, d, generator=g).to(torch.bfloat16)
    out = helpers.combine_decode(part, row_of.to(cuda_device), idx.to(cuda_device),
                                 w.to(cuda_device), plan, res.to(cuda_device))
    torch.cuda.synchronize()
    acc_s = torch.zeros(M, d)
    for sp in range(part.shape[0]):
        acc_s = acc_s + part[sp].cpu()
    yb = (acc_s + params["b2"][e_of_row]).to(torch.bfloat16).float()
    acc = torch.zeros(N, d)
    for j in range(k):
        acc = acc + w[:, j:j + 1] * yb[row_of[:, j].long()]
    assert torch.equal(out.cpu(), (acc + res.float()).to(torch.bfloat16))


@pytest.mark.parametrize("rows,d,f", DECODE_CASES)
def test_experts_decode_fused_repeats_bit_for_bit(cuda_device, rows, d, f):
    """The single-launch small-N kernel walks a static tile list with a fixed summation
    order: h and every partial sum come out bit-identical call after call, also when the
    completion counters it is handed are stale."""
    params, x, offsets = expert_inputs(rows, d, f, torch.bfloat16, seed=len(rows) + f)
    dp = helpers.device_params(params, torch.bfloat16, cuda_device)
    plan = helpers.Plan(dp["w1"], dp["b1"], dp["w2"], dp["b2"])
    xd, od = x.to(torch.bfloat16).to(cuda_device), offsets.to(cuda_device)
    h, part, status = helpers.experts_decode_fused(xd, od, plan)
    for _ in range(2):
        hf, partf, statusf = helpers.experts_decode_fused(xd, od, plan)
        torch.cuda.synchronize()
        assert statusf.cpu().tolist()[0] == 0
        assert torch.equal(hf, h)
        assert torch.equal(partf, part)


@pytest.mark.parametrize("rows,d,f", DECODE_CASES + [([3, 0, 1, 0, 0, 0, 2, 0], 1024, 4096), ([40, 9], 72, 264)])
def test_experts_gemv_bf16(cuda_device, rows, d, f):
    """The matrix-vector streaming kernels for a few rows per expert (any count works):
    h and sum(part) + bias against the oracle and against the single-launch small-N kernel."""
    params, x, offsets = expert_inputs(rows, d, f, torch.bfloat16, seed=len(rows) + f)
    dp = helpers.device_params(params, torch.bfloat16, cuda_device)
    plan = helpers.Plan(dp["w1"], dp["b1"], dp["w2"], dp["b2"])
    xd, od = x.to(torch.bfloat16).to(cuda_device), offsets.to(cuda_device)
    hf, partf, _ = helpers.experts_decode_fused(xd, od, plan)
    h_ref, y_ref = oracle_experts(params, x, offsets)
    M = sum(rows)
    e_of_row = torch.bucketize(torch.arange(M), offsets.long()[1:], right=True)
    for _ in range(2):
        h, part = helpers.experts_gemv(xd, od, plan)
        torch.cuda.synchronize()
        assert not torch.isnan(part).any() and not torch.isnan(h.float()).any()
        assert (h.float().cpu() - h_ref).abs().max() <= 2e-2 * h_ref.abs().max()
        assert (h.float() - hf.float()).abs().max() <= 1e-2 * hf.float().abs().max()
        y = part.sum(0).cpu() + params["b2"][e_of_row]
        assert (y - y_ref).abs().max() <= 2e-2 * y_ref.abs().max()
        assert (part.sum(0) - partf.sum(0)).abs().max() <= 1e-2 * partf.sum(0).abs().max()


@pytest.mark.parametrize("N,d,f,E,k", [(8, 1024, 4096, 8, 2), (8, 256, 200, 8, 4), (5, 2048, 1408, 16, 4),
                                       (1, 64, 24, 4, 4), (8, 128, 264, 32, 8), (8, 64, 64, 8, 8),
                                       (7, 1024, 4096, 8, 2)])
def test_decode_tiny_entry_point(cuda_device, N, d, f, E, k):
    """The one-launch block for one to eight tokens, called directly at sizes where most or all
    experts are hit (more weight rows than its shared memory holds, several column groups per
    block): routing results and output against the oracle, twice in a row."""
    dt = torch.bfloat16
    params = helpers.rounded_params(synthetic.make_params(d, E, f, seed=N + d), dt)
    dp = helpers.device_params(params, dt, cuda_device)
    plan = helpers.Plan(dp["w1"], dp["b1"], dp["w2"], dp["b2"])
    x = synthetic.round_to(synthetic.make_input(N, d, seed=N + f), dt)
    res = synthetic.round_to(synthetic.make_input(N, d, seed=N + f + 1), dt)
    xd, rd = x.to(dt).to(cuda_device), res.to(dt).to(cuda_device)
    for residual in (None, rd):
        r = helpers.decode_tiny(xd, dp["gate_w"], dp["gate_b"], plan, k, f, residual)
        torch.cuda.synchronize()
        assert int(r["status"][0]) == 0
        o = moe_oracle.moe_forward(x, params, k, logits=r["logits"].cpu())
        ok = ~moe_oracle.tie_rows(o["probs"], k)
        assert torch.equal(r["idx"].cpu()[ok].long(), o["idx"][ok])
        assert int(r["offsets"][-1]) == N * k
        assert torch.allclose(r["w"].cpu()[ok], o["w"][ok], atol=2e-6, rtol=0)
        ref = o["out"] if residual is None else o["out"] + res
        got = r["out"].float().cpu()
        assert (got - ref)[ok].abs().max() <= 2e-2 * ref.abs().max()
        assert (got - ref)[ok].norm() <= 2e-2 * ref[ok].norm()


SPEC_CASES = [(1, 64, 128, 2, 2), (8, 1024, 4096, 8, 2), (17, 72, 264, 5, 3), (32, 256, 1408, 32, 4),
              (64, 1024, 4096, 8, 2), (100, 128, 512, 3, 2), (128, 256, 384, 16, 2), (64, 128, 256, 8, 1)]


@pytest.mark.parametrize("N,d,f,E,k", SPEC_CASES)
def test_experts_decode_spec_equals_sorted_path(cuda_device, N, d, f, E, k):
    """The routing-independent small-N kernel works on the unsorted tokens and all
    experts; its partial sums, stored in dispatch row order, match the kernel that
    works on the sorted rows, and sum(part)+bias matches the oracle."""
    dt = torch.bfloat16
    params = synthetic.make_params(d, E, f, seed=N + E)
    g = torch.Generator().manual_seed(N + f)
    params["b1"] = torch.randn(E, 2 * f, generator=g) * 0.05
    params["b2"] = torch.randn(E, d, generator=g) * 0.05
    params["w1"] *= 3.0
    params["w2"] *= 3.0
    params = helpers.rounded_params(params, dt)
    x = synthetic.round_to(torch.randn(N, d, generator=g), dt)
    # random routing with k distinct experts per token; expert E-1 never chosen when E > k
    pool = E - 1 if E > k else E
    idx = torch.stack([torch.randperm(pool, generator=g)[:k] for _ in range(N)]).to(torch.int32)
    dp = helpers.device_params(params, dt, cuda_device)
    plan = helpers.Plan(dp["w1"], dp["b1"], dp["w2"], dp["b2"])
    xd, idxd = x.to(dt).to(cuda_device), idx.to(cuda_device)
    disp = helpers.dispatch(xd, idxd, E)
    h, part, status = helpers.experts_decode_fused(disp["perm"], disp["offsets"], plan)
    for _ in range(2):
        h_all, part_s, status_s = helpers.experts_decode_spec(xd, idxd, disp["offsets"], plan)
        torch.cuda.synchronize()
        assert status_s.cpu().tolist()[0] == 0
        assert not torch.isnan(part_s).any()
        assert (part_s.sum(0) - part.sum(0)).abs().max() <= 1e-3 * part.sum(0).abs().max()
    # h rows of the routed pairs, against the sorted kernel's h
    row_of = disp["row_of"].cpu().long()
    assert h_all.shape[1] == helpers.lib.moe_b200_decode_spec_rows(N)
    for t in range(0, N, max(1, N // 8)):
        for j in range(k):
            got = h_all[int(idx[t, j]), t].float().cpu()
            ref = h[row_of[t, j]].float().cpu()
            assert (got - ref).abs().max() <= 1e-2 * max(1e-3, float(ref.abs().max()))
    # against the oracle
    offsets = disp["offsets"].cpu()
    e_of_row = torch.bucketize(torch.arange(N * k), offsets.long()[1:], right=True)
    _, y_ref = oracle_experts(params, disp["perm"].float().cpu(), offsets)
    y = part_s.sum(0).cpu() + params["b2"][e_of_row]
    assert (y - y_ref).abs().max() <= 2e-2 * y_ref.abs().max()


@pytest.mark.parametrize("rows,d,f,ksplit", [([100, 0, 300, 57], 256, 1024, 2), ([128] * 8, 1024, 4096, 8),
                                             ([513, 1, 255, 256, 0, 700, 31, 64], 512, 2048, 4),
                                             ([40, 50], 72, 520, 1), ([0, 0, 129], 64, 128, 2),
                                             ([20, 33, 1, 40, 7, 64, 0, 65], 256, 1024, 3)])
def test_experts_rows_matches_prefill_kernels(cuda_device, rows, d, f, ksplit):
    """The streaming pipeline on sorted rows (calls between the decode and the prefill sizes):
    h and sum(part) + bias against the prefill kernels and against the oracle, twice in a row."""
    params, x, offsets = expert_inputs(rows, d, f, torch.bfloat16, seed=len(rows) + f)
    dp = helpers.device_params(params, torch.bfloat16, cuda_device)
    plan = helpers.Plan(dp["w1"], dp["b1"], dp["w2"], dp["b2"])
    xd, od = x.to(torch.bfloat16).to(cuda_device), offsets.to(cuda_device)
    h2, y2, _ = helpers.experts(xd, od, plan)
    M = sum(rows)
    e_of_row = torch.bucketize(torch.arange(M), offsets.long()[1:], right=True)
    h_ref, y_ref = oracle_experts(params, x, offsets)
    for _ in range(2):
        h, part, status = helpers.experts_rows(xd, od, plan, ksplit)
        torch.cuda.synchronize()
        assert status.cpu().tolist()[0] == 0
        assert not torch.isnan(part).any() and not torch.isnan(h.float()).any()
        assert (h.float() - h2.float()).abs().max() <= 1e-2 * h2.float().abs().max()
        assert (h.float().cpu() - h_ref).abs().max() <= 2e-2 * h_ref.abs().max()
        y = part.sum(0).cpu() + params["b2"][e_of_row]
        assert (y - y_ref).abs().max() <= 2e-2 * y_ref.abs().max()
        assert (y - y2.float().cpu()).abs().max() <= 1e-2 * y_ref.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N,d,k", [(1, 64, 2), (130, 128, 2), (1000, 512, 4), (33, 72, 1)])
def test_combine_is_exact(cuda_device, N, d, k, dtype):
    g = torch.Generator().manual_seed(N + d)
    y = torch.randn(N * k, d, generator=g).to(dtype)
    row_of = torch.randperm(N * k, generator=g).view(N, k).to(torch.int32)
    w = torch.rand(N, k, generator=g)
    res = torch.randn(N, d, generator=g).to(dtype)
    acc = torch.zeros(N, d)
    for j in range(k):
        acc = acc + w[:, j:j + 1] * y[row_of[:, j].long()].float()
    for residual, expect in ((None, acc), (res, acc + res.float())):
        out = helpers.combine(y.to(cuda_device), row_of.to(cuda_device), w.to(cuda_device),
                              None if residual is None else residual.to(cuda_device))
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), expect.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N,d,E,k", [(777, 256, 8, 2), (64, 1024, 64, 4), (4100, 72, 5, 3)])
def test_layernorm_stage_entry_points(cuda_device, N, d, E, k, dtype):
    """moe_b200_norm_fold + moe_b200_router_norm + moe_b200_dispatch_norm against
    F.layer_norm: row statistics, logits, and the normalised rows in the sorted buffer;
    moe_b200_layernorm against F.layer_norm."""
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(N + d + E)
    x = synthetic.round_to(torch.randn(N, d, generator=g) * (0.3 + torch.rand(N, 1, generator=g) * 3)
                           + 5.0 * torch.randn(N, 1, generator=g), dtype)
    gw = synthetic.round_to(torch.randn(E, d, generator=g) * 0.05, dtype)
    gb = synthetic.round_to(torch.randn(E, generator=g) * 0.1, dtype)
    gamma = synthetic.round_to(1.0 + 0.3 * torch.randn(d, generator=g), dtype)
    beta = synthetic.round_to(0.2 * torch.randn(d, generator=g), dtype)
    dev = cuda_device
    xd, gwd, gbd, gd, bd = (t.to(dtype).to(dev) for t in (x, gw, gb, gamma, beta))
    code = helpers.CODE[dtype]
    s = helpers.stream(dev)
    wn = torch.empty(E, d, dtype=dtype, device=dev)
    c = torch.empty(2 * E, dtype=torch.float32, device=dev)
    check(lib.moe_b200_norm_fold(gwd.data_ptr(), gbd.data_ptr(), gd.data_ptr(), bd.data_ptr(), E, d, code,
                                 wn.data_ptr(), c.data_ptr(), s), "norm_fold")
    logits = torch.empty(N, E, dtype=torch.float32, device=dev)
    idx = torch.empty(N, k, dtype=torch.int32, device=dev)
    w = torch.empty(N, k, dtype=torch.float32, device=dev)
    psum_part = torch.empty(max(1, lib.moe_b200_router_blocks(N)), E, dtype=torch.float32, device=dev)
    stats = torch.empty(N, 2, dtype=torch.float32, device=dev)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    check(lib.moe_b200_router_norm(xd.data_ptr(), wn.data_ptr(), c.data_ptr(), 1e-5, N, d, E, k, code,
                                   logits.data_ptr(), idx.data_ptr(), w.data_ptr(), psum_part.data_ptr(),
                                   stats.data_ptr(), status.data_ptr(), s), "router_norm")
    torch.cuda.synchronize()
    mean = x.mean(1)
    rstd = torch.rsqrt(x.var(1, unbiased=False) + 1e-5)
    assert torch.allclose(stats[:, 0].cpu(), mean, rtol=1e-5, atol=1e-5)
    assert torch.allclose(stats[:, 1].cpu(), rstd, rtol=2e-5, atol=0)
    xn = F.layer_norm(x, (d,), gamma, beta, 1e-5)
    ref_logits = F.linear(xn, gw, gb)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert (logits.cpu() - ref_logits).abs().max() <= tol * max(1.0, float(ref_logits.abs().max()))
    r = moe_oracle.route_from_logits(logits.cpu(), k)
    good = ~moe_oracle.tie_rows(r["probs"], k)
    assert torch.equal(idx.cpu()[good].long(), r["idx"][good])
    # dispatch: rows of the sorted buffer are the normalised rows
    nbytes = lib.moe_b200_dispatch_scratch_bytes(N, E, k)
    scratch = torch.empty(nbytes // 4, dtype=torch.int32, device=dev)
    cnt_slot = torch.empty(k, E, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    row_of = torch.empty(N, k, dtype=torch.int32, device=dev)
    perm = torch.empty(N * k, d, dtype=dtype, device=dev)
    check(lib.moe_b200_dispatch_norm(xd.data_ptr(), idx.data_ptr(), stats.data_ptr(), gd.data_ptr(),
                                     bd.data_ptr(), N, d, E, k, code, scratch.data_ptr(), cnt_slot.data_ptr(),
                                     offsets.data_ptr(), row_of.data_ptr(), perm.data_ptr(), None, None, None,
                                     status.data_ptr(), s), "dispatch_norm")
    out = torch.empty(N, d, dtype=dtype, device=dev)
    check(lib.moe_b200_layernorm(xd.data_ptr(), gd.data_ptr(), bd.data_ptr(), 1e-5, N, d, code, out.data_ptr(), s),
          "layernorm")
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    rtol = 2e-5 if dtype == torch.float32 else 1e-2
    scale = float(xn.abs().max())
    assert (out.float().cpu() - xn).abs().max() <= rtol * scale
    ro = row_of.cpu().long()
    for j in range(k):
        assert (perm.float().cpu()[ro[:, j]] - xn).abs().max() <= rtol * scale
