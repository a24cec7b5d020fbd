"""The whole block through the drop-in module (which calls moe_b200_forward)
against the CPU oracle and the fixtures generated from the reference class."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers
from gemmallm_b200 import MOE, _cabi, synthetic
from oracle import moe_oracle

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def sha(t):
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def build(params, d, E, f, k, dtype, dev):
    m = MOE(d, num_experts=E, d_ff=f, top_k=k, device="cuda").eval()
    synthetic.load_into(m, params, dtype, dev)
    return m


def check_against_oracle(m, params, x, k, dtype, dev, residual=None):
    """Routing bit-exact given the kernel's logits; output within the block's
    tolerance under identical routing: fp32 max-abs 1e-4, bf16 relative 2e-2."""
    N, d = x.shape
    xin = x.to(dtype).to(dev).view(1, N, d)
    res = None if residual is None else residual.to(dtype).to(dev).view(1, N, d)
    with torch.no_grad():
        out, aux = m(xin, residual=res)
    torch.cuda.synchronize()
    assert m.device_status() == 0
    last = {n: t.cpu() for n, t in m.last.items()}
    with torch.no_grad():
        o = moe_oracle.moe_forward(x, params, k, logits=last["logits"])
    ties = moe_oracle.tie_rows(o["probs"], k)
    ok = ~ties
    assert torch.equal(last["idx"][ok].long(), o["idx"][ok])
    if not ties.any():
        assert torch.equal(last["cnt_slot"].long(), o["cnt_slot"])
    assert int(last["offsets"][-1]) == N * k
    assert torch.allclose(last["w"][ok], o["w"][ok], atol=2e-6, rtol=0)
    assert abs(float(aux) - float(o["aux"])) <= 1e-5 * abs(float(o["aux"])) + 1e-7
    ref = o["out"] if residual is None else o["out"] + residual
    got = out.view(N, d).float().cpu()
    err = (got - ref)[ok].abs().max()
    if dtype == torch.float32:
        assert err <= 1e-4, f"max-abs {err}"
    else:
        assert err <= 2e-2 * ref.abs().max(), f"max-abs {err} vs scale {ref.abs().max()}"
        assert (got - ref)[ok].norm() <= 2e-2 * ref[ok].norm()
    return last, o


def test_tiny_fixture_from_reference(cuda_device):
    z = np.load(GOLDEN / "tiny_k2.npz")
    z = {n: torch.from_numpy(z[n]) for n in z.files}
    params = {n: z[n] for n in ("gate_w", "gate_b", "w1", "b1", "w2", "b2")}
    m = build(params, 32, 4, 64, 2, torch.float32, cuda_device)
    with torch.no_grad():
        out, aux = m(z["x"].to(cuda_device).view(2, 12, 32))
    torch.cuda.synchronize()
    assert torch.equal(m.last["idx"].cpu(), z["idx"])
    assert torch.equal(m.last["cnt_slot"].cpu(), z["cnt_slot"])
    assert (out.view(24, 32).cpu() - z["out"]).abs().max() <= 1e-4
    assert abs(float(aux) - float(z["aux"])) <= 1e-6


SMALL = [
    # N, d, E, f, k
    (1, 64, 8, 128, 2), (2, 64, 8, 128, 2), (3, 64, 8, 128, 2), (127, 64, 8, 128, 2),
    (128, 64, 8, 128, 2), (129, 64, 8, 128, 2), (1000, 128, 16, 200, 4), (513, 256, 5, 264, 3),
    (2048, 64, 8, 128, 2), (2049, 64, 8, 128, 2),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N,d,E,f,k", SMALL)
def test_small_shapes(cuda_device, N, d, E, f, k, dtype):
    """bf16 with N*k <= 256 takes the small-N weight-streaming kernels, up to 4096 rows the
    streaming kernel on sorted rows, beyond that the prefill kernels: the sizes straddle
    every switch."""
    params = helpers.rounded_params(synthetic.make_params(d, E, f, seed=N), dtype)
    params["w1"] *= 2.0
    x = synthetic.round_to(synthetic.make_input(N, d, seed=N + 1), dtype)
    m = build(params, d, E, f, k, dtype, cuda_device)
    check_against_oracle(m, params, x, k, dtype, cuda_device)
    res = synthetic.round_to(synthetic.make_input(N, d, seed=N + 2), dtype)
    check_against_oracle(m, params, x, k, dtype, cuda_device, residual=res)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_empty_expert_and_one_hot_expert(cuda_device, dtype):
    d, E, f, k, N = 64, 8, 128, 2, 300
    params = helpers.rounded_params(synthetic.make_params(d, E, f, seed=4), dtype)
    params["gate_b"] = torch.tensor([8.0, 4.0, -60.0, -60.0, -60.0, -60.0, -60.0, -60.0])
    x = synthetic.round_to(synthetic.make_input(N, d, seed=5), dtype)
    m = build(params, d, E, f, k, dtype, cuda_device)
    last, _ = check_against_oracle(m, params, x, k, dtype, cuda_device)
    assert last["cnt_slot"][0].tolist() == [N, 0, 0, 0, 0, 0, 0, 0]
    assert last["cnt_slot"][1].tolist() == [0, N, 0, 0, 0, 0, 0, 0]


def test_c0_full_size_fp32(cuda_device):
    wl = synthetic.WORKLOADS["c0"]
    pins = json.loads((GOLDEN / "routing_pins.json").read_text())["c0"]
    params = synthetic.make_params(wl.d_model, wl.n_experts, wl.d_ff, seed=0)
    x = synthetic.make_input(wl.tokens, wl.d_model, seed=1)
    m = build(params, wl.d_model, wl.n_experts, wl.d_ff, wl.top_k, torch.float32, cuda_device)
    last, o = check_against_oracle(m, params, x, wl.top_k, torch.float32, cuda_device)
    # routing equals the reference's routing on its own logits at this seed
    assert sha(last["idx"]) == pins["idx_sha256"]
    assert sha(last["cnt_slot"]) == pins["cnt_slot_sha256"]
    assert abs(float(o["aux"]) - pins["aux"]) < 1e-5


@pytest.mark.parametrize("name", ["c1_uniform", "c1_skew"])
def test_c1_full_size_bf16(cuda_device, name):
    wl = synthetic.WORKLOADS[name]
    pins = json.loads((GOLDEN / "routing_pins.json").read_text())[name]
    params = helpers.rounded_params(
        synthetic.make_params(wl.d_model, wl.n_experts, wl.d_ff, seed=0, gate_bias_kind=wl.gate_bias),
        torch.bfloat16)
    x = synthetic.round_to(synthetic.make_input(wl.tokens, wl.d_model, seed=1), torch.bfloat16)
    m = build(params, wl.d_model, wl.n_experts, wl.d_ff, wl.top_k, torch.bfloat16, cuda_device)
    last, _ = check_against_oracle(m, params, x, wl.top_k, torch.bfloat16, cuda_device)
    assert sha(last["idx"]) == pins["idx_sha256"]
    assert sha(last["cnt_slot"]) == pins["cnt_slot_sha256"]
    if name == "c1_skew":
        share = float(last["cnt_slot"][:, 0].sum()) / (wl.tokens * wl.top_k)
        assert abs(share - pins["expert0_share"]) < 1e-9


@pytest.mark.parametrize("name", ["c2_t1", "c2_t8", "c2_t32", "c2_t64"])
def test_c2_decode_shapes_bf16(cuda_device, name):
    wl = synthetic.WORKLOADS[name]
    params = helpers.rounded_params(
        synthetic.make_params(wl.d_model, wl.n_experts, wl.d_ff, seed=0), torch.bfloat16)
    x = synthetic.round_to(synthetic.make_input(wl.tokens, wl.d_model, seed=1), torch.bfloat16)
    m = build(params, wl.d_model, wl.n_experts, wl.d_ff, wl.top_k, torch.bfloat16, cuda_device)
    res = synthetic.round_to(synthetic.make_input(wl.tokens, wl.d_model, seed=7), torch.bfloat16)
    check_against_oracle(m, params, x, wl.top_k, torch.bfloat16, cuda_device)
    check_against_oracle(m, params, x, wl.top_k, torch.bfloat16, cuda_device, residual=res)


@pytest.mark.parametrize("d,E,f,k", [(1024, 8, 4096, 2), (256, 16, 200, 4), (2048, 8, 1408, 2),
                                     (128, 5, 264, 3), (64, 32, 136, 8), (72, 8, 24, 1)])
def test_one_to_eight_tokens_single_launch(cuda_device, d, E, f, k):
    """bf16 calls of one to eight tokens with fewer rows than experts run routing, both products and
    the weighted sum in one cooperative launch: every token count, shapes whose output columns
    per block need one and two column groups, feature counts that are no multiple of 16, all
    tokens equal (every row on the same k experts), with and without a residual, call after call."""
    params = helpers.rounded_params(synthetic.make_params(d, E, f, seed=d + f), torch.bfloat16)
    m = build(params, d, E, f, k, torch.bfloat16, cuda_device)
    for N in range(1, 9):
        x = synthetic.round_to(synthetic.make_input(N, d, seed=31 * N + k), torch.bfloat16)
        res = synthetic.round_to(synthetic.make_input(N, d, seed=31 * N + 7), torch.bfloat16)
        check_against_oracle(m, params, x, k, torch.bfloat16, cuda_device)
        check_against_oracle(m, params, x, k, torch.bfloat16, cuda_device, residual=res)
        same = x[:1].repeat(N, 1).contiguous()
        check_against_oracle(m, params, same, k, torch.bfloat16, cuda_device, residual=res)


@pytest.mark.parametrize("N,d,E,f,k", [(129, 64, 8, 128, 2), (300, 256, 8, 1024, 2), (512, 512, 8, 2048, 2),
                                       (400, 1024, 8, 4096, 2), (250, 128, 16, 200, 4), (1500, 256, 8, 1024, 2),
                                       (2048, 128, 8, 256, 2)])
def test_mid_sizes_rows_path(cuda_device, N, d, E, f, k):
    """Between the decode and the prefill sizes (257 to 4096 rows) the forward streams the
    weights over the sorted rows: the block's tolerance, with and without a residual, call
    after call."""
    params = helpers.rounded_params(synthetic.make_params(d, E, f, seed=N), torch.bfloat16)
    res = synthetic.round_to(synthetic.make_input(N, d, seed=N + 2), torch.bfloat16)
    m = build(params, d, E, f, k, torch.bfloat16, cuda_device)
    for call in range(2):
        x = synthetic.round_to(synthetic.make_input(N, d, seed=N + 10 + call), torch.bfloat16)
        check_against_oracle(m, params, x, k, torch.bfloat16, cuda_device)
        check_against_oracle(m, params, x, k, torch.bfloat16, cuda_device, residual=res)


def test_small_n_fresh_workspace_and_changing_inputs(cuda_device):
    """The small-N expert kernel runs while the routing kernel is still writing idx/offsets, and
    the combine may become resident before either has finished: every call on a fresh, zeroed
    workspace, and every call whose routing differs from the call before, must still come out
    right (a read of the routing that is served too early shows up here as a time-out or as
    the previous call's routing)."""
    N, d, E, f, k = 128, 64, 8, 128, 2
    params = helpers.rounded_params(synthetic.make_params(d, E, f, seed=0), torch.bfloat16)
    for trial in range(12):
        m = build(params, d, E, f, k, torch.bfloat16, cuda_device)
        for call in range(3):
            x = synthetic.round_to(synthetic.make_input(N, d, seed=100 * trial + call), torch.bfloat16)
            check_against_oracle(m, params, x, k, torch.bfloat16, cuda_device)


@pytest.mark.parametrize("N", [4, 64])
def test_small_n_layers_back_to_back(cuda_device, N):
    """Several blocks launched back to back with no host synchronisation, each one's output the
    next one's input: the first kernel of a block becomes resident while the last kernel of the
    block before it is still running, and has to wait for it before it reads x."""
    d, E, f, k, L = 256, 8, 512, 2, 5
    layers, params = [], []
    for l in range(L):
        p = helpers.rounded_params(synthetic.make_params(d, E, f, seed=10 + l), torch.bfloat16)
        params.append(p)
        layers.append(build(p, d, E, f, k, torch.bfloat16, cuda_device))
    x0 = synthetic.round_to(synthetic.make_input(N, d, seed=3), torch.bfloat16)
    for rep in range(3):      # the first pass also creates plans and workspaces
        xs = [(x0 * (1.0 + 0.25 * rep)).to(torch.bfloat16).to(cuda_device).view(1, N, d)]
        with torch.no_grad():
            for m in layers:
                out, _aux = m(xs[-1], residual=xs[-1])
                xs.append(out)
        torch.cuda.synchronize()
        for l, m in enumerate(layers):
            assert m.device_status() == 0
            xin = xs[l].view(N, d).float().cpu()
            with torch.no_grad():
                o = moe_oracle.moe_forward(xin, params[l], k, logits=m.last["logits"].cpu())
            ok = ~moe_oracle.tie_rows(o["probs"], k)
            assert torch.equal(m.last["idx"].cpu()[ok].long(), o["idx"][ok])
            ref = o["out"] + xin
            got = xs[l + 1].view(N, d).float().cpu()
            assert (got - ref)[ok].abs().max() <= 2e-2 * ref.abs().max()


def test_c4_router_pin(cuda_device):
    wl = synthetic.WORKLOADS["c4"]
    pins = json.loads((GOLDEN / "routing_pins.json").read_text())["c4"]
    g = torch.Generator().manual_seed(0)
    gate_w = (torch.randn(wl.n_experts, wl.d_model, generator=g) * 0.02).to(torch.bfloat16)
    gate_b = synthetic.gate_bias(wl.gate_bias, wl.n_experts).to(torch.bfloat16)
    x = synthetic.make_input(wl.tokens, wl.d_model, seed=1).to(torch.bfloat16)
    _, idx, _, _ = helpers.router(x.to(cuda_device), gate_w.to(cuda_device), gate_b.to(cuda_device),
                                  wl.top_k)
    torch.cuda.synchronize()
    assert sha(idx.cpu()) == pins["idx_sha256"]


def test_c4_shape_bf16(cuda_device):
    """The expert-parallel workload's block on one GPU at its full size: d 2048, f 1408 (eleven
    128-feature GEGLU tiles, not a multiple of 256), 64 experts, top-4, Zipf(1.1) router bias
    (tail experts of a few dozen rows next to one of tens of thousands), 65536 tokens. Routing
    and counts are compared on every token; outputs on a 4096-token slice (tokens are
    independent, model.py:201) under the kernel's own logits."""
    wl = synthetic.WORKLOADS["c4"]
    pins = json.loads((GOLDEN / "routing_pins.json").read_text())["c4"]
    N, d, f, E, k = wl.tokens, wl.d_model, wl.d_ff, wl.n_experts, wl.top_k
    dt = torch.bfloat16
    m = MOE(d, num_experts=E, d_ff=f, top_k=k, device="cuda").eval().to(device=cuda_device, dtype=dt)
    gate_w, gate_b = synthetic.make_gate(d, E, 0, wl.gate_bias)
    w1, w2 = [], []
    with torch.no_grad():
        m.gate.weight.copy_(gate_w)
        m.gate.bias.copy_(gate_b)
        for e, ex in enumerate(m.experts):
            pe = synthetic.make_expert(d, f, e, 0)
            ex.gate_and_up.weight.copy_(pe["w1"]); ex.gate_and_up.bias.zero_()
            ex.down.weight.copy_(pe["w2"]); ex.down.bias.zero_()
            w1.append(synthetic.round_to(pe["w1"], dt))
            w2.append(synthetic.round_to(pe["w2"], dt))
    params = {"gate_w": synthetic.round_to(gate_w, dt), "gate_b": synthetic.round_to(gate_b, dt),
              "w1": w1, "b1": torch.zeros(E, 2 * f), "w2": w2, "b2": torch.zeros(E, d)}
    x = synthetic.round_to(synthetic.make_input(N, d, seed=1), dt)
    with torch.no_grad():
        out, aux = m(x.to(dt).to(cuda_device).view(N // 64, 64, d))
    torch.cuda.synchronize()
    assert m.device_status() == 0
    last = {n: t.cpu() for n, t in m.last.items()}
    # routing on all tokens: bit-exact against topk(softmax(logits)) on the kernel's logits,
    # and equal to the pinned routing of the oracle on its own logits
    r = moe_oracle.route_from_logits(last["logits"], k)
    good = ~moe_oracle.tie_rows(r["probs"], k)
    assert torch.equal(last["idx"][good].long(), r["idx"][good])
    if good.all():
        assert torch.equal(last["cnt_slot"].long(), r["cnt_slot"])
    assert int(last["offsets"][-1]) == N * k
    assert sha(last["idx"]) == pins["idx_sha256"]
    assert abs(float(aux) - float(r["aux"])) <= 1e-5 * abs(float(r["aux"])) + 1e-7
    # outputs on a slice that holds rows of the hot experts and of the tail
    sl = slice(30000, 30000 + 4096)
    with torch.no_grad():
        o = moe_oracle.moe_forward(x[sl], params, k, logits=last["logits"][sl])
    ok = ~moe_oracle.tie_rows(o["probs"], k)
    got = out.view(N, d)[sl].float().cpu()
    err = (got - o["out"])[ok].abs().max()
    assert err <= 2e-2 * o["out"].abs().max(), f"max-abs {err} vs scale {o['out'].abs().max()}"
    assert (got - o["out"])[ok].norm() <= 2e-2 * o["out"][ok].norm()
    assert len(set(o["idx"].flatten().tolist())) >= 48      # the slice reaches the tail experts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N,d,E,f,k", [(5000, 256, 8, 512, 2), (3000, 1024, 64, 264, 4), (100, 128, 8, 256, 2),
                                       (1, 64, 8, 128, 2), (1500, 512, 16, 384, 2)])
def test_layernorm_folded_into_the_block(cuda_device, N, d, E, f, k, dtype):
    """The caller's norm2 (model.py:298,311-312) inside the block: the router forms the row
    statistics and the logits of the normalised row, the dispatch normalises while it copies
    (calls of up to 4096 rows normalise their few rows in a kernel of their own). Reference:
    F.layer_norm in fp32 on the same values, then the oracle; the residual is the tensor
    before the norm (model.py:310,319). Input rows get a mean far from zero and a per-row
    scale, as a residual stream has."""
    import torch.nn.functional as F
    params = helpers.rounded_params(synthetic.make_params(d, E, f, seed=N + 3), dtype)
    params["w1"] *= 2.0
    g = torch.Generator().manual_seed(N + d)
    x = synthetic.make_input(N, d, seed=N + 4) * (0.5 + 2.0 * torch.rand(N, 1, generator=g)) \
        + 3.0 * torch.randn(N, 1, generator=g)
    x = synthetic.round_to(x, dtype)
    gamma = synthetic.round_to(1.0 + 0.2 * torch.randn(d, generator=g), dtype)
    beta = synthetic.round_to(0.1 * torch.randn(d, generator=g), dtype)
    m = build(params, d, E, f, k, dtype, cuda_device)
    norm = torch.nn.LayerNorm(d, eps=1e-5).to(device=cuda_device, dtype=dtype)
    with torch.no_grad():
        norm.weight.copy_(gamma)
        norm.bias.copy_(beta)
        xin = x.to(dtype).to(cuda_device).view(1, N, d)
        out, aux = m(xin, residual=xin, norm=norm)
        out2, _ = m(xin, residual=xin, norm=norm)
    torch.cuda.synchronize()
    assert m.device_status() == 0
    assert torch.equal(out, out2)
    xn = F.layer_norm(x, (d,), gamma, beta, 1e-5)
    last = {n: t.cpu() for n, t in m.last.items()}
    # the kernel's logits against the logits of the fp32-normalised rows
    ref_logits = F.linear(xn, params["gate_w"], params["gate_b"])
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert (last["logits"] - ref_logits).abs().max() <= tol * max(1.0, float(ref_logits.abs().max()))
    with torch.no_grad():
        o = moe_oracle.moe_forward(xn, params, k, logits=last["logits"])
    ok = ~moe_oracle.tie_rows(o["probs"], k)
    assert torch.equal(last["idx"][ok].long(), o["idx"][ok])
    ref = o["out"] + x
    got = out.view(N, d).float().cpu()
    err = (got - ref)[ok].abs().max()
    if dtype == torch.float32:
        assert err <= 1e-4 * max(1.0, float(ref.abs().max())), f"max-abs {err}"
    else:
        assert err <= 2e-2 * ref.abs().max(), f"max-abs {err} vs scale {ref.abs().max()}"
        assert (got - ref)[ok].norm() <= 2e-2 * ref[ok].norm()


def test_state_survives_dtype_change_and_repeat_calls(cuda_device):
    d, E, f, k, N = 64, 8, 128, 2, 200
    params = synthetic.make_params(d, E, f, seed=9)
    m = build(params, d, E, f, k, torch.float32, cuda_device)
    x = synthetic.make_input(N, d, seed=10).to(cuda_device).view(1, N, d)
    with torch.no_grad():
        a, _ = m(x)
        b, _ = m(x)
        assert torch.equal(a, b)                      # deterministic
        m.to(torch.bfloat16)                          # parameter storage moves: plan is rebuilt
        c, _ = m(x.to(torch.bfloat16))
    assert c.dtype == torch.bfloat16
    assert (c.float() - a).abs().max() < 0.05 * a.abs().max() + 1e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fine_tuning_lora_branch(cuda_device, dtype):
    """fine_tuning=True (model.py:175-179,185-189): LoRA folded into merged weights."""
    from test_oracle import lora_dicts
    d, E, f, k, N = 128, 8, 256, 2, 600
    params = helpers.rounded_params(synthetic.make_params(d, E, f, seed=40), dtype)
    x = synthetic.round_to(synthetic.make_input(N, d, seed=41), dtype)
    torch.manual_seed(42)
    m = build(params, d, E, f, k, dtype, cuda_device)
    with torch.no_grad():
        for ex in m.experts:          # LoRA tensors of a size that matters
            for lin in (ex.lora_gate_and_up_a, ex.lora_gate_and_up_b, ex.lora_down_a, ex.lora_down_b):
                lin.weight.normal_(0, 0.05)
                lin.bias.normal_(0, 0.05)
        out, aux = m(x.to(dtype).to(cuda_device).view(1, N, d), fine_tuning=True)
        plain, _ = m(x.to(dtype).to(cuda_device).view(1, N, d))
    torch.cuda.synchronize()
    logits = m.last["logits"].cpu()
    with torch.no_grad():
        o = moe_oracle.moe_forward(x, params, k, logits=logits, lora=lora_dicts(m))
    ok = ~moe_oracle.tie_rows(o["probs"], k)
    err = (out.view(N, d).float().cpu() - o["out"])[ok].abs().max()
    if dtype == torch.float32:
        assert err <= 1e-4
    else:
        assert err <= 2e-2 * o["out"].abs().max()
    assert (out.float() - plain.float()).abs().max() > 10 * err   # not the plain forward


def test_empty_batch(cuda_device):
    m = build(synthetic.make_params(64, 8, 128, seed=1), 64, 8, 128, 2, torch.bfloat16, cuda_device)
    with torch.no_grad():
        out, aux = m(torch.zeros(0, 4, 64, dtype=torch.bfloat16, device=cuda_device))
    torch.cuda.synchronize()
    assert out.shape == (0, 4, 64)
    assert m.last["offsets"].cpu().tolist() == [0] * 9


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 200, 1000])
def test_feedforward_alone(cuda_device, dtype, rows):
    """The expert module on its own (the reference's dense FeedForward, model.py:154-190)
    runs through the grouped kernels with a single group."""
    from gemmallm_b200 import FeedForward
    d, f = 128, 384
    p = helpers.rounded_params(synthetic.make_params(d, 1, f, seed=rows), dtype)
    g = torch.Generator().manual_seed(rows + 1)
    p["b1"] = synthetic.round_to(torch.randn(1, 2 * f, generator=g) * 0.05, dtype)
    p["b2"] = synthetic.round_to(torch.randn(1, d, generator=g) * 0.05, dtype)
    ff = FeedForward(d, d_ff=f).eval().to(device=cuda_device, dtype=dtype)
    with torch.no_grad():
        ff.gate_and_up.weight.copy_(p["w1"][0]); ff.gate_and_up.bias.copy_(p["b1"][0])
        ff.down.weight.copy_(p["w2"][0]); ff.down.bias.copy_(p["b2"][0])
        x = synthetic.round_to(synthetic.make_input(rows, d, seed=rows + 2), dtype)
        y = ff(x.to(dtype).to(cuda_device).view(1, rows, d))
        y2 = ff(x.to(dtype).to(cuda_device).view(1, rows, d))
        ref = moe_oracle.expert_ffn(x, p["w1"][0], p["b1"][0], p["w2"][0], p["b2"][0])
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    err = (y.view(rows, d).float().cpu() - ref).abs().max()
    assert err <= (1e-4 if dtype == torch.float32 else 2e-2 * ref.abs().max())


def test_two_devices_in_one_process():
    """One process driving two GPUs: kernel attributes, occupancy results and SM counts are
    cached per device, so the second device gets its own (a per-process cache would leave its
    kernels without their shared-memory limit)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for dtype, N in ((torch.bfloat16, 6000), (torch.bfloat16, 40), (torch.bfloat16, 700), (torch.float32, 300)):
        d, E, f, k = 256, 8, 512, 2
        params = helpers.rounded_params(synthetic.make_params(d, E, f, seed=N), dtype)
        x = synthetic.round_to(synthetic.make_input(N, d, seed=N + 1), dtype)
        for index in (0, 1, 0):
            dev = torch.device("cuda", index)
            m = build(params, d, E, f, k, dtype, dev)
            check_against_oracle(m, params, x, k, dtype, dev)
