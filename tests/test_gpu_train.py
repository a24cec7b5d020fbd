"""Training mode: dropout on h (model.py:164,183) with a mask the CPU oracle can reproduce,
and the backward pass against torch.autograd on the oracle (the reference trains through this
block with loss.backward(), train.py:140-141)."""
import numpy as np
import pytest
import torch

import helpers
import philox_ref
from gemmallm_b200 import MOE, synthetic
from oracle import moe_oracle

DT = torch.bfloat16


def test_philox_known_answer():
    """Published Philox4x32-10 vectors (Random123 kat_vectors): zero counter and key; all-ones
    counter and key."""
    z = np.zeros(1, np.uint64)
    got = [int(a[0]) for a in philox_ref.philox4x32_10(z, z, 0, 0)]
    assert got == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]


def make_block(d, E, f, k, p, dev, seed):
    params = helpers.rounded_params(synthetic.make_params(d, E, f, seed=seed), DT)
    g = torch.Generator().manual_seed(seed + 1)
    params["w1"] = synthetic.round_to(params["w1"] * 2.0, DT)
    params["b1"] = synthetic.round_to(torch.randn(E, 2 * f, generator=g) * 0.05, DT)
    params["b2"] = synthetic.round_to(torch.randn(E, d, generator=g) * 0.05, DT)
    params["gate_w"] = synthetic.round_to(params["gate_w"] * 10.0, DT)   # routing with real preferences
    m = MOE(d, num_experts=E, d_ff=f, top_k=k, dropout_ratio=p, device="cuda")
    synthetic.load_into(m, params, DT, dev)
    return m, params


def oracle_run(x, params, k, mask, grad_out, grad_aux):
    """fp32 forward and torch.autograd backward of the oracle; returns outputs and gradients."""
    leaves = {n: t.clone().requires_grad_(True) for n, t in params.items()}
    xl = x.clone().requires_grad_(True)
    o = moe_oracle.moe_forward(xl, leaves, k, h_mask=mask)
    loss = (o["out"] * grad_out).sum() + grad_aux * o["aux"]
    loss.backward()
    return o, xl.grad, {n: t.grad for n, t in leaves.items()}


def close(got, ref, rel, what):
    got, ref = got.float().cpu(), ref.float()
    scale = float(ref.abs().max())
    err = float((got - ref).abs().max())
    assert err <= rel * scale + 1e-6, f"{what}: max-abs {err:.4g} vs scale {scale:.4g}"
    assert float((got - ref).norm()) <= rel * float(ref.norm()) + 1e-6, f"{what}: Frobenius"


@pytest.mark.gpu
@pytest.mark.parametrize("N,d,E,f,k,p", [(300, 128, 8, 256, 2, 0.1), (1000, 256, 4, 264, 2, 0.25),
                                         (64, 64, 8, 128, 2, 0.0), (700, 128, 16, 192, 4, 0.1)])
def test_training_forward_applies_the_reproducible_dropout_mask(cuda_device, N, d, E, f, k, p):
    m, params = make_block(d, E, f, k, p, cuda_device, seed=N)
    m.train()
    x = synthetic.round_to(synthetic.make_input(N, d, seed=N + 5), DT)
    with torch.no_grad():
        out, aux = m(x.to(DT).to(cuda_device).view(1, N, d))
    torch.cuda.synchronize()
    assert m.device_status() == 0
    seed = m.last.get("seed", 0)      # p = 0 without gradients is the inference path: no seed
    mult = torch.from_numpy(philox_ref.dropout_multiplier(N * k, f, p, seed)).view(N, k, f)
    if p > 0:
        kept = float((mult > 0).float().mean())
        assert abs(kept - (1 - p)) < 0.01
    logits = m.last["logits"].cpu()
    with torch.no_grad():
        o = moe_oracle.moe_forward(x, params, k, logits=logits, h_mask=mult)
        plain = moe_oracle.moe_forward(x, params, k, logits=logits)
    ok = ~moe_oracle.tie_rows(o["probs"], k)
    assert torch.equal(m.last["idx"].cpu()[ok].long(), o["idx"][ok])
    got = out.view(N, d).float().cpu()
    err = (got - o["out"])[ok].abs().max()
    assert err <= 2e-2 * o["out"].abs().max()
    if p > 0:   # and it is not the forward without dropout
        assert (got - plain["out"])[ok].abs().max() > 5 * err
    # eval mode: no mask
    m.eval()
    with torch.no_grad():
        out_e, _ = m(x.to(DT).to(cuda_device).view(1, N, d))
    torch.cuda.synchronize()
    assert (out_e.view(N, d).float().cpu() - plain["out"])[ok].abs().max() <= 2e-2 * plain["out"].abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("N,d,E,f,k,p", [(600, 128, 8, 256, 2, 0.1), (1500, 256, 4, 264, 2, 0.0),
                                         (320, 64, 8, 128, 4, 0.2), (2500, 512, 8, 1024, 2, 0.1)])
def test_backward_matches_autograd_on_the_oracle(cuda_device, N, d, E, f, k, p):
    """All gradients of the block (input, gate, both expert Linears with their biases) against
    torch.autograd on the fp32 oracle with the same dropout mask, the same output gradient
    and a load-balancing loss weight. bf16 storage of the intermediate gradients: relative 3e-2."""
    m, params = make_block(d, E, f, k, p, cuda_device, seed=N + 1)
    m.train()
    x = synthetic.round_to(synthetic.make_input(N, d, seed=N + 6), DT)
    g = torch.Generator().manual_seed(N + 7)
    grad_out = synthetic.round_to(torch.randn(N, d, generator=g), DT)
    grad_aux = 0.5
    xd = x.to(DT).to(cuda_device).view(1, N, d).requires_grad_(True)
    res = synthetic.round_to(synthetic.make_input(N, d, seed=N + 8), DT).to(DT).to(cuda_device).view(1, N, d)
    res.requires_grad_(True)
    out, aux = m(xd, residual=res)
    loss = (out.float() * grad_out.to(cuda_device).view(1, N, d)).sum() + grad_aux * aux
    loss.backward()
    torch.cuda.synchronize()
    assert m.device_status() == 0
    seed = m.last["seed"]
    mult = torch.from_numpy(philox_ref.dropout_multiplier(N * k, f, p, seed)).view(N, k, f)
    o, gx, gp = oracle_run(x, params, k, mult, grad_out, grad_aux)
    # the gradients only compare under the same routing: the seeds are chosen so that it is
    assert torch.equal(m.last["idx"].cpu().long(), o["idx"]), "routing differs from the oracle's own"
    close(out.view(N, d), o["out"].detach() + res.detach().view(N, d).float().cpu(), 2e-2, "forward")
    assert torch.equal(res.grad.view(N, d).float().cpu(), grad_out)          # the residual's gradient
    close(xd.grad.view(N, d), gx, 3e-2, "grad x")
    close(m.gate.weight.grad, gp["gate_w"], 3e-2, "grad gate.weight")
    close(m.gate.bias.grad, gp["gate_b"], 3e-2, "grad gate.bias")
    for e, ex in enumerate(m.experts):
        close(ex.gate_and_up.weight.grad, gp["w1"][e], 3e-2, f"grad experts.{e}.gate_and_up.weight")
        close(ex.gate_and_up.bias.grad, gp["b1"][e], 3e-2, f"grad experts.{e}.gate_and_up.bias")
        close(ex.down.weight.grad, gp["w2"][e], 3e-2, f"grad experts.{e}.down.weight")
        close(ex.down.bias.grad, gp["b2"][e], 3e-2, f"grad experts.{e}.down.bias")
    # a second step on the same module: buffers are reused, gradients accumulate
    out2, aux2 = m(xd, residual=res)
    ((out2.float() * grad_out.to(cuda_device).view(1, N, d)).sum() + grad_aux * aux2).backward()
    torch.cuda.synchronize()
    assert torch.isfinite(m.experts[0].down.weight.grad.float()).all()


LORA_NAMES = (("lora_gate_and_up_a", "gu_a"), ("lora_gate_and_up_b", "gu_b"),
              ("lora_down_a", "dn_a"), ("lora_down_b", "dn_b"))


@pytest.mark.gpu
@pytest.mark.parametrize("N,d,E,f,k,p", [(600, 128, 8, 256, 2, 0.1), (900, 256, 4, 264, 2, 0.0)])
def test_fine_tuning_trains_the_lora_tensors(cuda_device, N, d, E, f, k, p):
    """fine_tuning=True under .train() (what the reference's fine-tuning loop runs,
    model.py:175-179,185-189 with train.py's backward): the gradients of the four LoRA Linears
    of every expert, of the base Linears, the gate and the input against torch.autograd on the
    fp32 oracle with the same dropout mask."""
    m, params = make_block(d, E, f, k, p, cuda_device, seed=N + 11)
    g = torch.Generator().manual_seed(N + 12)
    with torch.no_grad():
        for ex in m.experts:
            for name, _ in LORA_NAMES:
                lin = getattr(ex, name)
                lin.weight.copy_(synthetic.round_to(torch.randn(lin.weight.shape, generator=g) * 0.05, DT))
                lin.bias.copy_(synthetic.round_to(torch.randn(lin.bias.shape, generator=g) * 0.05, DT))
    m.train()
    x = synthetic.round_to(synthetic.make_input(N, d, seed=N + 13), DT)
    grad_out = synthetic.round_to(torch.randn(N, d, generator=g), DT)
    grad_aux = 0.25
    xd = x.to(DT).to(cuda_device).view(1, N, d).requires_grad_(True)
    out, aux = m(xd, fine_tuning=True)
    ((out.float() * grad_out.to(cuda_device).view(1, N, d)).sum() + grad_aux * aux).backward()
    torch.cuda.synchronize()
    assert m.device_status() == 0
    mult = torch.from_numpy(philox_ref.dropout_multiplier(N * k, f, p, m.last["seed"])).view(N, k, f)
    leaves = {n: t.clone().requires_grad_(True) for n, t in params.items()}
    lora = []
    for ex in m.experts:
        dct = {"scale": ex.lora_scale}
        for name, short in LORA_NAMES:
            lin = getattr(ex, name)
            dct[short + "_w"] = lin.weight.detach().float().cpu().requires_grad_(True)
            dct[short + "_b"] = lin.bias.detach().float().cpu().requires_grad_(True)
        lora.append(dct)
    xl = x.clone().requires_grad_(True)
    o = moe_oracle.moe_forward(xl, leaves, k, lora=lora, h_mask=mult)
    ((o["out"] * grad_out).sum() + grad_aux * o["aux"]).backward()
    assert torch.equal(m.last["idx"].cpu().long(), o["idx"]), "routing differs from the oracle's own"
    close(out.view(N, d), o["out"].detach(), 2e-2, "forward")
    close(xd.grad.view(N, d), xl.grad, 3e-2, "grad x")
    close(m.gate.weight.grad, leaves["gate_w"].grad, 3e-2, "grad gate.weight")
    for e, ex in enumerate(m.experts):
        close(ex.gate_and_up.weight.grad, leaves["w1"].grad[e], 3e-2, f"grad experts.{e}.gate_and_up.weight")
        close(ex.down.bias.grad, leaves["b2"].grad[e], 3e-2, f"grad experts.{e}.down.bias")
        for name, short in LORA_NAMES:
            lin = getattr(ex, name)
            close(lin.weight.grad, lora[e][short + "_w"].grad, 4e-2, f"grad experts.{e}.{name}.weight")
            close(lin.bias.grad, lora[e][short + "_b"].grad, 4e-2, f"grad experts.{e}.{name}.bias")


@pytest.mark.gpu
def test_training_mode_limits(cuda_device):
    m, _ = make_block(64, 8, 128, 2, 0.1, cuda_device, seed=3)
    m.train()
    x = torch.zeros(1, 16, 64, dtype=DT, device=cuda_device)
    with pytest.raises(NotImplementedError):
        m(x, norm=torch.nn.LayerNorm(64).to(device=cuda_device, dtype=DT))
    with pytest.raises(NotImplementedError):
        m.float()(x.float())


@pytest.mark.gpu
@pytest.mark.parametrize("rows,d,f,p", [(700, 128, 384, 0.1), (64, 64, 128, 0.0), (3000, 256, 520, 0.2)])
def test_dense_feedforward_trains(cuda_device, rows, d, f, p):
    """The reference's dense FeedForward (use_moe=False, model.py:302,316) under .train(): forward
    with the reproducible dropout mask and every gradient against torch.autograd on the oracle's
    expert_ffn (model.py:173-184)."""
    from gemmallm_b200 import FeedForward
    prm = helpers.rounded_params(synthetic.make_params(d, 1, f, seed=rows), DT)
    g = torch.Generator().manual_seed(rows + 1)
    prm["w1"] = synthetic.round_to(prm["w1"] * 2.0, DT)
    prm["b1"] = synthetic.round_to(torch.randn(1, 2 * f, generator=g) * 0.05, DT)
    prm["b2"] = synthetic.round_to(torch.randn(1, d, generator=g) * 0.05, DT)
    ff = FeedForward(d, dropout_ratio=p, d_ff=f).to(device=cuda_device, dtype=DT).train()
    with torch.no_grad():
        ff.gate_and_up.weight.copy_(prm["w1"][0]); ff.gate_and_up.bias.copy_(prm["b1"][0])
        ff.down.weight.copy_(prm["w2"][0]); ff.down.bias.copy_(prm["b2"][0])
    x = synthetic.round_to(synthetic.make_input(rows, d, seed=rows + 2), DT)
    grad_y = synthetic.round_to(torch.randn(rows, d, generator=g), DT)
    xd = x.to(DT).to(cuda_device).view(1, rows, d).requires_grad_(True)
    y = ff(xd)
    (y.float() * grad_y.to(cuda_device).view(1, rows, d)).sum().backward()
    torch.cuda.synchronize()
    mult = torch.from_numpy(philox_ref.dropout_multiplier(rows, f, p, ff.last_seed))
    leaves = [t.clone().requires_grad_(True) for t in (x, prm["w1"][0], prm["b1"][0], prm["w2"][0], prm["b2"][0])]
    ref = moe_oracle.expert_ffn(*leaves, h_mask=mult)
    (ref * grad_y).sum().backward()
    close(y.view(rows, d), ref.detach(), 2e-2, "forward")
    close(xd.grad.view(rows, d), leaves[0].grad, 3e-2, "grad x")
    close(ff.gate_and_up.weight.grad, leaves[1].grad, 3e-2, "grad gate_and_up.weight")
    close(ff.gate_and_up.bias.grad, leaves[2].grad, 3e-2, "grad gate_and_up.bias")
    close(ff.down.weight.grad, leaves[3].grad, 3e-2, "grad down.weight")
    close(ff.down.bias.grad, leaves[4].grad, 3e-2, "grad down.bias")


@pytest.mark.gpu
def test_dense_feedforward_fine_tuning_trains_the_lora_tensors(cuda_device):
    """The dense FeedForward with fine_tuning=True under .train(): LoRA gradients against
    torch.autograd on the oracle's expert_ffn with the same dropout mask."""
    from gemmallm_b200 import FeedForward
    rows, d, f, p = 900, 128, 264, 0.1
    g = torch.Generator().manual_seed(77)
    ff = FeedForward(d, dropout_ratio=p, d_ff=f).to(device=cuda_device, dtype=DT).train()
    with torch.no_grad():
        for prm in ff.parameters():
            prm.copy_(synthetic.round_to(torch.randn(prm.shape, generator=g) * 0.05, DT))
    x = synthetic.round_to(synthetic.make_input(rows, d, seed=78), DT)
    grad_y = synthetic.round_to(torch.randn(rows, d, generator=g), DT)
    xd = x.to(DT).to(cuda_device).view(1, rows, d).requires_grad_(True)
    y = ff(xd, fine_tuning=True)
    (y.float() * grad_y.to(cuda_device).view(1, rows, d)).sum().backward()
    torch.cuda.synchronize()
    mult = torch.from_numpy(philox_ref.dropout_multiplier(rows, f, p, ff.last_seed))
    cpu = lambda t: t.detach().float().cpu().requires_grad_(True)
    lora = {"scale": ff.lora_scale}
    for name, short in LORA_NAMES:
        lora[short + "_w"], lora[short + "_b"] = cpu(getattr(ff, name).weight), cpu(getattr(ff, name).bias)
    xl = x.clone().requires_grad_(True)
    base = [cpu(ff.gate_and_up.weight), cpu(ff.gate_and_up.bias), cpu(ff.down.weight), cpu(ff.down.bias)]
    ref = moe_oracle.expert_ffn(xl, *base, lora, mult)
    (ref * grad_y).sum().backward()
    close(y.view(rows, d), ref.detach(), 2e-2, "forward")
    close(xd.grad.view(rows, d), xl.grad, 3e-2, "grad x")
    close(ff.down.weight.grad, base[2].grad, 3e-2, "grad down.weight")
    for name, short in LORA_NAMES:
        close(getattr(ff, name).weight.grad, lora[short + "_w"].grad, 4e-2, f"grad {name}.weight")
        close(getattr(ff, name).bias.grad, lora[short + "_b"].grad, 4e-2, f"grad {name}.bias")
