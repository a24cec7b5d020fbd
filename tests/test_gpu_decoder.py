"""The block inside the reference's own decoder: ``LLM`` of model.py:322-372 (12 pre-norm
layers: LayerNorm -> multi-query attention with RoPE and a sigmoid head gate -> += skip ->
LayerNorm -> MoE -> += skip; 16 query heads, 1 KV head, head_dim 64, context 64), built
from the unmodified reference module under oracle/_ref, with every ``layer.moe`` replaced by
the new block through ``load_state_dict(strict=True)``. The reference's attention, norms
and classifier run as they are (torch ops, bf16); each layer's MoE call is checked
teacher-forced against the CPU oracle on the input it actually saw, and the logits of the
whole forward are compared with the fp32 reference model on the CPU."""
import pytest
import torch

from gemmallm_b200 import MOE, synthetic
from oracle import make_ref, moe_oracle

pytestmark = pytest.mark.gpu

D, HEADS, HEAD_DIM, E, FACTOR, K, S, VOCAB = 1024, 16, 64, 8, 4, 2, 64, 32000


def build_reference_llm(layers, device, seed=0):
    """The reference LLM with the weight rule of the benchmarks (weights ~ N(0, 0.02^2), biases
    0, LayerNorm at its identity), in fp32 on `device`."""
    ref = make_ref.load()
    torch.manual_seed(seed)
    # every Linear is overwritten below: skip torch's own (slow, 1.3 G numbers) initialisation
    reset = torch.nn.Linear.reset_parameters
    torch.nn.Linear.reset_parameters = lambda self: None
    try:
        with torch.device(device):
            llm = ref.LLM(layers, VOCAB, S, D, expansion_factor=FACTOR, head_dim=HEAD_DIM, q_head=HEADS,
                          kv_head=1, use_moe=True, num_experts=E, device=str(device)).eval()
    finally:
        torch.nn.Linear.reset_parameters = reset
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in llm.named_parameters():
            if "pos_emb" in name or "norm" in name:
                continue
            if name.endswith(".bias"):
                p.zero_()
            else:
                p.copy_((torch.randn(p.shape, generator=g) * 0.02).to(p.device))
    return llm


def swap_in_new_blocks(llm, device, dtype):
    """layer.moe := the new block, parameters carried over by the strict state_dict."""
    for layer in llm.transformer:
        new = MOE(D, num_experts=E, expansion_factor=FACTOR, device="cuda").eval()
        new.load_state_dict(layer.moe.state_dict(), strict=True)
        layer.moe = new
        layer.device = str(device)     # where the reference creates its scalar tensors
    llm.device = str(device)
    return llm.to(device=device, dtype=dtype)


def causal_mask(device, dtype):
    return torch.triu(torch.full((S, S), float("-inf"), device=device, dtype=dtype), diagonal=1)


def layer_params(moe):
    """CPU fp32 copies of one block's parameters in the oracle's layout."""
    f32 = lambda t: t.detach().float().cpu()
    return {"gate_w": f32(moe.gate.weight), "gate_b": f32(moe.gate.bias),
            "w1": torch.stack([f32(ex.gate_and_up.weight) for ex in moe.experts]),
            "b1": torch.stack([f32(ex.gate_and_up.bias) for ex in moe.experts]),
            "w2": torch.stack([f32(ex.down.weight) for ex in moe.experts]),
            "b2": torch.stack([f32(ex.down.bias) for ex in moe.experts])}


@pytest.mark.skipif(not make_ref.available(), reason="oracle/_ref/model.py absent (run oracle/make_ref.py)")
@pytest.mark.parametrize("layers,batch", [(12, 16), (2, 512)])
def test_new_block_inside_the_reference_decoder(cuda_device, layers, batch):
    dt = torch.bfloat16
    llm = build_reference_llm(layers, "cpu")
    with torch.no_grad():
        for p in llm.parameters():        # bf16-representable values, so that every run below sees the same numbers
            p.copy_(p.to(dt).float())
    ids = torch.randint(0, VOCAB, (batch, S), generator=torch.Generator().manual_seed(3))
    table = torch.randn(VOCAB, D, generator=torch.Generator().manual_seed(2)) * 0.02
    x = table[ids].to(dt).float()
    # the unmodified reference (its own MoE) in fp32 on the CPU, small batches only
    ref_logits = None
    if batch <= 16:
        with torch.no_grad():
            ref_logits, ref_aux = llm(x.clone(), causal_mask("cpu", torch.float32), False)
    swap_in_new_blocks(llm, cuda_device, torch.float32)
    msg = f"{layers} layers x {batch * S} tokens"
    if ref_logits is not None:
        # (1) drop-in in fp32: the whole forward with the new block in every layer against the
        # reference's own forward. Same arithmetic type, so the logits have to agree closely.
        with torch.no_grad():
            logits32, aux32 = llm(x.to(cuda_device), causal_mask(cuda_device, torch.float32), False)
        torch.cuda.synchronize()
        assert all(layer.moe.device_status() == 0 for layer in llm.transformer)
        scale = float(ref_logits.abs().max())
        per_token = (logits32.cpu() - ref_logits).abs().amax(-1).flatten() / scale
        agree = float((logits32.cpu().argmax(-1) == ref_logits.argmax(-1)).float().mean())
        msg += (f"; fp32 logits vs the reference's forward: per-token max-abs/max median "
                f"{float(per_token.median()):.2e}, worst {float(per_token.max()):.2e}, arg-max agreement {agree:.4f}")
        assert float(per_token.quantile(0.99)) < 1e-3      # a routing flip may move a token; the rest agree
        assert agree > 0.99
        assert abs(float(aux32) - float(ref_aux)) <= 1e-4 * abs(float(ref_aux)) + 1e-7
    # (2) bf16 (the benchmarked type): every layer's MoE call teacher-forced against the oracle on
    # the input it actually saw
    llm.to(dtype=dt)
    trace = []

    def hook(moe, args, output):
        trace.append((moe, args[0].detach(), output[0].detach().clone(), moe.last["logits"].clone()))

    handles = [layer.moe.register_forward_hook(hook) for layer in llm.transformer]
    with torch.no_grad():
        logits, aux = llm(x.to(dt).to(cuda_device), causal_mask(cuda_device, dt), False)
    torch.cuda.synchronize()
    for h in handles:
        h.remove()
    assert torch.isfinite(logits.float()).all()
    assert all(layer.moe.device_status() == 0 for layer in llm.transformer)
    assert len(trace) == layers
    worst = 0.0
    for moe, xin, out, lg in trace:
        n = min(xin.shape[0] * xin.shape[1], 2048)        # tokens are independent (model.py:201)
        xi = xin.reshape(-1, D)[:n].float().cpu()
        with torch.no_grad():
            o = moe_oracle.moe_forward(xi, layer_params(moe), K, logits=lg[:n].cpu())
        ok = ~moe_oracle.tie_rows(o["probs"], K)
        got = out.reshape(-1, D)[:n].float().cpu()
        err = (got - o["out"])[ok].abs().max()
        # bf16 tolerance of the block: relative 2e-2 (against the largest reference value)
        assert err <= 2e-2 * o["out"].abs().max(), f"max-abs {err} vs scale {o['out'].abs().max()}"
        worst = max(worst, float(err / o["out"].abs().max()))
    msg += f"; bf16: worst per-layer relative error of the block {worst:.2e}"
    if ref_logits is not None:
        # informative: a whole bf16 forward (the reference's attention and classifier in bf16 too)
        # against fp32; tokens whose routing flips in some layer end far from the reference
        got = logits.float().cpu()
        per_token = (got - ref_logits).abs().amax(-1).flatten() / float(ref_logits.abs().max())
        agree = float((got.argmax(-1) == ref_logits.argmax(-1)).float().mean())
        msg += (f", bf16 logits vs fp32 reference: per-token max-abs/max median {float(per_token.median()):.2e}, "
                f"90th percentile {float(per_token.quantile(0.9)):.2e}, arg-max agreement {agree:.3f}")
    print(msg)


@pytest.mark.skipif(not make_ref.available(), reason="oracle/_ref/model.py absent (run oracle/make_ref.py)")
def test_decoder_layer_drop_in(cuda_device):
    """gemmallm_b200.LLMLayer against the reference's own LLMLayer (model.py:278-321): the strict
    state_dict loads, and the bf16 layer (attention kernel, second LayerNorm folded into the
    block, skip connection in the combine kernel) reproduces the fp32 reference layer on
    bf16-representable parameters and inputs. A routing flip may move a token; the rest agree."""
    from gemmallm_b200 import LLMLayer
    dt = torch.bfloat16
    llm = build_reference_llm(1, "cpu", seed=5)
    ref_layer = llm.transformer[0]
    g = torch.Generator().manual_seed(6)
    with torch.no_grad():
        for norm in (ref_layer.norm1, ref_layer.norm2):
            norm.weight.copy_(1.0 + 0.2 * torch.randn(D, generator=g))
            norm.bias.copy_(0.1 * torch.randn(D, generator=g))
        for p in ref_layer.parameters():
            p.copy_(p.to(dt).float())
    batch = 8
    x = (torch.randn(batch, S, D, generator=g) * 0.5).to(dt).float()
    with torch.no_grad():
        ref_out, ref_aux = ref_layer(x.clone(), causal_mask("cpu", torch.float32), False)
    new = LLMLayer(D, HEAD_DIM, HEADS, 1, ref_layer.mqa.embedding, expansion_factor=FACTOR, use_moe=True,
                   num_experts=E, device="cuda").eval()
    new.load_state_dict(ref_layer.state_dict(), strict=True)
    new.to(device=cuda_device, dtype=dt)
    with torch.no_grad():
        out, aux = new(x.to(dt).to(cuda_device), causal_mask(cuda_device, dt), False)
    torch.cuda.synchronize()
    assert new.moe.device_status() == 0
    scale = float(ref_out.abs().max())
    per_token = (out.float().cpu() - ref_out).abs().amax(-1).flatten() / scale
    assert float(per_token.median()) < 1e-2, float(per_token.median())
    assert float(per_token.quantile(0.97)) < 3e-2, float(per_token.quantile(0.97))
    assert abs(float(aux) - float(ref_aux)) <= 2e-2 * abs(float(ref_aux)) + 1e-6
