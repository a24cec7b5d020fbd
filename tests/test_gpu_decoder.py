"""The block inside a 12-layer pre-norm decoder stack in bf16 (the shape of the
reference's LLMLayer, model.py:305-321: norm1 -> attention -> += skip -> norm2 ->
MoE -> += skip), with the skip connection fused into the block's combine kernel.
The non-MoE parts are plain torch ops of this test harness (multi-query
attention with 16 query heads, 1 KV head, head_dim 64, causal; LayerNorm);
every layer's MoE call is checked teacher-forced against the CPU oracle on the
input it actually saw."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import helpers
from gemmallm_b200 import MOE, synthetic
from oracle import moe_oracle

pytestmark = pytest.mark.gpu


class Layer(nn.Module):
    def __init__(self, d, heads, head_dim, E, f, k):
        super().__init__()
        self.heads, self.head_dim = heads, head_dim
        self.norm1, self.norm2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.q = nn.Linear(d, heads * head_dim)
        self.kv = nn.Linear(d, 2 * head_dim)          # one KV head
        self.o = nn.Linear(heads * head_dim, d)
        self.moe = MOE(d, num_experts=E, d_ff=f, top_k=k, device="cuda")

    def forward(self, x, trace):
        B, S, d = x.shape
        skip = x
        h = self.norm1(x)
        q = self.q(h).view(B, S, self.heads, self.head_dim).transpose(1, 2)
        kk, vv = self.kv(h).view(B, S, 2, self.head_dim).unbind(2)
        kk = kk.unsqueeze(1).expand(B, self.heads, S, self.head_dim)
        vv = vv.unsqueeze(1).expand(B, self.heads, S, self.head_dim)
        a = F.scaled_dot_product_attention(q, kk, vv, is_causal=True)
        x = self.o(a.transpose(1, 2).reshape(B, S, -1)) + skip
        skip = x
        h = self.norm2(x)
        y, aux = self.moe(h, residual=skip)           # `tensor += skip_connection` fused
        trace.append((h.detach(), skip.detach(), y.detach(), self.moe.last["logits"].clone(), aux))
        return y, aux


def check_layer(layer_params, h, skip, y, logits, k):
    N, d = h.shape[0] * h.shape[1], h.shape[2]
    x = h.reshape(N, d).float().cpu()
    with torch.no_grad():
        o = moe_oracle.moe_forward(x, layer_params, k, logits=logits.cpu())
    ok = ~moe_oracle.tie_rows(o["probs"], k)
    ref = o["out"] + skip.reshape(N, d).float().cpu()
    got = y.reshape(N, d).float().cpu()
    err = (got - ref)[ok].abs().max()
    # bf16 tolerance of the block: relative 2e-2 (against the largest reference value)
    assert err <= 2e-2 * ref.abs().max(), f"max-abs {err} vs scale {ref.abs().max()}"
    return float(err / ref.abs().max())


@pytest.mark.parametrize("layers,batch", [(12, 32), (1, 512)])
def test_moe_inside_decoder_stack(cuda_device, layers, batch):
    d, heads, head_dim, E, f, k, S = 1024, 16, 64, 8, 4096, 2, 64
    dt = torch.bfloat16
    torch.manual_seed(0)
    stack, cpu_params = [], []
    for i in range(layers):
        layer = Layer(d, heads, head_dim, E, f, k).eval()
        p = helpers.rounded_params(synthetic.make_params(d, E, f, seed=100 + i), dt)
        synthetic.load_into(layer.moe, p, dt, cuda_device)
        layer.to(device=cuda_device, dtype=dt)
        stack.append(layer)
        cpu_params.append(p)
    table = (torch.randn(32000, d, generator=torch.Generator().manual_seed(2)) * 0.02)
    ids = torch.randint(0, 32000, (batch, S), generator=torch.Generator().manual_seed(3))
    x = table[ids].to(dt).to(cuda_device)
    trace, total_aux = [], 0.0
    with torch.no_grad():
        for layer in stack:
            x, aux = layer(x, trace)
            total_aux = total_aux + aux
    torch.cuda.synchronize()
    assert torch.isfinite(x.float()).all()
    assert all(layer.moe.device_status() == 0 for layer in stack)
    worst = 0.0
    for p, (h, skip, y, logits, aux) in zip(cpu_params, trace):
        worst = max(worst, check_layer(p, h, skip, y, logits, k))
    print(f"{layers} layers x {batch * S} tokens: worst relative error {worst:.3e}, "
          f"mean load-balancing loss {float(total_aux) / layers:.4f}")
