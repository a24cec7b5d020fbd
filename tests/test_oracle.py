"""The CPU oracle against the fixtures generated from the reference class
(tests/golden/make_golden.py) and, where a reference checkout is present,
against the reference class itself."""
import hashlib
import json
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from gemmallm_b200 import synthetic
from oracle import moe_oracle

GOLDEN = Path(__file__).resolve().parent / "golden"
# a reference checkout next to this repository, or wherever MOE_REFERENCE_DIR points
REF_DIR = os.environ.get("MOE_REFERENCE_DIR", str(Path(__file__).resolve().parents[2] / "reference"))


def sha(t):
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def load_tiny():
    z = np.load(GOLDEN / "tiny_k2.npz")
    return {k: torch.from_numpy(z[k]) for k in z.files}


def test_tiny_fixture_replays():
    z = load_tiny()
    params = {n: z[n] for n in ("gate_w", "gate_b", "w1", "b1", "w2", "b2")}
    with torch.no_grad():
        o = moe_oracle.moe_forward(z["x"], params, k=2)
    assert torch.equal(o["idx"].to(torch.int32), z["idx"])
    assert torch.equal(o["cnt_slot"].to(torch.int32), z["cnt_slot"])
    # fp32 sums depend on the BLAS thread count: tolerance, not bits
    assert torch.allclose(o["out"], z["out"], atol=1e-6, rtol=0)
    assert torch.allclose(o["w"], z["w"], atol=1e-7, rtol=0)
    assert abs(float(o["aux"]) - float(z["aux"])) < 1e-6


@pytest.mark.parametrize("name", ["c0", "c1_uniform", "c1_skew", "c4"])
def test_routing_pins(name):
    pins = json.loads((GOLDEN / "routing_pins.json").read_text())[name]
    wl = synthetic.WORKLOADS[name]
    dt = synthetic.torch_dtype(wl.dtype)
    g = torch.Generator().manual_seed(0)
    gate_w = synthetic.round_to(torch.randn(wl.n_experts, wl.d_model, generator=g) * 0.02, dt)
    gate_b = synthetic.round_to(synthetic.gate_bias(wl.gate_bias, wl.n_experts), dt)
    x = synthetic.round_to(synthetic.make_input(wl.tokens, wl.d_model, seed=1), dt)
    with torch.no_grad():
        r = moe_oracle.route_from_logits(F.linear(x, gate_w, gate_b), wl.top_k)
    assert int(moe_oracle.tie_rows(r["probs"], wl.top_k).sum()) == pins["tie_rows"] == 0
    assert sha(r["idx"].to(torch.int32)) == pins["idx_sha256"]
    assert sha(r["cnt_slot"].to(torch.int32)) == pins["cnt_slot_sha256"]
    assert int(r["cnt_slot"].sum()) == wl.tokens * wl.top_k


def test_tie_rows_detects_equal_probabilities():
    p = torch.tensor([[0.25, 0.25, 0.25, 0.25], [0.4, 0.3, 0.2, 0.1], [0.4, 0.2, 0.2, 0.2],
                      [0.3, 0.3, 0.3, 0.1]])
    assert moe_oracle.tie_rows(p, 2).tolist() == [True, False, True, True]
    assert moe_oracle.tie_rows(p, 1).tolist() == [True, False, False, True]


def test_weights_sum_to_one_and_slots_ordered():
    torch.manual_seed(3)
    logits = torch.randn(257, 16)
    r = moe_oracle.route_from_logits(logits, 4)
    assert torch.allclose(r["w"].sum(1), torch.ones(257), atol=1e-6)
    assert (r["vals"][:, :-1] >= r["vals"][:, 1:]).all()
    assert int(r["cnt_slot"].sum()) == 257 * 4


def test_empty_expert_and_single_token():
    params = synthetic.make_params(16, 4, 32, seed=5)
    params["gate_b"] = torch.tensor([0.0, 0.0, -50.0, 0.0])  # expert 2 never chosen
    x = synthetic.make_input(1, 16, seed=6)
    with torch.no_grad():
        o = moe_oracle.moe_forward(x, params, 2)
    assert o["out"].shape == (1, 16)
    assert int(o["cnt_slot"][:, 2].sum()) == 0


@pytest.mark.skipif(not Path(REF_DIR, "model.py").exists(), reason="no reference checkout")
def test_oracle_equals_reference_class():
    sys.path.insert(0, REF_DIR)
    from model import MOE
    d, E, factor, N = 48, 8, 3, 96
    params = synthetic.make_params(d, E, d * factor, seed=21)
    params["gate_b"] = torch.linspace(-0.3, 0.3, E)
    x = synthetic.make_input(N, d, seed=22)
    ref = MOE(d, num_experts=E, expansion_factor=factor, device="cpu").eval()
    synthetic.load_into(ref, params, torch.float32, "cpu")
    with torch.no_grad():
        out, aux = ref(x.reshape(4, N // 4, d))
        o = moe_oracle.moe_forward(x, params, 2)
    assert torch.equal(out.reshape(N, d), o["out"])
    assert torch.equal(aux, o["aux"])


def lora_dicts(module):
    """Per-expert LoRA tensors of a (reference or drop-in) MOE module, for the oracle."""
    out = []
    for ex in module.experts:
        out.append({
            "scale": ex.lora_scale,
            "gu_a_w": ex.lora_gate_and_up_a.weight.detach().float().cpu(),
            "gu_a_b": ex.lora_gate_and_up_a.bias.detach().float().cpu(),
            "gu_b_w": ex.lora_gate_and_up_b.weight.detach().float().cpu(),
            "gu_b_b": ex.lora_gate_and_up_b.bias.detach().float().cpu(),
            "dn_a_w": ex.lora_down_a.weight.detach().float().cpu(),
            "dn_a_b": ex.lora_down_a.bias.detach().float().cpu(),
            "dn_b_w": ex.lora_down_b.weight.detach().float().cpu(),
            "dn_b_b": ex.lora_down_b.bias.detach().float().cpu(),
        })
    return out


@pytest.mark.skipif(not Path(REF_DIR, "model.py").exists(), reason="no reference checkout")
def test_oracle_lora_branch_equals_reference_class():
    sys.path.insert(0, REF_DIR)
    from model import MOE
    d, E, factor, N = 32, 4, 2, 64
    params = synthetic.make_params(d, E, d * factor, seed=31)
    x = synthetic.make_input(N, d, seed=32)
    torch.manual_seed(33)
    ref = MOE(d, num_experts=E, expansion_factor=factor, device="cpu").eval()   # default-initialised LoRA
    synthetic.load_into(ref, params, torch.float32, "cpu")
    with torch.no_grad():
        out, aux = ref(x.reshape(2, N // 2, d), fine_tuning=True)
        o = moe_oracle.moe_forward(x, params, 2, lora=lora_dicts(ref))
        plain = moe_oracle.moe_forward(x, params, 2)
    assert torch.equal(out.reshape(N, d), o["out"])
    assert not torch.equal(o["out"], plain["out"])        # the branch does something
