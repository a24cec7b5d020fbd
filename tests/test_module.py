"""Host-side drop-in contract of the module: constructor, parameter names and
shapes, state_dict round trips with the reference class, error behaviour."""
import os
import sys
from pathlib import Path

import pytest
import torch

from gemmallm_b200 import MOE, FeedForward

# a reference checkout next to this repository, or wherever MOE_REFERENCE_DIR points
REF_DIR = os.environ.get("MOE_REFERENCE_DIR", str(Path(__file__).resolve().parents[2] / "reference"))


def expected_keys(E):
    keys = ["gate.weight", "gate.bias"]
    for i in range(E):
        for m in ("gate_and_up", "down", "lora_gate_and_up_a", "lora_gate_and_up_b", "lora_down_a",
                  "lora_down_b"):
            keys += [f"experts.{i}.{m}.weight", f"experts.{i}.{m}.bias"]
    return keys


def test_state_dict_layout():
    m = MOE(64, num_experts=8, expansion_factor=4, device="cpu")
    sd = m.state_dict()
    assert list(sd) == expected_keys(8) and len(sd) == 98
    assert sd["gate.weight"].shape == (8, 64)
    assert sd["experts.3.gate_and_up.weight"].shape == (512, 64)
    assert sd["experts.3.gate_and_up.bias"].shape == (512,)
    assert sd["experts.3.down.weight"].shape == (64, 256)
    assert sd["experts.3.lora_gate_and_up_a.weight"].shape == (16, 64)
    assert sd["experts.3.lora_gate_and_up_b.weight"].shape == (512, 16)
    assert sd["experts.3.lora_down_a.weight"].shape == (16, 256)
    assert sd["experts.3.lora_down_b.weight"].shape == (64, 16)
    assert m.num_experts == 8 and m.device == "cpu"
    assert isinstance(m.experts, torch.nn.ModuleList)
    assert isinstance(m.experts[0].dropout, torch.nn.Dropout)
    assert m.experts[0].lora_scale == 2.0
    lora = [n for n, _ in m.named_parameters() if "lora" in n]
    assert len(lora) == 8 * 8


def test_keyword_extensions():
    m = MOE(64, num_experts=16, top_k=4, d_ff=88)
    assert m.top_k == 4 and m.d_ff == 88
    assert m.experts[0].gate_and_up.weight.shape == (176, 64)


@pytest.mark.skipif(not Path(REF_DIR, "model.py").exists(), reason="no reference checkout")
def test_state_dict_round_trip_with_reference():
    sys.path.insert(0, REF_DIR)
    from model import MOE as RefMOE
    ref = RefMOE(32, num_experts=4, expansion_factor=2, device="cpu")
    new = MOE(32, num_experts=4, expansion_factor=2, device="cpu")
    assert list(ref.state_dict()) == list(new.state_dict())
    new.load_state_dict(ref.state_dict(), strict=True)
    for (n1, p1), (n2, p2) in zip(ref.state_dict().items(), new.state_dict().items()):
        assert n1 == n2 and torch.equal(p1, p2)
    ref.load_state_dict(new.state_dict(), strict=True)
    assert [n for n, _ in ref.named_modules()] == [n for n, _ in new.named_modules()]


def test_no_cpu_path_and_unimplemented_branches_raise():
    m = MOE(32, num_experts=4, expansion_factor=2).eval()
    x = torch.zeros(1, 4, 32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(x)
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(x, fine_tuning=True)
    m.train()
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(x)
    ff = FeedForward(32, 2).eval()
    with pytest.raises(RuntimeError, match="no CPU path"):
        ff(x)
