"""Generate the golden fixtures from the reference implementation.

Run where the reference checkout is importable (its directory as argv[1] or
$MOE_REFERENCE_DIR):

    python tests/golden/make_golden.py /path/to/GemmaLLM

It imports the reference ``model.MOE`` (model.py:192-276), loads seeded
parameters into it, runs its CPU fp32 forward, checks that oracle/moe_oracle.py
is bit-identical on the same inputs, and writes

  tiny_k2.npz        parameters, input and every reference result of a small
                     block (E=4, d=32, f=64, N=24, k=2)
  routing_pins.json  SHA-256 of the routing indices and per-slot counts of the
                     named workloads' routers (reference for k=2 shapes, the
                     oracle's k-slot generalisation for the k=4 shape, which
                     the reference class cannot express), plus tie counts and
                     expert shares.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from gemmallm_b200 import synthetic  # noqa: E402
from oracle import moe_oracle  # noqa: E402


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def reference_moe(ref_dir: str, d: int, E: int, factor: int, params: dict):
    sys.path.insert(0, ref_dir)
    from model import MOE  # the reference class
    m = MOE(d, num_experts=E, expansion_factor=factor, device="cpu").eval()
    synthetic.load_into(m, params, torch.float32, "cpu")
    return m


def tiny(ref_dir: str) -> None:
    d, E, factor, N, k = 32, 4, 2, 24, 2
    f = d * factor
    params = synthetic.make_params(d, E, f, seed=10)
    g = torch.Generator().manual_seed(11)
    params["gate_b"] = torch.randn(E, generator=g) * 0.1
    params["b1"] = torch.randn(E, 2 * f, generator=g) * 0.02
    params["b2"] = torch.randn(E, d, generator=g) * 0.02
    x = synthetic.make_input(N, d, seed=12)
    ref = reference_moe(ref_dir, d, E, factor, params)
    with torch.no_grad():
        out, aux = ref(x.reshape(2, N // 2, d))
        o = moe_oracle.moe_forward(x, params, k)
    assert torch.equal(out.reshape(N, d), o["out"]), "oracle != reference (tiny)"
    assert torch.equal(aux, o["aux"])
    np.savez(HERE / "tiny_k2.npz",
             x=x.numpy(), out=out.reshape(N, d).numpy(), aux=aux.numpy(),
             logits=o["logits"].numpy(), idx=o["idx"].numpy().astype(np.int32),
             w=o["w"].numpy(), cnt_slot=o["cnt_slot"].numpy().astype(np.int32),
             **{name: t.numpy() for name, t in params.items()})
    print("tiny_k2.npz written; oracle == reference bit for bit")


def routing_pins(ref_dir: str) -> None:
    pins = {}
    for name in ("c0", "c1_uniform", "c1_skew", "c4"):
        wl = synthetic.WORKLOADS[name]
        dt = synthetic.torch_dtype(wl.dtype)
        g = torch.Generator().manual_seed(0)
        gate_w = synthetic.round_to(torch.randn(wl.n_experts, wl.d_model, generator=g) * 0.02, dt)
        gate_b = synthetic.round_to(synthetic.gate_bias(wl.gate_bias, wl.n_experts), dt)
        x = synthetic.round_to(synthetic.make_input(wl.tokens, wl.d_model, seed=1), dt)
        with torch.no_grad():
            logits = F.linear(x, gate_w, gate_b)
            r = moe_oracle.route_from_logits(logits, wl.top_k)
        ties = int(moe_oracle.tie_rows(r["probs"], wl.top_k).sum())
        total = r["cnt_slot"].sum(0)
        pins[name] = {
            "tokens": wl.tokens, "top_k": wl.top_k, "n_experts": wl.n_experts,
            "idx_sha256": sha(r["idx"].to(torch.int32)),
            "cnt_slot_sha256": sha(r["cnt_slot"].to(torch.int32)),
            "cnt_slot": r["cnt_slot"].tolist() if wl.n_experts <= 8 else None,
            "tie_rows": ties,
            "expert0_share": float(total[0]) / float(total.sum()),
            "source": "reference model.MOE" if wl.top_k == 2 else "oracle (k-slot generalisation)",
        }
        print(name, "ties", ties, "expert0 share %.3f" % pins[name]["expert0_share"])

    # the k=2 pins come from the reference class itself: full forward at c0 and
    # c1 shapes, compared with the oracle bit for bit
    for name in ("c0", "c1_uniform"):
        wl = synthetic.WORKLOADS[name]
        dt = synthetic.torch_dtype(wl.dtype)
        params = {n: synthetic.round_to(t, dt) for n, t in synthetic.make_params(
            wl.d_model, wl.n_experts, wl.d_ff, seed=0, gate_bias_kind=wl.gate_bias).items()}
        x = synthetic.round_to(synthetic.make_input(wl.tokens, wl.d_model, seed=1), dt)
        ref = reference_moe(ref_dir, wl.d_model, wl.n_experts, wl.d_ff // wl.d_model, params)
        with torch.no_grad():
            out, aux = ref(x.reshape(8, wl.tokens // 8, wl.d_model))
            o = moe_oracle.moe_forward(x, params, wl.top_k)
        same = torch.equal(out.reshape(wl.tokens, wl.d_model), o["out"])
        close = float((out.reshape(wl.tokens, wl.d_model) - o["out"]).abs().max())
        assert sha(o["idx"].to(torch.int32)) == pins[name]["idx_sha256"]
        pins[name]["oracle_equals_reference"] = bool(same)
        pins[name]["oracle_vs_reference_max_abs"] = close
        pins[name]["aux"] = float(aux)
        pins[name]["out_abs_max"] = float(out.abs().max())
        print(name, "oracle == reference:", same, "max abs diff", close)
        assert close < 1e-6
    (HERE / "routing_pins.json").write_text(json.dumps(pins, indent=1) + "\n")
    print("routing_pins.json written")


if __name__ == "__main__":
    ref_dir = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MOE_REFERENCE_DIR", "")
    if not ref_dir or not Path(ref_dir, "model.py").exists():
        sys.exit("usage: make_golden.py <reference checkout containing model.py>")
    torch.manual_seed(0)
    tiny(ref_dir)
    routing_pins(ref_dir)
