"""Seeded synthetic parameters and inputs for the named workloads.

The reference trains on Wikipedia token files that are not part of either
repository; every test and benchmark here uses these generators instead:
weights ~ N(0, 0.02^2), biases 0, inputs ~ N(0, 1), all drawn on the CPU from
``torch.Generator`` in parameter-registration order so that the CUDA path and
the CPU oracle see the same bits.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    tokens: int
    d_model: int
    n_experts: int
    d_ff: int
    top_k: int
    dtype: str            # "f32" | "bf16"
    gate_bias: str = "zero"   # "zero" | "expert0+2" | "zipf1.1"


WORKLOADS = {
    # single block at the reference's own CPU-runnable scale
    "c0": Workload("c0", 512, 512, 8, 2048, 2, "f32"),
    # prefill on one B200, uniform and skewed routing
    "c1_uniform": Workload("c1_uniform", 16384, 1024, 8, 4096, 2, "bf16"),
    "c1_skew": Workload("c1_skew", 16384, 1024, 8, 4096, 2, "bf16", "expert0+2"),
    # decode-shaped calls of the same block
    "c2_t1": Workload("c2_t1", 1, 1024, 8, 4096, 2, "bf16"),
    "c2_t8": Workload("c2_t8", 8, 1024, 8, 4096, 2, "bf16"),
    "c2_t32": Workload("c2_t32", 32, 1024, 8, 4096, 2, "bf16"),
    "c2_t64": Workload("c2_t64", 64, 1024, 8, 4096, 2, "bf16"),
    # the same block at batch sizes between decode and prefill (not BASELINE configurations)
    "c2_t256": Workload("c2_t256", 256, 1024, 8, 4096, 2, "bf16"),
    "c2_t1024": Workload("c2_t1024", 1024, 1024, 8, 4096, 2, "bf16"),
    # per-layer shape of the 12-layer decoder forward (batch 512 x context 64)
    "c3_layer": Workload("c3_layer", 32768, 1024, 8, 4096, 2, "bf16"),
    # expert-parallel block, Zipf(1.1) expert popularity
    "c4": Workload("c4", 65536, 2048, 64, 1408, 4, "bf16", "zipf1.1"),
}


def torch_dtype(name: str) -> torch.dtype:
    return {"f32": torch.float32, "bf16": torch.bfloat16}[name]


def gate_bias(kind: str, E: int) -> torch.Tensor:
    if kind == "zero":
        return torch.zeros(E)
    if kind == "expert0+2":
        b = torch.zeros(E)
        b[0] = 2.0
        return b
    if kind == "zipf1.1":
        return torch.tensor([-1.1 * math.log(e + 1) for e in range(E)], dtype=torch.float32)
    raise ValueError(kind)


def make_params(d: int, E: int, f: int, seed: int = 0, gate_bias_kind: str = "zero") -> dict:
    """fp32 CPU tensors: gate_w [E,d], gate_b [E], w1 [E,2f,d], b1 [E,2f],
    w2 [E,d,f], b2 [E,d]; drawn in the order gate, then expert by expert."""
    g = torch.Generator().manual_seed(seed)
    gate_w = torch.randn(E, d, generator=g) * 0.02
    w1 = torch.empty(E, 2 * f, d)
    w2 = torch.empty(E, d, f)
    for e in range(E):
        w1[e] = torch.randn(2 * f, d, generator=g) * 0.02
        w2[e] = torch.randn(d, f, generator=g) * 0.02
    return {
        "gate_w": gate_w, "gate_b": gate_bias(gate_bias_kind, E),
        "w1": w1, "b1": torch.zeros(E, 2 * f), "w2": w2, "b2": torch.zeros(E, d),
    }


def make_input(N: int, d: int, seed: int = 1) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(N, d, generator=g)


def round_to(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Round to ``dtype`` and return fp32 holding exactly those values."""
    return t.to(dtype).to(torch.float32)


def load_into(module, params: dict, dtype: torch.dtype, device) -> None:
    """Copy a ``make_params`` dict into a ``MOE`` module (ours or the reference's)."""
    module.to(device=device, dtype=dtype)
    with torch.no_grad():
        module.gate.weight.copy_(params["gate_w"])
        module.gate.bias.copy_(params["gate_b"])
        for e, ex in enumerate(module.experts):
            ex.gate_and_up.weight.copy_(params["w1"][e])
            ex.gate_and_up.bias.copy_(params["b1"][e])
            ex.down.weight.copy_(params["w2"][e])
            ex.down.bias.copy_(params["b2"][e])


def make_gate(d: int, E: int, seed: int = 0, gate_bias_kind: str = "zero"):
    """gate_w [E,d], gate_b [E]: the first draws of ``make_params`` with the same seed."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(E, d, generator=g) * 0.02, gate_bias(gate_bias_kind, E)


def make_expert(d: int, f: int, e: int, seed: int = 0) -> dict:
    """One expert's fp32 parameters from its own generator (seed, e), so that a rank
    of the expert-parallel configuration draws only the experts it owns."""
    g = torch.Generator().manual_seed(1000003 * (seed + 1) + e)
    return {"w1": torch.randn(2 * f, d, generator=g) * 0.02, "b1": torch.zeros(2 * f),
            "w2": torch.randn(d, f, generator=g) * 0.02, "b2": torch.zeros(d)}
