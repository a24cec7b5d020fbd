"""CPU oracle for the Mixture-of-Experts block. TEST INFRASTRUCTURE ONLY.

A restatement, in fp32 PyTorch CPU ops, of the algorithm of the reference's
``MOE.forward`` (model.py:200-276) and ``FeedForward.forward``
(model.py:173-190, fine_tuning=False, eval mode), generalised from the
reference's hard-coded two slots to ``k`` slots and to a free expert width.
The reference's arithmetic lives in PyTorch ATen (``F.linear``, ``F.softmax``,
``topk``, ``F.gelu(approximate="tanh")``, ``index_copy_``); this file calls the
same operators in the same order, so at k = 2 it is bit-identical to the
reference class on the same thread count. The reference pins no torch
version (requirements.txt:1); torch 2.11.0 CPU is what it was checked on.

Parity pin: the reference's own tests never run its MoE block, so there are no
reference-held golden vectors. The pin is the importable reference class:
tests/golden/make_golden.py imports it, checks ``torch.equal`` against this
oracle, and writes the fixtures that tests/test_oracle.py replays.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
import this file. Nothing under gemmallm_b200/ does.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def expert_ffn(x, w1, b1, w2, b2, lora=None, h_mask=None):
    """One expert on rows ``x`` [n,d]: model.py:174 (gate_and_up), :180 (chunk),
    :181 (tanh GELU on the gate half), :182 (product), :184 (down).

    ``lora`` (the fine_tuning=True branch, model.py:175-179 and 185-189): dict with
    ``scale`` and the eight tensors ``gu_a_w, gu_a_b, gu_b_w, gu_b_b, dn_a_w, dn_a_b,
    dn_b_w, dn_b_b`` of this expert's four LoRA Linears.

    ``h_mask`` [n,f]: multiplier applied to h where the reference applies nn.Dropout in
    training mode (model.py:183): 0 for dropped elements, 1/(1-p) for kept ones."""
    gu = F.linear(x, w1, b1)
    if lora is not None:
        t = F.linear(x, lora["gu_a_w"], lora["gu_a_b"])
        t = F.linear(t, lora["gu_b_w"], lora["gu_b_b"])
        gu = gu + t * lora["scale"]
    gate, up = gu.chunk(2, dim=-1)
    h = F.gelu(gate, approximate="tanh") * up
    if h_mask is not None:
        h = h * h_mask
    y = F.linear(h, w2, b2)
    if lora is not None:
        t = F.linear(h, lora["dn_a_w"], lora["dn_a_b"])
        t = F.linear(t, lora["dn_b_w"], lora["dn_b_b"])
        y = y + t * lora["scale"]
    return y


def route_from_logits(logits: torch.Tensor, k: int):
    """softmax -> top-k -> renormalise -> per-slot counts -> loss, from given
    fp32 logits [N,E]: model.py:207 (softmax), :210 (topk), :213-216 (loss,
    first slot only), :219-223 (scores divided by their left-to-right sum),
    :237-245 (counts per slot)."""
    N, E = logits.shape
    probs = F.softmax(logits, dim=-1)
    vals, idx = probs.topk(k=k, dim=-1)
    counts0 = torch.bincount(idx[:, 0], minlength=E)
    freq = counts0.float() / N
    aux = (probs.mean(0) * freq).mean() * float(E ** 2)
    total = vals[:, 0]
    for j in range(1, k):
        total = total + vals[:, j]
    weights = torch.stack([vals[:, j] / total for j in range(k)], dim=1)
    cnt_slot = torch.stack([torch.bincount(idx[:, j], minlength=E) for j in range(k)])
    return {"probs": probs, "vals": vals, "idx": idx, "w": weights, "cnt_slot": cnt_slot,
            "aux": aux}


def tie_rows(probs: torch.Tensor, k: int) -> torch.Tensor:
    """Rows whose top-k choice or order is not determined by the values: two
    equal probabilities among the k+1 largest. torch.topk's order among equal
    values is unspecified, so such rows are excluded from index equality."""
    E = probs.shape[1]
    s, _ = probs.sort(dim=-1, descending=True)
    upto = min(k + 1, E)
    return (s[:, 1:upto] == s[:, : upto - 1]).any(dim=1)


def moe_forward(x: torch.Tensor, params: dict, k: int = 2, logits: torch.Tensor | None = None,
                lora: list | None = None, h_mask: torch.Tensor | None = None):
    """The whole block on x [N,d] (fp32, CPU). ``params`` as produced by
    gemmallm_b200.synthetic.make_params (fp32). With ``logits`` given, routing
    is derived from them instead of from x (used to impose the CUDA router's
    own logits, so that outputs are compared under identical routing). ``lora``: one
    dict per expert (see expert_ffn) for the fine_tuning=True forward. ``h_mask``
    [N,k,f]: the training-mode dropout multiplier of every (token, slot) pair's h row.

    Per slot, as model.py:226-268: sort token ids by chosen expert, run each
    non-empty expert on its rows, concatenate, scatter back with index_copy_
    into an fp32 zero buffer; then the weighted sum in slot order (model.py:271).
    """
    N, d = x.shape
    E = params["gate_w"].shape[0]
    if logits is None:
        logits = F.linear(x, params["gate_w"], params["gate_b"])
    r = route_from_logits(logits, k)
    final = None
    for j in range(k):
        chosen = r["idx"][:, j]
        order = chosen.argsort()
        counts = r["cnt_slot"][j].tolist()
        rows = x[order]
        pieces = torch.split(rows, counts, dim=0)
        masks = [None] * E if h_mask is None else torch.split(h_mask[order, j], counts, dim=0)
        outs = [expert_ffn(pieces[e], params["w1"][e], params["b1"][e], params["w2"][e],
                           params["b2"][e], None if lora is None else lora[e], masks[e])
                if counts[e] > 0 else torch.zeros(0, d)
                for e in range(E)]
        buf = torch.zeros(N, d, dtype=torch.float32)
        buf.index_copy_(0, order, torch.cat(outs, dim=0))
        term = r["w"][:, j].unsqueeze(-1) * buf
        final = term if final is None else final + term
    r["logits"] = logits
    r["out"] = final
    return r


def time_forward(x, params, k, repeats: int = 3, warmup: int = 1):
    """Median seconds of moe_forward on this host's cores (CPU baseline)."""
    import time
    with torch.no_grad():
        for _ in range(warmup):
            moe_forward(x, params, k)
        ts = []
        for _ in range(repeats):
            t0 = time.perf_counter()
            moe_forward(x, params, k)
            ts.append(time.perf_counter() - t0)
    ts.sort()
    return ts[len(ts) // 2]
