"""Thin test-side wrappers: call each C-ABI entry point with torch tensors."""
from __future__ import annotations

import torch

from gemmallm_b200 import _cabi, synthetic
from gemmallm_b200._cabi import lib, check

CODE = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16}


def stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def router(x, gate_w, gate_b, k):
    N, d = x.shape
    E = gate_w.shape[0]
    dev = x.device
    logits = torch.empty(N, E, dtype=torch.float32, device=dev)
    idx = torch.empty(N, k, dtype=torch.int32, device=dev)
    w = torch.empty(N, k, dtype=torch.float32, device=dev)
    psum_part = torch.empty(max(1, lib.moe_b200_router_blocks(N)), E, dtype=torch.float32, device=dev)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    check(lib.moe_b200_router(x.data_ptr(), gate_w.data_ptr(), gate_b.data_ptr(), N, d, E, k,
                              CODE[x.dtype], logits.data_ptr(), idx.data_ptr(), w.data_ptr(),
                              psum_part.data_ptr(), status.data_ptr(), stream(dev)), "router")
    return logits, idx, w, psum_part


def dispatch(x, idx, E, psum_part=None):
    N, d = x.shape
    k = idx.shape[1]
    dev = x.device
    nbytes = lib.moe_b200_dispatch_scratch_bytes(N, E, k)
    # poison the scratch: the kernel must not depend on its previous contents
    scratch = torch.full((nbytes // 4,), 0x5A5A5A5A, dtype=torch.int32, device=dev)
    cnt_slot = torch.empty(k, E, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    row_of = torch.empty(N, k, dtype=torch.int32, device=dev)
    perm = torch.empty(N * k, d, dtype=x.dtype, device=dev)
    psum = torch.empty(E, dtype=torch.float32, device=dev)
    aux = torch.zeros(1, dtype=torch.float32, device=dev)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    check(lib.moe_b200_dispatch(x.data_ptr(), idx.data_ptr(), N, d, E, k, CODE[x.dtype],
                                scratch.data_ptr(), cnt_slot.data_ptr(), offsets.data_ptr(),
                                row_of.data_ptr(), perm.data_ptr(),
                                None if psum_part is None else psum_part.data_ptr(),
                                psum.data_ptr(), aux.data_ptr(), status.data_ptr(), stream(dev)),
          "dispatch")
    return {"cnt_slot": cnt_slot, "offsets": offsets, "row_of": row_of, "perm": perm,
            "psum": psum, "aux": aux, "status": status}


class Plan:
    def __init__(self, w1, b1, w2, b2):
        """w1 [E,2f,d], b1 [E,2f], w2 [E,d,f], b2 [E,d] on the device."""
        E, f2, d = w1.shape
        self.E, self.d, self.f = E, d, f2 // 2
        dev = w1.device
        nbytes = lib.moe_b200_plan_bytes(E)
        self.buf = torch.empty(nbytes + 128, dtype=torch.uint8, device=dev)
        self.ptr = (self.buf.data_ptr() + 127) & ~127
        self.keep = (w1, b1, w2, b2)
        arr = lambda t: _cabi.ptr_array([t[e].data_ptr() for e in range(E)])
        check(lib.moe_b200_plan_build(arr(w1), arr(b1), arr(w2), arr(b2), E, d, self.f,
                                      CODE[w1.dtype], self.ptr, nbytes, stream(dev)), "plan_build")


def experts(perm, offsets, plan: Plan):
    M, d = perm.shape
    dev = perm.device
    h = torch.empty(M, plan.f, dtype=perm.dtype, device=dev)
    y = torch.empty(M, d, dtype=perm.dtype, device=dev)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    check(lib.moe_b200_experts(perm.data_ptr(), offsets.data_ptr(), plan.ptr, M, d, plan.f, plan.E,
                               CODE[perm.dtype], 0, h.data_ptr(), y.data_ptr(),
                               status.data_ptr(), stream(dev)), "experts")
    return h, y, status


def combine(y, row_of, w, residual=None):
    N, k = row_of.shape
    d = y.shape[1]
    out = torch.empty(N, d, dtype=y.dtype, device=y.device)
    check(lib.moe_b200_combine(y.data_ptr(), row_of.data_ptr(), w.data_ptr(),
                               None if residual is None else residual.data_ptr(), N, d, k,
                               CODE[y.dtype], out.data_ptr(), stream(y.device)), "combine")
    return out


def device_params(params: dict, dtype, dev) -> dict:
    return {n: t.to(dtype).to(dev).contiguous() for n, t in params.items()}


def rounded_params(params: dict, dtype) -> dict:
    return {n: synthetic.round_to(t, dtype) for n, t in params.items()}


def experts_rows(perm, offsets, plan: Plan, ksplit: int):
    M, d = perm.shape
    dev = perm.device
    h = torch.full((M, plan.f), float("nan"), dtype=perm.dtype, device=dev)
    part = torch.full((ksplit, M, d), float("nan"), dtype=torch.float32, device=dev)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    ready = torch.full((_cabi.READY_INTS,), 7, dtype=torch.int32, device=dev)
    check(lib.moe_b200_experts_rows(perm.data_ptr(), offsets.data_ptr(), plan.ptr, M, d, plan.f,
                                    plan.E, ksplit, h.data_ptr(), part.data_ptr(), ready.data_ptr(),
                                    status.data_ptr(), stream(dev)), "experts_rows")
    return h, part, status


def experts_decode_fused(perm, offsets, plan: Plan):
    M, d = perm.shape
    dev = perm.device
    splits = lib.moe_b200_decode_splits(plan.f)
    h = torch.empty(M, plan.f, dtype=perm.dtype, device=dev)
    part = torch.full((splits, M, d), float("nan"), dtype=torch.float32, device=dev)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    # stale counters on purpose: the entry point has to zero them
    ready = torch.full((_cabi.READY_INTS,), 7, dtype=torch.int32, device=dev)
    check(lib.moe_b200_experts_decode_fused(perm.data_ptr(), offsets.data_ptr(), plan.ptr, M, d,
                                            plan.f, plan.E, h.data_ptr(), part.data_ptr(),
                                            ready.data_ptr(), status.data_ptr(), stream(dev)),
          "experts_decode_fused")
    return h, part, status


def experts_gemv(perm, offsets, plan: Plan):
    M, d = perm.shape
    dev = perm.device
    splits = lib.moe_b200_decode_splits(plan.f)
    h = torch.full((M, plan.f), float("nan"), dtype=perm.dtype, device=dev)
    part = torch.full((splits, M, d), float("nan"), dtype=torch.float32, device=dev)
    check(lib.moe_b200_experts_gemv(perm.data_ptr(), offsets.data_ptr(), plan.ptr, M, d, plan.f, plan.E,
                                    h.data_ptr(), part.data_ptr(), stream(dev)), "experts_gemv")
    return h, part


def decode_tiny(x, gate_w, gate_b, plan: Plan, k: int, f: int, residual=None):
    """moe_b200_decode_tiny: the whole block for one to eight bf16 tokens in one launch."""
    N, d = x.shape
    E = gate_w.shape[0]
    dev = x.device
    i32 = dict(dtype=torch.int32, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    r = {"logits": torch.empty(N, E, **f32), "idx": torch.empty(N, k, **i32), "w": torch.empty(N, k, **f32),
         "cnt_slot": torch.empty(k, E, **i32), "offsets": torch.empty(E + 1, **i32),
         "row_of": torch.empty(N, k, **i32), "perm": torch.empty(N * k, d, dtype=x.dtype, device=dev),
         "psum": torch.empty(E, **f32), "aux": torch.empty(1, **f32),
         "h": torch.empty(N * k, f, dtype=x.dtype, device=dev), "out": torch.empty_like(x),
         "status": torch.zeros(16, **i32)}
    check(lib.moe_b200_decode_tiny(
        x.data_ptr(), gate_w.data_ptr(), gate_b.data_ptr(), plan.ptr,
        residual.data_ptr() if residual is not None else None, N, d, f, E, k,
        r["logits"].data_ptr(), r["idx"].data_ptr(), r["w"].data_ptr(), r["cnt_slot"].data_ptr(),
        r["offsets"].data_ptr(), r["row_of"].data_ptr(), r["perm"].data_ptr(), r["psum"].data_ptr(),
        r["aux"].data_ptr(), r["h"].data_ptr(), r["out"].data_ptr(), r["status"].data_ptr(), stream(dev)),
        "decode_tiny")
    return r


def experts_decode_spec(x, idx, offsets, plan: Plan):
    """x [N,d] unsorted tokens; returns part [splits, N*k, d] in dispatch row order."""
    N, d = x.shape
    k = idx.shape[1]
    dev = x.device
    splits = lib.moe_b200_decode_splits(plan.f)
    NP = lib.moe_b200_decode_spec_rows(N)
    # poisoned slabs: rows of tokens not routed to an expert are never written and must not matter
    h_all = torch.full((plan.E, NP, plan.f), float("nan"), dtype=x.dtype, device=dev)
    part = torch.full((splits, N * k, d), float("nan"), dtype=torch.float32, device=dev)
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    ready = torch.full((_cabi.READY_INTS,), 7, dtype=torch.int32, device=dev)
    check(lib.moe_b200_experts_decode_spec(x.data_ptr(), idx.data_ptr(), offsets.data_ptr(), plan.ptr,
                                           N, k, d, plan.f, plan.E, h_all.data_ptr(), part.data_ptr(),
                                           ready.data_ptr(), status.data_ptr(), stream(dev)),
          "experts_decode_spec")
    return h_all, part, status


def combine_decode(part, row_of, idx, w, plan: Plan, residual=None):
    splits, M, d = part.shape
    N, k = row_of.shape
    out = torch.empty(N, d, dtype=torch.bfloat16, device=part.device)
    check(lib.moe_b200_combine_decode(part.data_ptr(), splits, M, row_of.data_ptr(), idx.data_ptr(),
                                      w.data_ptr(), plan.ptr, plan.E,
                                      None if residual is None else residual.data_ptr(), N, d, k,
                                      out.data_ptr(), stream(part.device)), "combine_decode")
    return out
