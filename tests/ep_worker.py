"""Worker of the expert-parallel GPU test; launched with torch.distributed.run,
one process per GPU. Each rank owns a slice of the tokens and some of the
experts, runs ExpertParallelMOE twice (the second call reuses every buffer) and
checks its slice against the CPU oracle under the kernel's own routing."""
import argparse
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from gemmallm_b200 import synthetic  # noqa: E402
from gemmallm_b200.ep import ExpertParallelMOE, lpt_placement  # noqa: E402
from oracle import moe_oracle  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)   # total over all ranks
    ap.add_argument("--dmodel", type=int, default=256)
    ap.add_argument("--dff", type=int, default=384)
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--topk", type=int, default=4)
    ap.add_argument("--bias", default="zipf1.1")
    ap.add_argument("--placement", default="strided")
    ap.add_argument("--replicate", type=int, default=0, help="copy the N most popular experts to every rank")
    ap.add_argument("--lora", action="store_true", help="fine_tuning=True with random LoRA tensors")
    ap.add_argument("--check-tokens", type=int, default=0,
                    help="compare only the first N tokens of every rank with the oracle (0 = all)")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    N, d, f, E, k = args.tokens, args.dmodel, args.dff, args.experts, args.topk
    assert N % world == 0
    Nl = N // world
    dt = torch.bfloat16
    params = {n: synthetic.round_to(t, dt) for n, t in synthetic.make_params(
        d, E, f, seed=0, gate_bias_kind=args.bias).items()}
    params["w1"] *= 2.0
    g = torch.Generator().manual_seed(5)
    params["b1"] = synthetic.round_to(torch.randn(E, 2 * f, generator=g) * 0.05, dt)
    params["b2"] = synthetic.round_to(torch.randn(E, d, generator=g) * 0.05, dt)
    x_all = synthetic.round_to(synthetic.make_input(N, d, seed=1), dt)
    res_all = synthetic.round_to(synthetic.make_input(N, d, seed=2), dt)
    x = x_all[rank * Nl:(rank + 1) * Nl]
    res = res_all[rank * Nl:(rank + 1) * Nl]
    placement = None
    if args.placement == "lpt":
        placement = lpt_placement([1.0 / (e + 1) ** 1.1 for e in range(E)], world)
    replicate = list(range(args.replicate)) if args.replicate else None   # Zipf bias: lowest ids are hottest
    m = ExpertParallelMOE(d, num_experts=E, d_ff=f, top_k=k, device="cuda", placement=placement,
                          replicate=replicate).eval()
    m.to(device=dev, dtype=dt)
    with torch.no_grad():
        m.gate.weight.copy_(params["gate_w"])
        m.gate.bias.copy_(params["gate_b"])
        for e in sorted(set(m.local_ids)):
            ex = m.experts[str(e)]
            ex.gate_and_up.weight.copy_(params["w1"][e])
            ex.gate_and_up.bias.copy_(params["b1"][e])
            ex.down.weight.copy_(params["w2"][e])
            ex.down.bias.copy_(params["b2"][e])
    lora = None
    if args.lora:
        # every expert's LoRA tensors from its own seed, so that the oracle (all experts) and the
        # ranks (their own experts) agree
        lora = []
        for e in range(E):
            ge = torch.Generator().manual_seed(900 + e)
            rnd = lambda *shape: synthetic.round_to(torch.randn(*shape, generator=ge) * 0.05, dt)
            lora.append({"scale": 2.0, "gu_a_w": rnd(16, d), "gu_a_b": rnd(16), "gu_b_w": rnd(2 * f, 16),
                         "gu_b_b": rnd(2 * f), "dn_a_w": rnd(16, f), "dn_a_b": rnd(16),
                         "dn_b_w": rnd(d, 16), "dn_b_b": rnd(d)})
        with torch.no_grad():
            for e in sorted(set(m.local_ids)):
                ex, l = m.experts[str(e)], lora[e]
                assert ex.lora_scale == l["scale"]
                ex.lora_gate_and_up_a.weight.copy_(l["gu_a_w"]); ex.lora_gate_and_up_a.bias.copy_(l["gu_a_b"])
                ex.lora_gate_and_up_b.weight.copy_(l["gu_b_w"]); ex.lora_gate_and_up_b.bias.copy_(l["gu_b_b"])
                ex.lora_down_a.weight.copy_(l["dn_a_w"]); ex.lora_down_a.bias.copy_(l["dn_a_b"])
                ex.lora_down_b.weight.copy_(l["dn_b_w"]); ex.lora_down_b.bias.copy_(l["dn_b_b"])
    xd = x.to(dt).to(dev).view(1, Nl, d)
    rd = res.to(dt).to(dev).view(1, Nl, d)
    ok = True
    for call, residual in enumerate((None, rd, None)):
        with torch.no_grad():
            out, aux = m(xd, fine_tuning=args.lora, residual=residual)
        torch.cuda.synchronize()
        status = m.device_status()
        logits = m.last["logits"].clone()
        gathered = [torch.empty_like(logits) for _ in range(world)]
        dist.all_gather(gathered, logits)
        logits_all = torch.cat(gathered).cpu()
        c = min(args.check_tokens, Nl) if args.check_tokens else Nl    # tokens are independent
        with torch.no_grad():
            o = moe_oracle.moe_forward(x[:c], params, k, logits=logits.cpu()[:c], lora=lora)
            r_all = moe_oracle.route_from_logits(logits_all, k)
            r_own = moe_oracle.route_from_logits(logits.cpu(), k)
        ref = o["out"] if residual is None else o["out"] + res[:c]
        got = out.view(Nl, d).float().cpu()[:c]
        ties = moe_oracle.tie_rows(o["probs"], k)
        good = ~ties
        err = float((got - ref)[good].abs().max())
        bound = 2e-2 * float(ref.abs().max())
        good_all = ~moe_oracle.tie_rows(r_own["probs"], k)
        idx_ok = torch.equal(m.last["idx"].cpu()[good_all].long(), r_own["idx"][good_all])
        aux_ok = abs(float(aux) - float(r_all["aux"])) <= 1e-5 * abs(float(r_all["aux"])) + 1e-7
        cnt0_ok = torch.equal(m.last["cnt_slot0"].cpu().long(), r_all["cnt_slot"][0])
        # rows received per owned expert = global count of that expert
        total = r_all["cnt_slot"].sum(0)
        recv = m.last["offsets_local"].cpu().long().diff()
        if args.replicate:
            # copies split an expert's rows; over all ranks every pair is received exactly once
            got_rows = torch.tensor([int(recv.sum())], device=dev)
            dist.all_reduce(got_rows)
            recv_ok = int(got_rows) == N * k
        else:
            recv_ok = torch.equal(recv, total[m.local_ids]) if not moe_oracle.tie_rows(r_all["probs"], k).any() else True
        this = status == 0 and idx_ok and aux_ok and cnt0_ok and recv_ok and err <= bound
        print(f"rank {rank} call {call}: status {status} idx {idx_ok} aux {aux_ok} cnt0 {cnt0_ok} "
              f"recv {recv_ok} max-abs {err:.4g} (bound {bound:.4g}) -> {'ok' if this else 'FAIL'}", flush=True)
        ok = ok and this
        if call == 2 and not args.lora:
            # the NCCL all-to-all baseline computes the same block
            with torch.no_grad():
                out_n = m.forward_nccl(xd)
            torch.cuda.synchronize()
            err_n = float((out_n.view(Nl, d).float().cpu()[:c] - ref)[good].abs().max())
            print(f"rank {rank} nccl baseline: max-abs {err_n:.4g} (bound {bound:.4g})", flush=True)
            ok = ok and err_n <= bound
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    if int(flag) != 1:
        sys.exit(1)
    print(f"EP_OK rank {rank}", flush=True)


if __name__ == "__main__":
    main()
