"""Host-side logic of the expert-parallel path on CPU: placement functions, and
the exchange protocol itself simulated over the gloo backend with two ranks
(counts all-gather, destination rows ordered by owned expert, source rank,
token; rows out, expert outputs back, combine), which must reproduce the
single-process oracle."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gemmallm_b200 import synthetic
from gemmallm_b200.ep import lpt_placement, strided_placement, virtual_experts
from oracle import moe_oracle


def test_placements():
    assert strided_placement(8, 4) == [0, 1, 2, 3, 0, 1, 2, 3]
    load = [1.0 / (e + 1) ** 1.1 for e in range(64)]
    owner = lpt_placement(load, 8)
    assert sorted(owner.count(r) for r in range(8)) == [8] * 8          # sharded evenly
    per_rank = [sum(l for l, o in zip(load, owner) if o == r) for r in range(8)]
    strided = [sum(l for e, l in enumerate(load) if e % 8 == r) for r in range(8)]
    assert max(per_rank) <= max(strided) + 1e-12                         # never worse than strided
    assert max(per_rank) >= load[0]                                      # the hottest expert bounds it


def test_virtual_experts():
    v_owner, v_real, vmap = virtual_experts([0, 1, 0, 1], {}, 2)
    assert v_owner == [0, 1, 0, 1] and v_real == [0, 1, 2, 3] and vmap == [[e, e] for e in range(4)]
    # expert 0 copied to both ranks: each rank keeps its own rows of expert 0
    v_owner, v_real, vmap = virtual_experts([0, 1, 0, 1], {0: [0, 1]}, 2)
    assert v_owner == [0, 1, 0, 1, 1] and v_real == [0, 1, 2, 3, 0]
    assert vmap[0] == [0, 4] and vmap[1] == [1, 1]
    # a partial copy set: holders use their own copy, the other ranks alternate
    v_owner, v_real, vmap = virtual_experts([0, 1, 2, 3, 0, 1, 2, 3], {1: [1, 3]}, 4)
    assert v_owner[8] == 3 and v_real[8] == 1
    assert vmap[1][1] == 1 and vmap[1][3] == 8 and sorted([vmap[1][0], vmap[1][2]]) == [1, 8]
    for e in range(8):
        assert all(v_real[v] == e for v in vmap[e])


def dest_rows(cnt_all, owner, rank):
    """First row, in its owner's receive buffer, of the pairs (source `rank`,
    expert e): experts of one owner in increasing id, inside an expert sources
    in increasing rank. The rule the dispatch kernel implements."""
    G, E = cnt_all.shape
    total = cnt_all.sum(0)
    base = torch.zeros(E, dtype=torch.long)
    for e in range(E):
        b = sum(int(total[e2]) for e2 in range(e) if owner[e2] == owner[e])
        b += int(cnt_all[:rank, e].sum())
        base[e] = b
    return base


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    N, d, f, E, k = 96, 32, 48, 8, 2
    params = synthetic.make_params(d, E, f, seed=3, gate_bias_kind="zipf1.1")
    x_all = synthetic.make_input(N, d, seed=4)
    owner = strided_placement(E, world)
    Nl = N // world
    x = x_all[rank * Nl:(rank + 1) * Nl]
    with torch.no_grad():
        r = moe_oracle.route_from_logits(torch.nn.functional.linear(x, params["gate_w"], params["gate_b"]), k)
        cnt = r["cnt_slot"].sum(0)
        rows = [torch.zeros(E, dtype=torch.long) for _ in range(world)]
        dist.all_gather(rows, cnt)
        cnt_all = torch.stack(rows)
        base = dest_rows(cnt_all, owner, rank)
        # stable rank of each pair inside (this source, expert), in (token, slot) order
        pairs_e = r["idx"].flatten()
        seen = torch.zeros(E, dtype=torch.long)
        dest = torch.empty(Nl * k, dtype=torch.long)
        for p, e in enumerate(pairs_e.tolist()):
            dest[p] = base[e] + seen[e]
            seen[e] += 1
        # rows out: one message per destination (stands in for the peer stores)
        send = [[] for _ in range(world)]
        for p, e in enumerate(pairs_e.tolist()):
            send[owner[e]].append((int(dest[p]), rank, p, x[p // k]))
        gathered = [None] * world
        dist.all_gather_object(gathered, send)
        mine = sorted((m for src in gathered for m in src[rank]), key=lambda m: m[0])
        assert [m[0] for m in mine] == list(range(len(mine)))            # receive buffer is dense
        recv = torch.stack([m[3] for m in mine]) if mine else torch.zeros(0, d)
        local_ids = [e for e in range(E) if owner[e] == rank]
        total = cnt_all.sum(0)
        offs = torch.tensor([0] + [int(total[e]) for e in local_ids]).cumsum(0)
        ys = [moe_oracle.expert_ffn(recv[offs[i]:offs[i + 1]], params["w1"][e], params["b1"][e],
                                    params["w2"][e], params["b2"][e]) for i, e in enumerate(local_ids)]
        y = torch.cat(ys) if ys else torch.zeros(0, d)
        back = [[] for _ in range(world)]
        for i, m in enumerate(mine):
            back[m[1]].append((m[2], y[i]))
        gathered = [None] * world
        dist.all_gather_object(gathered, back)
        ret = torch.zeros(Nl * k, d)
        for src in gathered:
            for p, row in src[rank]:
                ret[p] = row
        out = (r["w"].unsqueeze(-1) * ret.view(Nl, k, d)).sum(1)
        ref = moe_oracle.moe_forward(x_all, params, k)["out"][rank * Nl:(rank + 1) * Nl]
    ok = torch.allclose(out, ref, atol=1e-5)
    out_q.put((rank, bool(ok), float((out - ref).abs().max())))
    dist.barrier()
    dist.destroy_process_group()


def test_exchange_protocol_over_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29581, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results), results
