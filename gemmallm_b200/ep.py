"""Expert-parallel Mixture-of-Experts block: tokens sharded over the ranks of a
process group (one process per GPU), experts owned by ranks, dispatch and
combine as peer-store all-to-all inside the kernels (libmoe_b200's
moe_b200_ep_forward). The reference has no multi-GPU path; this extends
MOE.forward (model.py:200-276) to that sharding with the same parameter names:
``gate`` is replicated, ``experts`` holds only the owned experts under their
global ids (``experts.{e}.gate_and_up.weight`` ...), so a full checkpoint loads
with ``strict=False``.

torch.distributed is used for rendezvous and for allocating the peer-mapped
("symmetric") buffer; no collective runs on the data path.
"""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.nn as nn

from . import _cabi
from ._cabi import lib, check
from .moe import FeedForward, _MergedLora, _Plan, _dtype_code, _stream


def strided_placement(num_experts: int, world: int) -> list[int]:
    """Owner of each expert: e mod world. Keeps neighbouring (similarly popular,
    under a Zipf-like router bias) experts on different ranks."""
    return [e % world for e in range(num_experts)]


def lpt_placement(load: list[float], world: int) -> list[int]:
    """Greedy longest-processing-time placement with equal expert counts per
    rank: heaviest expert first onto the least-loaded rank that still has room."""
    E = len(load)
    room = [E // world + (1 if r < E % world else 0) for r in range(world)]
    total = [0.0] * world
    owner = [0] * E
    for e in sorted(range(E), key=lambda i: (-load[i], i)):
        r = min((r for r in range(world) if room[r] > 0), key=lambda r: (total[r], r))
        owner[e] = r
        room[r] -= 1
        total[r] += load[e]
    return owner


def virtual_experts(owner: list[int], replicate: dict[int, list[int]], world: int):
    """Virtual expert table. ``owner[e]`` places every real expert; ``replicate[e]``
    lists the ranks that hold a copy of expert e (its owner is added if missing).
    Returns (v_owner, v_real, vmap): rank and real expert of every virtual id, and
    vmap[e][r] = the virtual expert rank r sends its rows for e to — the copy on r
    itself when there is one (those rows never leave the GPU), else the copies in
    turn by source rank."""
    E = len(owner)
    v_owner, v_real = list(owner), list(range(E))
    vmap = [[e] * world for e in range(E)]
    for e in sorted(replicate):
        ranks = sorted(set(replicate[e]) | {owner[e]})
        ids = {owner[e]: e}
        for r in ranks:
            if r != owner[e]:
                ids[r] = len(v_owner)
                v_owner.append(r)
                v_real.append(e)
        others = [r for r in range(world) if r not in ids]
        for r in ids:
            vmap[e][r] = ids[r]
        for i, r in enumerate(others):
            vmap[e][r] = ids[ranks[i % len(ranks)]]
    return v_owner, v_real, vmap


class ExpertParallelMOE(nn.Module):
    """``placement[e]``: owner rank of expert e (default strided). ``replicate``:
    {expert: [ranks]} extra copies of popular experts; a list of expert ids means
    "on every rank". Replicas are ordinary entries of ``experts`` under the same
    global id, so checkpoints load the same way."""

    def __init__(self, hidden_size: int, num_experts: int = 8, expansion_factor: int = 4,
                 dropout_ratio: float = 0.1, lora_rank: int = 16, lora_alpha: int = 32,
                 device: str = "mps", *, top_k: int = 2, d_ff: int | None = None, group=None,
                 placement: list[int] | None = None, replicate=None):
        super().__init__()
        import torch.distributed as dist
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.owner = list(placement) if placement is not None else strided_placement(num_experts, self.world)
        if len(self.owner) != num_experts or any(not 0 <= o < self.world for o in self.owner):
            raise ValueError("placement must give a rank in [0, world) for every expert")
        if replicate is None:
            replicate = {}
        elif not isinstance(replicate, dict):
            replicate = {int(e): list(range(self.world)) for e in replicate}
        self.v_owner, self.v_real, self.vmap = virtual_experts(self.owner, replicate, self.world)
        if len(self.v_owner) > 256:
            raise ValueError("too many expert copies (at most 256 virtual experts)")
        self.gate = nn.Linear(hidden_size, num_experts)
        self.num_experts = num_experts
        # virtual experts this rank runs, in increasing virtual id, and their real experts
        self.local_virtual = [v for v, o in enumerate(self.v_owner) if o == self.rank]
        self.local_ids = [self.v_real[v] for v in self.local_virtual]
        self.experts = nn.ModuleDict({
            str(e): FeedForward(hidden_size, expansion_factor=expansion_factor,
                                dropout_ratio=dropout_ratio, lora_rank=lora_rank,
                                lora_alpha=lora_alpha, d_ff=d_ff) for e in sorted(set(self.local_ids))})
        self.device = device
        self.hidden_size = hidden_size
        self.d_ff = hidden_size * expansion_factor if d_ff is None else d_ff
        self.top_k = top_k
        self._plan = _Plan()
        self._plan_ft = _Plan()
        self._lora = _MergedLora()
        self._state = None
        self._stage_events = None    # ctypes array of cudaEvent_t, see time_stages()
        self.last = None

    def _setup(self, N_local: int, dev: torch.device):
        key = (N_local, str(dev))
        if self._state is not None and self._state["key"] == key:
            return self._state
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only
        import torch.distributed._symmetric_memory as symm_mem
        d, f, E, k, G = self.hidden_size, self.d_ff, self.num_experts, self.top_k, self.world
        sizes = [None] * G
        dist.all_gather_object(sizes, N_local, group=self.group)
        if any(s != N_local for s in sizes):
            raise ValueError(f"every rank must pass the same number of tokens, got {sizes}")
        nbytes = lib.moe_b200_ep_symm_bytes(N_local, d, E, k, G)
        if nbytes == 0:
            raise _cabi.MoeB200Error(lib.moe_b200_last_error_string().decode())
        symm = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        hdl = symm_mem.rendezvous(symm, group=self.group)
        symm.zero_()
        torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)
        bases = [int(p) for p in hdl.buffer_ptrs]
        wbytes = lib.moe_b200_ep_workspace_bytes(N_local, d, f, E, k, G)
        ws = torch.zeros(wbytes + 1024, dtype=torch.uint8, device=dev)
        ws_base = (ws.data_ptr() + 1023) & ~1023
        owner = (C.c_int32 * len(self.v_owner))(*self.v_owner)
        vmap = (C.c_int32 * (E * G))(*[v for row in self.vmap for v in row])
        # the placement tables live in the workspace: uploaded here, once per workspace
        check(lib.moe_b200_ep_setup(owner, vmap, N_local, d, f, E, k, G, len(self.v_owner), ws_base,
                                    wbytes, _stream(dev)), "ep_setup")
        self._state = {
            "key": key, "symm": symm, "hdl": hdl, "bases": (C.c_void_p * G)(*bases),
            "ws": ws, "ws_base": ws_base, "ws_bytes": wbytes,
            "ws_layout": _cabi.ep_workspace_layout(N_local, d, f, E, k, G),
            "symm_layout": _cabi.ep_symm_layout(N_local, d, E, k, G),
        }
        return self._state

    def _ws_view(self, name, dtype, shape):
        st = self._state
        start = st["ws_base"] - st["ws"].data_ptr() + st["ws_layout"][name]
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty(0, dtype=dtype).element_size()
        return st["ws"][start:start + nb].view(dtype).view(*shape)

    def forward(self, tensor: torch.Tensor, fine_tuning: bool = False, *,
                residual: torch.Tensor | None = None):
        """Local tokens [B,S,d] (bf16, same count on every rank) ->
        ([B,S,d], load-balancing loss over the tokens of all ranks). ``fine_tuning=True``
        runs the owned experts with their LoRA branches folded in, as ``MOE.forward`` does."""
        if self.training and len(self.experts) and next(iter(self.experts.values())).dropout.p > 0:
            raise NotImplementedError("dropout in training mode is not implemented; call .eval()")
        if not tensor.is_cuda:
            raise RuntimeError("libmoe_b200 runs on CUDA tensors only; there is no CPU path")
        dtype = _dtype_code(tensor)
        shape = tensor.shape
        d, f, E, k = self.hidden_size, self.d_ff, self.num_experts, self.top_k
        x = tensor.reshape(-1, d).contiguous()
        N = x.shape[0]
        dev = x.device
        res_ptr = None
        if residual is not None:
            residual = residual.reshape(-1, d).contiguous()
            res_ptr = residual.data_ptr()
        out = torch.empty_like(x)
        with torch.cuda.device(dev):
            st = self._setup(N, dev)
            local = [self.experts[str(e)] for e in self.local_ids]
            if not local:
                plan = None
            elif fine_tuning:
                # LoRA branches (model.py:175-179,185-189) folded into merged copies of the owned experts
                uniq = sorted(set(self.local_ids))
                merged = dict(zip(uniq, self._lora.get([self.experts[str(e)] for e in uniq], dtype, dev)))
                plan = self._plan_ft.get([merged[e] for e in self.local_ids], d, f, dtype, dev)
            else:
                plan = self._plan.get(local, d, f, dtype, dev)
            check(lib.moe_b200_ep_forward(
                x.data_ptr(), self.gate.weight.data_ptr(), self.gate.bias.data_ptr(), plan, res_ptr,
                N, d, f, E, k, dtype, 0, self.rank, self.world, len(self.v_owner),
                len(self.local_virtual), st["bases"],
                st["ws_base"], st["ws_bytes"], out.data_ptr(), self._stage_events, _stream(dev)),
                "ep_forward")
        self.last = {
            "logits": self._ws_view("logits", torch.float32, (N, E)),
            "idx": self._ws_view("idx", torch.int32, (N, k)),
            "w": self._ws_view("w", torch.float32, (N, k)),
            "cnt_slot0": self._ws_view("cnt_slot0", torch.int32, (E,)),
            "psum": self._ws_view("psum", torch.float32, (E,)),
            "offsets_local": self._ws_view("offsets_local", torch.int32, (len(self.local_ids) + 1,)),
            "status": self._ws_view("status", torch.int32, (16,)),
        }
        aux = self._ws_view("aux", torch.float32, (1,))[0].clone()
        return out.reshape(shape), aux

    def forward_nccl(self, tensor: torch.Tensor, *, residual: torch.Tensor | None = None):
        """The same sharded forward with the two exchange steps done by NCCL
        (``all_to_all_single`` with split sizes read back to the host) instead of peer stores
        inside the kernels: the baseline the in-kernel exchange is timed against. Router, expert
        and combine kernels are the library's; the permutations around the collectives are plain
        torch index operations, as a host-side implementation would write them."""
        import torch.distributed as dist
        dtype = _dtype_code(tensor)
        shape = tensor.shape
        d, f, E, k, G = self.hidden_size, self.d_ff, self.num_experts, self.top_k, self.world
        x = tensor.reshape(-1, d).contiguous()
        N = x.shape[0]
        dev = x.device
        EV = len(self.v_owner)
        with torch.cuda.device(dev):
            s = _stream(dev)
            logits = torch.empty(N, E, dtype=torch.float32, device=dev)
            idx = torch.empty(N, k, dtype=torch.int32, device=dev)
            w = torch.empty(N, k, dtype=torch.float32, device=dev)
            psum_part = torch.empty(max(1, lib.moe_b200_router_blocks(N)), E, dtype=torch.float32, device=dev)
            status = torch.zeros(16, dtype=torch.int32, device=dev)
            check(lib.moe_b200_router(x.data_ptr(), self.gate.weight.data_ptr(), self.gate.bias.data_ptr(),
                                      N, d, E, k, dtype, logits.data_ptr(), idx.data_ptr(), w.data_ptr(),
                                      psum_part.data_ptr(), status.data_ptr(), s), "router")
            if getattr(self, "_nccl_tables", None) is None or self._nccl_tables[0].device != dev:
                vmap_r = torch.tensor([self.vmap[e][self.rank] for e in range(E)], device=dev)
                v_owner = torch.tensor(self.v_owner, device=dev)
                # position of a virtual expert in the send order: by owner, then by virtual id
                order = sorted(range(EV), key=lambda v: (self.v_owner[v], v))
                vpos = torch.empty(EV, dtype=torch.long)
                vpos[torch.tensor(order)] = torch.arange(EV)
                self._nccl_tables = (vmap_r, v_owner, vpos.to(dev), torch.tensor(order, device=dev))
            vmap_r, v_owner, vpos, order = self._nccl_tables
            v_pair = vmap_r[idx.long().view(-1)]                      # [N*k] virtual expert of each pair
            key = vpos[v_pair]
            sort = torch.argsort(key, stable=True)                    # pairs in send order
            cnt = torch.bincount(key, minlength=EV)                   # per virtual expert, in send order
            cnt_all = torch.empty(G, EV, dtype=cnt.dtype, device=dev)
            dist.all_gather_into_tensor(cnt_all, cnt, group=self.group)
            owner_sorted = v_owner[order]                             # owner of each send-order slot
            mine = (owner_sorted == self.rank)
            send_splits = torch.zeros(G, dtype=cnt.dtype, device=dev).index_add_(0, owner_sorted, cnt).tolist()
            recv_cnt = cnt_all[:, mine]                               # [G, E_local] rows from each source
            recv_splits = recv_cnt.sum(1).tolist()
            rows = int(sum(recv_splits))
            send = x[(sort // k)]
            recv = torch.empty(rows, d, dtype=x.dtype, device=dev)
            dist.all_to_all_single(recv, send, recv_splits, send_splits, group=self.group)
            # received order is (source, expert); the grouped kernels want (expert, source)
            E_local = recv_cnt.shape[1]
            start_se = torch.cumsum(recv_cnt.reshape(-1), 0) - recv_cnt.reshape(-1)     # [G*E_local]
            cnt_es = recv_cnt.t().contiguous()                        # [E_local, G]
            start_es = (torch.cumsum(cnt_es.reshape(-1), 0) - cnt_es.reshape(-1)).view(E_local, G)
            seg_src = start_se.view(G, E_local).t()                   # [E_local, G]
            rep = cnt_es.reshape(-1)
            src_start = torch.repeat_interleave(seg_src.reshape(-1), rep, output_size=rows)
            dst_start = torch.repeat_interleave(start_es.reshape(-1), rep, output_size=rows)
            gather = src_start + (torch.arange(rows, device=dev) - dst_start)          # row r of (expert, source) order
            xs = recv[gather]
            offsets = torch.zeros(E_local + 1, dtype=torch.int32, device=dev)
            offsets[1:] = torch.cumsum(cnt_es.sum(1), 0).to(torch.int32)
            h = torch.empty(max(rows, 1), f, dtype=x.dtype, device=dev)
            y = torch.empty(max(rows, 1), d, dtype=x.dtype, device=dev)
            if rows > 0 and E_local > 0:
                local = [self.experts[str(e)] for e in self.local_ids]
                plan = self._plan.get(local, d, f, dtype, dev)
                check(lib.moe_b200_experts(xs.data_ptr(), offsets.data_ptr(), plan, rows, d, f, E_local,
                                           dtype, 0, h.data_ptr(), y.data_ptr(), status.data_ptr(), s),
                      "experts")
            back = torch.empty(rows, d, dtype=x.dtype, device=dev)
            back[gather] = y[:rows]
            ret = torch.empty(N * k, d, dtype=x.dtype, device=dev)
            dist.all_to_all_single(ret, back, send_splits, recv_splits, group=self.group)
            row_of = torch.empty(N * k, dtype=torch.int32, device=dev)
            row_of[sort] = torch.arange(N * k, dtype=torch.int32, device=dev)
            out = torch.empty_like(x)
            res_ptr = None if residual is None else residual.reshape(-1, d).contiguous().data_ptr()
            check(lib.moe_b200_combine(ret.data_ptr(), row_of.data_ptr(), w.data_ptr(), res_ptr, N, d, k,
                                       dtype, out.data_ptr(), s), "combine")
        return out.reshape(shape)

    def time_stages(self, tensor: torch.Tensor, reps: int = 10) -> dict:
        """CUDA-event time (ms, mean over ``reps`` calls) of each stage of the sharded forward on
        this rank: the library records an event at every stage boundary of the call. The waits
        on peers sit at the head of the stage that needs the data ("experts" waits for the rows,
        "combine" for the outputs), so a rank that is ahead of its peers shows its lead there.
        All ranks must call this together."""
        n = len(_cabi.EP_STAGES) + 1
        sets = []
        for _ in range(reps):
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
            for e in evs:
                e.record()          # creates the underlying cudaEvent_t
            sets.append(evs)
        torch.cuda.synchronize(tensor.device)
        with torch.no_grad():
            for evs in sets:
                self._stage_events = (C.c_void_p * n)(*[e.cuda_event for e in evs])
                try:
                    self.forward(tensor)
                finally:
                    self._stage_events = None
        torch.cuda.synchronize(tensor.device)
        out = {}
        for i, name in enumerate(_cabi.EP_STAGES):
            out[name] = sum(evs[i].elapsed_time(evs[i + 1]) for evs in sets) / reps
        return out

    def device_status(self) -> int:
        return int(self.last["status"][0].item()) if self.last else 0
