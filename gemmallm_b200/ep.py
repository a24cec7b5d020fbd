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
from .moe import FeedForward, _Plan, _dtype_code, _stream


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
        self.epoch = 0
        self.flags = _cabi.FLAG_DEFAULT
        self._plan = _Plan()
        self._state = None
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
        ws = torch.empty(wbytes + 1024, dtype=torch.uint8, device=dev)
        self.epoch = 0
        self._state = {
            "key": key, "symm": symm, "hdl": hdl, "bases": (C.c_void_p * G)(*bases),
            "ws": ws, "ws_base": (ws.data_ptr() + 1023) & ~1023, "ws_bytes": wbytes,
            "ws_layout": _cabi.ep_workspace_layout(N_local, d, f, E, k, G),
            "symm_layout": _cabi.ep_symm_layout(N_local, d, E, k, G),
            "owner": (C.c_int32 * len(self.v_owner))(*self.v_owner),
            "vmap": (C.c_int32 * (E * G))(*[v for row in self.vmap for v in row]),
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
        ([B,S,d], load-balancing loss over the tokens of all ranks)."""
        if fine_tuning:
            raise NotImplementedError("the LoRA branch (fine_tuning=True) is not implemented")
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
            plan = self._plan.get(local, d, f, dtype, dev) if local else None
            self.epoch += 1
            check(lib.moe_b200_ep_forward(
                x.data_ptr(), self.gate.weight.data_ptr(), self.gate.bias.data_ptr(), plan, res_ptr,
                N, d, f, E, k, dtype, self.flags, self.rank, self.world, self.epoch, len(self.v_owner),
                st["owner"], st["vmap"], st["bases"],
                st["ws_base"], st["ws_bytes"], out.data_ptr(), _stream(dev)), "ep_forward")
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

    def device_status(self) -> int:
        return int(self.last["status"][0].item()) if self.last else 0
