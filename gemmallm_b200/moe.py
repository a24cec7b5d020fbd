"""Drop-in modules for GemmaLLM's Mixture-of-Experts block.

``MOE`` and ``FeedForward`` keep the constructor, attribute names, parameter
names/shapes and ``state_dict`` layout of the reference classes
(model.py:192-198 and model.py:154-171), so
``new.load_state_dict(ref.state_dict(), strict=True)`` works in both
directions. ``forward`` runs the hand-written sm_100a kernels of
libmoe_b200.so through its C ABI: this module only hands over device pointers,
sizes and the current CUDA stream. There is no CPU or eager-PyTorch path.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _cabi
from ._cabi import lib, check

_DTYPES = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"libmoe_b200 computes in float32 or bfloat16, got {t.dtype}") from None


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_LORA_NAMES = ("gate_and_up", "down", "lora_gate_and_up_a", "lora_gate_and_up_b", "lora_down_a",
               "lora_down_b")


class _MergedExpert:
    """An expert's two Linears with the LoRA branch folded in (moe_b200_lora_merge):
    W' = W + s * B A and b' = b + s * (B a + b_lora), which makes
    x W'^T + b' = x W^T + b + s * (B (A x + a) + b_lora), the fine_tuning=True
    expression of model.py:175-179 and 185-189. Has the attribute shape _Plan expects
    (gate_and_up/down with .weight/.bias); the buffers are written in place on every
    refresh, so a plan built on them stays valid."""

    class _Lin:
        def __init__(self, w, b):
            self.weight, self.bias = w, b

    def __init__(self, ex):
        self.gate_and_up = self._Lin(torch.empty_like(ex.gate_and_up.weight), torch.empty_like(ex.gate_and_up.bias))
        self.down = self._Lin(torch.empty_like(ex.down.weight), torch.empty_like(ex.down.bias))

    def refresh(self, ex, dtype: int, stream: int) -> None:
        for lin, a, b, out in ((ex.gate_and_up, ex.lora_gate_and_up_a, ex.lora_gate_and_up_b, self.gate_and_up),
                               (ex.down, ex.lora_down_a, ex.lora_down_b, self.down)):
            check(lib.moe_b200_lora_merge(
                lin.weight.data_ptr(), lin.bias.data_ptr(), a.weight.data_ptr(), a.bias.data_ptr(),
                b.weight.data_ptr(), b.bias.data_ptr(), float(ex.lora_scale), lin.out_features,
                lin.in_features, a.out_features, dtype, out.weight.data_ptr(), out.bias.data_ptr(),
                stream), "lora_merge")


class _MergedLora:
    """Merged copies of a list of experts, refreshed only when one of their twelve tensors
    was replaced or written since the last call (data pointer and torch's version counter),
    so that a fine_tuning=True forward on unchanged parameters launches no merge kernel and
    rebuilds no plan."""

    def __init__(self):
        self.key = None
        self.merged = None

    def get(self, experts, dtype: int, device: torch.device):
        params = [p for ex in experts for n in _LORA_NAMES
                  for p in (getattr(ex, n).weight, getattr(ex, n).bias)]
        for p in params:
            if p.device != device or _dtype_code(p) != dtype or not p.is_contiguous():
                raise ValueError("expert and LoRA parameters must be contiguous and share the "
                                 "input's device and dtype")
        shape_key = (dtype, str(device), tuple(tuple(p.shape) for p in params))
        key = (shape_key, tuple((p.data_ptr(), p._version) for p in params))
        if self.key is None or self.key[0] != shape_key:
            self.merged = [_MergedExpert(ex) for ex in experts]
        if key != self.key:
            for ex, mg in zip(experts, self.merged):
                mg.refresh(ex, dtype, _stream(device))
            self.key = key
        return self.merged


def _lora_grads(ex, g_w1, g_b1, g_w2, g_b2):
    """Gradients of an expert's four LoRA Linears (weight, bias each, in the order
    gate_and_up a, b, down a, b) from the gradients G = dL/dW', g = dL/db' of its two merged
    Linears W' = W + s B A, b' = b + s (B a + b_lora) (model.py:175-179,185-189):
    dL/dA = s B^T G, dL/da = s B^T g, dL/dB = s (G A^T + g a^T), dL/db_lora = s g."""
    out = []
    s = float(ex.lora_scale)
    with torch.no_grad():
        for G, g, a, b in ((g_w1, g_b1, ex.lora_gate_and_up_a, ex.lora_gate_and_up_b),
                           (g_w2, g_b2, ex.lora_down_a, ex.lora_down_b)):
            Gf, gf = G.float(), g.float()
            Af, af, Bf = a.weight.float(), a.bias.float(), b.weight.float()
            dA = (Bf.t() @ Gf).mul_(s)
            da = (Bf.t() @ gf).mul_(s)
            dB = (Gf @ Af.t()).addr_(gf, af).mul_(s)
            out += [dA.to(G.dtype), da.to(G.dtype), dB.to(G.dtype), (gf * s).to(G.dtype)]
    return out


class _Plan:
    """Device copy of the experts' parameter pointers and TMA tensor maps.

    Rebuilt whenever a parameter's storage, dtype or device changes (``.to()``,
    ``load_state_dict`` keep storage; ``.to(dtype)`` replaces it)."""

    def __init__(self):
        self.key = None
        self.buf = None

    def get(self, experts, d: int, f: int, dtype: int, device: torch.device) -> int:
        params = []
        for ex in experts:
            params += [ex.gate_and_up.weight, ex.gate_and_up.bias, ex.down.weight, ex.down.bias]
        key = (dtype, str(device), tuple(p.data_ptr() for p in params))
        if key != self.key:
            for p in params:
                if p.device != device or _dtype_code(p) != dtype or not p.is_contiguous():
                    raise ValueError("expert parameters must be contiguous and share the input's "
                                     "device and dtype")
            E = len(experts)
            nbytes = lib.moe_b200_plan_bytes(E)
            buf = torch.empty(nbytes + 128, dtype=torch.uint8, device=device)
            base = (buf.data_ptr() + 127) & ~127
            w1 = _cabi.ptr_array([ex.gate_and_up.weight.data_ptr() for ex in experts])
            b1 = _cabi.ptr_array([ex.gate_and_up.bias.data_ptr() for ex in experts])
            w2 = _cabi.ptr_array([ex.down.weight.data_ptr() for ex in experts])
            b2 = _cabi.ptr_array([ex.down.bias.data_ptr() for ex in experts])
            check(lib.moe_b200_plan_build(w1, b1, w2, b2, E, d, f, dtype, base, nbytes,
                                          _stream(device)), "plan_build")
            self.key, self.buf, self.base = key, buf, base
        return self.base


class _TrainFn(torch.autograd.Function):
    """MOE.forward in training mode as one autograd node: moe_b200_forward_train /
    moe_b200_backward (dropout on h, model.py:183; gradients of model.py:200-276)."""

    @staticmethod
    def forward(ctx, module, x, residual, seed, fine_tuning, *params):
        out, aux = module._forward_train(x, residual, seed, fine_tuning)
        ctx.module, ctx.seed, ctx.gen = module, seed, module._train_gen
        ctx.fine_tuning = fine_tuning
        ctx.has_residual = residual is not None
        ctx.save_for_backward(x)
        return out, aux

    @staticmethod
    def backward(ctx, grad_out, grad_aux):
        m = ctx.module
        if ctx.gen != m._train_gen:
            raise RuntimeError("this block ran another training forward before the backward of this "
                               "one: its workspace holds the later call's tensors")
        (x,) = ctx.saved_tensors
        grads = m._backward_train(x, grad_out.contiguous(), float(grad_aux), ctx.seed, ctx.fine_tuning)
        grad_x = grads.pop(0)
        grad_res = grad_out if ctx.has_residual else None
        return (None, grad_x, grad_res, None, None, *grads)


class _FfnTrainFn(torch.autograd.Function):
    """FeedForward.forward in training mode as one autograd node (moe_b200_experts_train /
    moe_b200_experts_backward: dropout on h, model.py:183; gradients of model.py:173-184)."""

    @staticmethod
    def forward(ctx, module, x, seed, fine_tuning, *params):
        y, h = module._forward_train(x, seed, fine_tuning)
        ctx.module, ctx.seed, ctx.gen = module, seed, module._train_gen
        ctx.fine_tuning = fine_tuning
        ctx.save_for_backward(x, h)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        m = ctx.module
        if ctx.gen != m._train_gen:
            raise RuntimeError("this module ran another training forward before the backward of this "
                               "one: its training workspace holds the later call's tensors")
        x, h = ctx.saved_tensors
        (grad_x,) = m._backward_train(x, h, grad_y.contiguous(), ctx.seed, ctx.fine_tuning)
        return (None, grad_x, None, None, *m._last_param_grads)


class FeedForward(nn.Module):
    """GeGLU feed-forward expert; mirrors reference model.py:154-190.

    ``gate_and_up`` maps d -> 2f (rows [0,f) gate, rows [f,2f) up), ``down`` maps
    f -> d, plus the four LoRA Linears of the reference (rank ``lora_rank``,
    scale ``lora_alpha / lora_rank``), used when ``fine_tuning=True``.

    ``d_ff`` (keyword-only) sets f directly for widths that are not an integer
    multiple of ``hidden_size``."""

    def __init__(self, hidden_size: int, expansion_factor: int = 4, dropout_ratio: float = 0.1,
                 lora_rank: int = 16, lora_alpha: int = 32, *, d_ff: int | None = None):
        super().__init__()
        f = hidden_size * expansion_factor if d_ff is None else d_ff
        self.hidden_size, self.d_ff = hidden_size, f
        self.gate_and_up = nn.Linear(hidden_size, f * 2)
        self.down = nn.Linear(f, hidden_size)
        self.dropout = nn.Dropout(p=dropout_ratio)
        self.lora_scale = lora_alpha / lora_rank
        self.lora_gate_and_up_a = nn.Linear(hidden_size, lora_rank)
        self.lora_gate_and_up_b = nn.Linear(lora_rank, f * 2)
        self.lora_down_a = nn.Linear(f, lora_rank)
        self.lora_down_b = nn.Linear(lora_rank, hidden_size)
        self._plan = _Plan()
        self._plan_ft = _Plan()
        self._lora = _MergedLora()
        self._offsets = None   # ((rows, device), int32 [0, rows]) of the last call
        self._tws = None
        self._tws_key = None
        self._train_gen = 0
        self._last_param_grads = None
        self.last_seed = None

    # -- training mode (bf16): dropout on h and a backward pass -----------------
    def _train_ws(self, M: int, device: torch.device):
        key = (M, str(device))
        if key != self._tws_key:
            d, f = self.hidden_size, self.d_ff
            nbytes = lib.moe_b200_train_workspace_bytes(M, d, f, 1, 1, _cabi.BF16)
            if nbytes == 0:
                raise _cabi.MoeB200Error(lib.moe_b200_last_error_string().decode())
            buf = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=device)
            base = (buf.data_ptr() + 1023) & ~1023
            check(lib.moe_b200_train_setup(M, d, f, 1, 1, _cabi.BF16, base, nbytes, _stream(device)), "train_setup")
            self._tws = (buf, base, nbytes, _cabi.train_workspace_layout(M, d, f, 1, 1, _cabi.BF16))
            self._tws_key = key
        return self._tws

    def _tws_view(self, name: str, shape) -> torch.Tensor:
        buf, base, _, layout = self._tws
        start = base - buf.data_ptr() + layout[name]
        n = 2
        for s in shape:
            n *= s
        return buf[start:start + n].view(torch.bfloat16).view(*shape)

    def _rows(self, tensor):
        x = tensor.reshape(-1, tensor.shape[-1]).contiguous()
        M, dev = x.shape[0], x.device
        if self._offsets is None or self._offsets[0] != (M, str(dev)):
            self._offsets = ((M, str(dev)), torch.tensor([0, M], dtype=torch.int32, device=dev))
        return x, M, dev, self._offsets[1]

    def _train_plan(self, fine_tuning: bool, d, f, dev):
        if fine_tuning:
            return self._plan_ft.get(self._lora.get([self], _cabi.BF16, dev), d, f, _cabi.BF16, dev)
        return self._plan.get([self], d, f, _cabi.BF16, dev)

    def _forward_train(self, tensor, seed: int, fine_tuning: bool = False):
        x, M, dev, offsets = self._rows(tensor)
        d, f = self.hidden_size, self.d_ff
        h = torch.empty(M, f, dtype=x.dtype, device=dev)
        y = torch.empty(M, d, dtype=x.dtype, device=dev)
        with torch.cuda.device(dev):
            plan = self._train_plan(fine_tuning, d, f, dev)
            _, tbase, tbytes, _ = self._train_ws(M, dev)
            status = torch.zeros(16, dtype=torch.int32, device=dev)
            check(lib.moe_b200_experts_train(x.data_ptr(), offsets.data_ptr(), plan, M, d, f, 1,
                                             float(self.dropout.p), seed, tbase, tbytes, h.data_ptr(),
                                             y.data_ptr(), status.data_ptr(), _stream(dev)), "experts_train")
        self._train_gen += 1
        self.last_seed = seed
        return y.reshape(tensor.shape), h

    def _backward_train(self, tensor, h, grad_y, seed: int, fine_tuning: bool = False):
        x, M, dev, offsets = self._rows(tensor)
        d, f = self.hidden_size, self.d_ff
        g = grad_y.reshape(-1, d).contiguous().to(x.dtype)
        grad_x = torch.empty_like(x)
        with torch.cuda.device(dev):
            plan = self._train_plan(fine_tuning, d, f, dev)
            _, tbase, tbytes, _ = self._train_ws(M, dev)
            status = torch.zeros(16, dtype=torch.int32, device=dev)
            check(lib.moe_b200_experts_backward(x.data_ptr(), h.data_ptr(), offsets.data_ptr(), plan, g.data_ptr(),
                                                M, d, f, 1, float(self.dropout.p), seed, tbase, tbytes,
                                                grad_x.data_ptr(), status.data_ptr(), _stream(dev)),
                  "experts_backward")
        self._last_param_grads = [self._tws_view("g_w1", (2 * f, d)).clone(), self._tws_view("g_b1", (2 * f,)).clone(),
                                  self._tws_view("g_w2", (d, f)).clone(), self._tws_view("g_b2", (d,)).clone()]
        if fine_tuning:
            self._last_param_grads += _lora_grads(self, *self._last_param_grads[:4])
        return [grad_x.reshape(tensor.shape)]

    def forward(self, tensor: torch.Tensor, fine_tuning: bool = False) -> torch.Tensor:
        """y = down(gelu_tanh(gate) * up) for every row, through the grouped
        expert kernels with a single group. ``fine_tuning=True`` adds the LoRA
        branch (model.py:175-179,185-189) folded into merged copies of the two weight
        matrices (refreshed when a parameter changes); under ``.train()`` the LoRA tensors
        receive gradients too."""
        if not tensor.is_cuda:
            raise RuntimeError("libmoe_b200 runs on CUDA tensors only; there is no CPU path")
        if self.training and (torch.is_grad_enabled() or self.dropout.p > 0):
            if tensor.dtype != torch.bfloat16:
                raise NotImplementedError("training mode computes in bfloat16")
            seed = int(torch.randint(0, 2 ** 62, (1,), dtype=torch.int64).item())
            params = [self.gate_and_up.weight, self.gate_and_up.bias, self.down.weight, self.down.bias]
            if fine_tuning:
                for lin in (self.lora_gate_and_up_a, self.lora_gate_and_up_b, self.lora_down_a, self.lora_down_b):
                    params += [lin.weight, lin.bias]
            return _FfnTrainFn.apply(self, tensor, seed, bool(fine_tuning), *params)
        dtype = _dtype_code(tensor)
        shape = tensor.shape
        x = tensor.reshape(-1, shape[-1]).contiguous()
        M, d, f = x.shape[0], self.hidden_size, self.d_ff
        dev = x.device
        with torch.cuda.device(dev):
            plan = (self._plan_ft if fine_tuning else self._plan).get(
                self._lora.get([self], dtype, dev) if fine_tuning else [self], d, f, dtype, dev)
            if self._offsets is None or self._offsets[0] != (M, str(dev)):
                self._offsets = ((M, str(dev)), torch.tensor([0, M], dtype=torch.int32, device=dev))
            offsets = self._offsets[1]
            status = torch.zeros(16, dtype=torch.int32, device=dev)
            h = torch.empty(M, f, dtype=x.dtype, device=dev)
            y = torch.empty(M, d, dtype=x.dtype, device=dev)
            check(lib.moe_b200_experts(x.data_ptr(), offsets.data_ptr(), plan, M, d, f, 1, dtype, 0,
                                       h.data_ptr(), y.data_ptr(), status.data_ptr(), _stream(dev)),
                  "experts")
        return y.reshape(shape)


class MOE(nn.Module):
    """Mixture-of-experts feed-forward block; mirrors reference model.py:192-276.

    Same positional/keyword arguments as the reference constructor
    (model.py:193); ``device`` is accepted and stored but not used, the kernels
    run where the input lives. Keyword-only extensions: ``top_k`` (the reference
    fixes 2, model.py:210) and ``d_ff`` (free per-branch width)."""

    def __init__(self, hidden_size: int, num_experts: int = 8, expansion_factor: int = 4,
                 dropout_ratio: float = 0.1, lora_rank: int = 16, lora_alpha: int = 32,
                 device: str = "mps", *, top_k: int = 2, d_ff: int | None = None):
        super().__init__()
        self.gate = nn.Linear(hidden_size, num_experts)
        self.num_experts = num_experts
        self.experts = nn.ModuleList([
            FeedForward(hidden_size, expansion_factor=expansion_factor, dropout_ratio=dropout_ratio,
                        lora_rank=lora_rank, lora_alpha=lora_alpha, d_ff=d_ff)
            for _ in range(num_experts)])
        self.device = device
        self.hidden_size = hidden_size
        self.d_ff = self.experts[0].d_ff
        self.top_k = top_k
        self._plan = _Plan()
        self._plan_ft = _Plan()
        self._lora = _MergedLora()
        self._ws = None
        self._ws_key = None
        self._tws = None
        self._tws_key = None
        self._train_gen = 0
        self.last = None  # views into the workspace of the most recent call

    # -- workspace ---------------------------------------------------------
    def _workspace(self, N: int, dtype: int, device: torch.device):
        key = (N, dtype, str(device))
        if key != self._ws_key:
            d, f, E, k = self.hidden_size, self.d_ff, self.num_experts, self.top_k
            nbytes = _cabi.workspace_bytes(N, d, f, E, k, dtype)
            # zeroed: the small-N kernels keep their counters in the status region and leave
            # them zero after every call (FLAG_WS_CLEAN below)
            buf = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=device)
            base = (buf.data_ptr() + 1023) & ~1023
            self._ws = (buf, base, nbytes, _cabi.workspace_layout(N, d, f, E, k, dtype))
            self._ws_key = key
        return self._ws

    def _view(self, name: str, dtype: torch.dtype, shape) -> torch.Tensor:
        buf, base, _, layout = self._ws
        start = base - buf.data_ptr() + layout[name]
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        return buf[start:start + nbytes].view(dtype).view(*shape)

    def forward(self, tensor: torch.Tensor, fine_tuning: bool = False, *,
                residual: torch.Tensor | None = None,
                norm: nn.LayerNorm | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """``tensor`` [B,S,d] -> ([B,S,d] in the input dtype, load-balancing loss).

        With ``residual`` (same shape and dtype) the caller's skip connection
        (model.py:319) is added inside the combine kernel. With ``norm`` (the caller's
        ``norm2``, model.py:298,312) ``tensor`` is the tensor BEFORE that LayerNorm: the
        block normalises it on the fly in its router and dispatch kernels, so
        ``moe(x, residual=x, norm=layer.norm2)`` replaces model.py:311-319. ``fine_tuning=True``
        runs the experts with their LoRA branches (model.py:175-179,185-189)
        folded into merged copies of their weights (refreshed when a parameter
        changes); under ``.train()`` the LoRA tensors receive gradients too."""
        if not tensor.is_cuda:
            raise RuntimeError("libmoe_b200 runs on CUDA tensors only; there is no CPU path")
        if self.training and (torch.is_grad_enabled() or self.experts[0].dropout.p > 0):
            # training mode: dropout on h (model.py:183) and a backward pass
            if norm is not None:
                raise NotImplementedError("training mode has no backward pass for the folded LayerNorm: "
                                          "apply the LayerNorm in front of the block")
            if tensor.dtype != torch.bfloat16:
                raise NotImplementedError("training mode computes in bfloat16")
            seed = int(torch.randint(0, 2 ** 62, (1,), dtype=torch.int64).item())   # torch's CPU generator
            params = [self.gate.weight, self.gate.bias]
            for ex in self.experts:
                params += [ex.gate_and_up.weight, ex.gate_and_up.bias, ex.down.weight, ex.down.bias]
            if fine_tuning:
                for ex in self.experts:
                    for lin in (ex.lora_gate_and_up_a, ex.lora_gate_and_up_b, ex.lora_down_a, ex.lora_down_b):
                        params += [lin.weight, lin.bias]
            return _TrainFn.apply(self, tensor, residual, seed, bool(fine_tuning), *params)
        dtype = _dtype_code(tensor)
        shape = tensor.shape
        d, f, E, k = self.hidden_size, self.d_ff, self.num_experts, self.top_k
        if shape[-1] != d:
            raise ValueError(f"last dimension {shape[-1]} != hidden_size {d}")
        x = tensor.reshape(-1, d).contiguous()
        N = x.shape[0]
        dev = x.device
        res_ptr = None
        if residual is not None:
            if residual.shape != shape or residual.dtype != tensor.dtype or residual.device != dev:
                raise ValueError("residual must match the input's shape, dtype and device")
            residual = residual.reshape(-1, d).contiguous()
            res_ptr = residual.data_ptr()
        gw, gb = self.gate.weight, self.gate.bias
        if gw.device != dev or _dtype_code(gw) != dtype:
            raise ValueError("gate parameters must share the input's device and dtype")
        nw = nb = None
        eps = 0.0
        if norm is not None:
            if (tuple(norm.normalized_shape) != (d,) or norm.weight is None or norm.bias is None
                    or norm.weight.device != dev or _dtype_code(norm.weight) != dtype):
                raise ValueError("norm must be an affine LayerNorm over the last dimension with "
                                 "the input's device and dtype")
            nw, nb, eps = norm.weight.data_ptr(), norm.bias.data_ptr(), float(norm.eps)
        out = torch.empty_like(x)
        with torch.cuda.device(dev):
            if fine_tuning:
                plan = self._plan_ft.get(self._lora.get(list(self.experts), dtype, dev), d, f, dtype, dev)
            else:
                plan = self._plan.get(self.experts, d, f, dtype, dev)
            _, base, nbytes, _ = self._workspace(N, dtype, dev)
            check(lib.moe_b200_forward(x.data_ptr(), gw.data_ptr(), gb.data_ptr(), plan, res_ptr,
                                       nw, nb, eps, N, d, f, E, k, dtype, _cabi.FLAG_WS_CLEAN, base, nbytes,
                                       out.data_ptr(), _stream(dev)), "forward")
        self.last = {
            "logits": self._view("logits", torch.float32, (N, E)),
            "idx": self._view("idx", torch.int32, (N, k)),
            "w": self._view("w", torch.float32, (N, k)),
            "cnt_slot": self._view("cnt_slot", torch.int32, (k, E)),
            "offsets": self._view("offsets", torch.int32, (E + 1,)),
            "psum": self._view("psum", torch.float32, (E,)),
            "row_of": self._view("row_of", torch.int32, (N, k)),
            "status": self._view("status", torch.int32, (16,)),
        }
        aux = self._view("aux", torch.float32, (1,))[0].clone()
        return out.reshape(shape), aux

    # -- training mode -------------------------------------------------------
    def _train_workspace(self, N: int, dtype: int, device: torch.device):
        key = (N, dtype, str(device))
        if key != self._tws_key:
            d, f, E, k = self.hidden_size, self.d_ff, self.num_experts, self.top_k
            nbytes = lib.moe_b200_train_workspace_bytes(N, d, f, E, k, dtype)
            if nbytes == 0:
                raise _cabi.MoeB200Error(lib.moe_b200_last_error_string().decode())
            buf = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=device)
            base = (buf.data_ptr() + 1023) & ~1023
            check(lib.moe_b200_train_setup(N, d, f, E, k, dtype, base, nbytes, _stream(device)), "train_setup")
            self._tws = (buf, base, nbytes, _cabi.train_workspace_layout(N, d, f, E, k, dtype))
            self._tws_key = key
        return self._tws

    def _tws_view(self, name: str, shape) -> torch.Tensor:
        buf, base, _, layout = self._tws
        start = base - buf.data_ptr() + layout[name]
        n = 2
        for s in shape:
            n *= s
        return buf[start:start + n].view(torch.bfloat16).view(*shape)

    def _train_plan(self, fine_tuning: bool, d, f, dtype, dev):
        if fine_tuning:
            return self._plan_ft.get(self._lora.get(list(self.experts), dtype, dev), d, f, dtype, dev)
        return self._plan.get(self.experts, d, f, dtype, dev)

    def _forward_train(self, tensor, residual, seed: int, fine_tuning: bool = False):
        dtype = _dtype_code(tensor)
        shape = tensor.shape
        d, f, E, k = self.hidden_size, self.d_ff, self.num_experts, self.top_k
        if shape[-1] != d:
            raise ValueError(f"last dimension {shape[-1]} != hidden_size {d}")
        x = tensor.reshape(-1, d).contiguous()
        N = x.shape[0]
        dev = x.device
        res_ptr = None
        if residual is not None:
            if residual.shape != shape or residual.dtype != tensor.dtype or residual.device != dev:
                raise ValueError("residual must match the input's shape, dtype and device")
            res_ptr = residual.reshape(-1, d).contiguous().data_ptr()
        out = torch.empty_like(x)
        with torch.cuda.device(dev):
            plan = self._train_plan(fine_tuning, d, f, dtype, dev)
            _, base, nbytes, _ = self._workspace(N, dtype, dev)
            _, tbase, tbytes, _ = self._train_workspace(N, dtype, dev)
            check(lib.moe_b200_forward_train(
                x.data_ptr(), self.gate.weight.data_ptr(), self.gate.bias.data_ptr(), plan, res_ptr,
                N, d, f, E, k, dtype, float(self.experts[0].dropout.p), seed, base, nbytes, tbase, tbytes,
                out.data_ptr(), _stream(dev)), "forward_train")
        self._train_gen += 1
        self.last = {
            "logits": self._view("logits", torch.float32, (N, E)),
            "idx": self._view("idx", torch.int32, (N, k)),
            "w": self._view("w", torch.float32, (N, k)),
            "cnt_slot": self._view("cnt_slot", torch.int32, (k, E)),
            "offsets": self._view("offsets", torch.int32, (E + 1,)),
            "psum": self._view("psum", torch.float32, (E,)),
            "row_of": self._view("row_of", torch.int32, (N, k)),
            "status": self._view("status", torch.int32, (16,)),
            "seed": seed,
        }
        aux = self._view("aux", torch.float32, (1,))[0].clone()
        return out.reshape(shape), aux

    def _backward_train(self, tensor, grad_out, grad_aux: float, seed: int, fine_tuning: bool = False):
        """[grad_x, grad gate.weight, grad gate.bias, then per expert the gradients of
        gate_and_up.weight, gate_and_up.bias, down.weight, down.bias; with ``fine_tuning`` then
        per expert those of the four LoRA Linears (weight, bias each)].

        With ``fine_tuning`` the kernels run on the merged weights W' = W + s B A,
        b' = b + s (B a + b_lora) (model.py:175-179,185-189), so what they return for a Linear
        is G = dL/dW' = dL/dW and g = dL/db' = dL/db; _lora_grads forms the LoRA tensors'
        gradients from them: four small products per Linear on the gradient the grouped
        kernel already produced."""
        dtype = _dtype_code(tensor)
        shape = tensor.shape
        d, f, E, k = self.hidden_size, self.d_ff, self.num_experts, self.top_k
        x = tensor.reshape(-1, d).contiguous()
        N = x.shape[0]
        dev = x.device
        g = grad_out.reshape(-1, d).contiguous()
        if g.dtype != tensor.dtype:
            g = g.to(tensor.dtype)
        grad_x = torch.empty_like(x)
        with torch.cuda.device(dev):
            plan = self._train_plan(fine_tuning, d, f, dtype, dev)
            _, base, nbytes, _ = self._workspace(N, dtype, dev)
            _, tbase, tbytes, _ = self._train_workspace(N, dtype, dev)
            check(lib.moe_b200_backward(
                x.data_ptr(), self.gate.weight.data_ptr(), plan, g.data_ptr(), grad_aux, N, d, f, E, k, dtype,
                float(self.experts[0].dropout.p), seed, base, nbytes, tbase, tbytes, grad_x.data_ptr(),
                _stream(dev)), "backward")
        # copies: the workspace is overwritten by the next backward
        grads = [grad_x.reshape(shape), self._tws_view("g_wg", (E, d)).clone(), self._tws_view("g_bg", (E,)).clone()]
        g_w1 = self._tws_view("g_w1", (E, 2 * f, d)).clone()
        g_b1 = self._tws_view("g_b1", (E, 2 * f)).clone()
        g_w2 = self._tws_view("g_w2", (E, d, f)).clone()
        g_b2 = self._tws_view("g_b2", (E, d)).clone()
        for e in range(E):
            grads += [g_w1[e], g_b1[e], g_w2[e], g_b2[e]]
        if fine_tuning:
            for e, ex in enumerate(self.experts):
                grads += _lora_grads(ex, g_w1[e], g_b1[e], g_w2[e], g_b2[e])
        return grads

    def device_status(self) -> int:
        """Status word of the most recent call (0 = ok); synchronises. A non-zero status is
        returned once: the status region is zeroed again so that later calls start clean."""
        if not self.last:
            return 0
        code = int(self.last["status"][0].item())
        if code != 0:
            self._view("status", torch.int32, (_cabi.READY_OFFSET + _cabi.READY_INTS,)).zero_()
        return code
