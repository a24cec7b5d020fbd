"""Drop-in for the reference's ``Attention`` (model.py:59-152): same constructor, attribute
and parameter names, ``state_dict`` layout and ``forward`` signature. The two Linears
(fused QKV, output) and the head-gate Linear are plain library GEMMs; everything between
them — head split, shared KV heads, RoPE from the model's own table, scores, mask, softmax,
the product with V and the sigmoid head gate — is one kernel of libmoe_b200
(``moe_b200_attention``), so the [B, H, S, S] score tensor is never materialised.

bf16 on CUDA, head_dim 64, contexts up to 128 tokens, mask None or one additive [S, S] mask
shared by the batch (the causal mask of model.py:585-591); other inputs raise.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _cabi
from ._cabi import lib, check
from .moe import _stream


class _MergedLinear:
    """W + s * B A and b + s * (B a + b_lora) of one Linear with its LoRA pair (model.py:98-102,
    144-149), refreshed when one of the six tensors changes."""

    def __init__(self):
        self.key, self.w, self.b = None, None, None

    def get(self, lin, a, b, scale):
        params = (lin.weight, lin.bias, a.weight, a.bias, b.weight, b.bias)
        key = tuple((p.data_ptr(), p._version) for p in params)
        if key != self.key:
            if self.w is None or self.w.shape != lin.weight.shape or self.w.device != lin.weight.device:
                self.w, self.b = torch.empty_like(lin.weight), torch.empty_like(lin.bias)
            dev = lin.weight.device
            with torch.cuda.device(dev):
                check(lib.moe_b200_lora_merge(
                    lin.weight.data_ptr(), lin.bias.data_ptr(), a.weight.data_ptr(), a.bias.data_ptr(),
                    b.weight.data_ptr(), b.bias.data_ptr(), float(scale), lin.out_features, lin.in_features,
                    a.out_features, _cabi.BF16, self.w.data_ptr(), self.b.data_ptr(), _stream(dev)),
                    "lora_merge")
            self.key = key
        return self.w, self.b


class Attention(nn.Module):
    def __init__(self, hidden_dim: int, head_dim: int, q_head: int, kv_head: int, embedding: nn.Module,
                 lora_rank: int = 16, lora_alpha: int = 32):
        super().__init__()
        self.head_dim = head_dim
        self.q_head = q_head
        self.kv_head = kv_head
        self.embedding = embedding          # the model's RoPE table: rows [cos | signed sin], model.py:14-36
        self.qkv = nn.Linear(hidden_dim, (q_head + kv_head * 2) * head_dim)
        self.o = nn.Linear(q_head * head_dim, hidden_dim)
        self.scaler = 1 / math.sqrt(head_dim)
        self.lora_scale = lora_alpha / lora_rank
        self.lora_qkv_a = nn.Linear(hidden_dim, lora_rank)
        self.lora_qkv_b = nn.Linear(lora_rank, (q_head + kv_head * 2) * head_dim)
        self.lora_o_a = nn.Linear(q_head * head_dim, lora_rank)
        self.lora_o_b = nn.Linear(lora_rank, hidden_dim)
        if q_head != kv_head:
            assert q_head % kv_head == 0
            self.multi_query_attention = True
            self.q_kv_scale = q_head // kv_head
        else:
            self.multi_query_attention = False
        self.gate = nn.Linear(hidden_dim, q_head)
        self._merged_qkv, self._merged_o = _MergedLinear(), _MergedLinear()
        self._table = None

    def _pos_table(self, device):
        pe = self.embedding.pos_emb
        key = (pe.data_ptr(), pe._version, str(device))
        if self._table is None or self._table[0] != key:
            self._table = (key, pe.detach().to(device=device, dtype=torch.float32).contiguous())
        return self._table[1]

    def forward(self, tensor: torch.Tensor, attention_mask: torch.Tensor = None,
                fine_tuning: bool = False) -> torch.Tensor:
        if not tensor.is_cuda or tensor.dtype != torch.bfloat16:
            raise NotImplementedError("the attention kernel runs on CUDA tensors in bfloat16")
        if torch.is_grad_enabled() and (tensor.requires_grad or self.qkv.weight.requires_grad):
            raise NotImplementedError("the attention kernel has no backward pass; use torch.no_grad()")
        B, S, hid = tensor.shape
        dev = tensor.device
        if fine_tuning:
            wq, bq = self._merged_qkv.get(self.qkv, self.lora_qkv_a, self.lora_qkv_b, self.lora_scale)
            wo, bo = self._merged_o.get(self.o, self.lora_o_a, self.lora_o_b, self.lora_scale)
        else:
            wq, bq, wo, bo = self.qkv.weight, self.qkv.bias, self.o.weight, self.o.bias
        x = tensor.contiguous()
        qkv = F.linear(x, wq, bq)
        gate = F.linear(x, self.gate.weight, self.gate.bias)          # [B,S,q_head] logits (model.py:139)
        mask_ptr = None
        if attention_mask is not None:
            m = attention_mask
            if m.numel() != S * S:
                raise NotImplementedError("one additive [S, S] mask for the whole batch is supported")
            mask = m.reshape(S, S).to(device=dev, dtype=torch.float32).contiguous()
            mask_ptr = mask.data_ptr()
        table = self._pos_table(dev)
        if table.shape[0] < S or table.shape[1] != 2 * self.head_dim:
            raise ValueError("the RoPE table is shorter than the sequence or has another head_dim")
        out = torch.empty(B, S, self.q_head * self.head_dim, dtype=tensor.dtype, device=dev)
        with torch.cuda.device(dev):
            check(lib.moe_b200_attention(qkv.data_ptr(), gate.data_ptr(), table.data_ptr(), mask_ptr, B, S,
                                         self.q_head, self.kv_head, self.head_dim, float(self.scaler),
                                         out.data_ptr(), _stream(dev)), "attention")
        return F.linear(out, wo, bo)
