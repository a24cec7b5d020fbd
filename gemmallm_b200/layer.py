"""Drop-in for the reference's ``LLMLayer`` (model.py:278-321): the decoder layer the
Mixture-of-Experts block sits in. Same constructor, attribute and parameter names and
``state_dict`` layout (``norm1``, ``mqa``, ``norm2``, ``moe`` or ``ffn``), same ``forward``
signature and return value (tensor, load-balancing loss).

What the layer adds over assigning ``layer.moe`` / ``layer.mqa`` in the reference's own layer:
in inference the second LayerNorm (model.py:298,312) is folded into the block's router and
dispatch kernels and the second skip connection (model.py:319) into its combine kernel, so
neither is a pass over the activations of its own; the first LayerNorm runs the library's row
kernel (``moe_b200_layernorm``). The attention's Linears and the first skip connection stay
library code around ``moe_b200_attention``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _cabi
from ._cabi import lib, check
from .attention import Attention
from .moe import MOE, FeedForward, _stream


def _layernorm(norm: nn.LayerNorm, x: torch.Tensor) -> torch.Tensor:
    """norm(x) by the library's row kernel (moe_b200_layernorm) for contiguous bf16/fp32 CUDA
    tensors outside autograd; torch's own LayerNorm otherwise (training)."""
    d = x.shape[-1]
    if (not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float32) or d % 8 != 0
            or norm.weight is None or norm.bias is None or norm.weight.dtype != x.dtype
            or (torch.is_grad_enabled() and (x.requires_grad or norm.weight.requires_grad))):
        return norm(x)
    xc = x.contiguous()
    out = torch.empty_like(xc)
    code = _cabi.BF16 if x.dtype == torch.bfloat16 else _cabi.F32
    with torch.cuda.device(x.device):
        check(lib.moe_b200_layernorm(xc.data_ptr(), norm.weight.data_ptr(), norm.bias.data_ptr(),
                                     float(norm.eps), xc.numel() // d, d, code, out.data_ptr(),
                                     _stream(x.device)), "layernorm")
    return out


class LLMLayer(nn.Module):
    def __init__(self, hidden_dim: int, head_dim: int, q_head: int, kv_head: int, embedding: nn.Module,
                 expansion_factor: int = 4, dropout_ratio: float = 0.1, use_moe: bool = False,
                 num_experts: int = 8, lora_rank: int = 16, lora_alpha: int = 32, device: str = "mps"):
        super().__init__()
        self.use_moe = use_moe
        self.norm1 = nn.LayerNorm(hidden_dim)
        self.mqa = Attention(hidden_dim, head_dim, q_head, kv_head, embedding, lora_rank=lora_rank,
                             lora_alpha=lora_alpha)
        self.norm2 = nn.LayerNorm(hidden_dim)
        if self.use_moe:
            self.moe = MOE(hidden_dim, num_experts=num_experts, expansion_factor=expansion_factor,
                           dropout_ratio=dropout_ratio, lora_rank=lora_rank, device=device)
        else:
            self.ffn = FeedForward(hidden_dim, expansion_factor=expansion_factor, dropout_ratio=dropout_ratio,
                                   lora_rank=lora_rank, lora_alpha=lora_alpha)
        self.device = device

    def forward(self, tensor: torch.Tensor, attention_mask: torch.Tensor = None, fine_tuning: bool = False):
        skip_connection = tensor
        tensor = _layernorm(self.norm1, tensor)
        tensor = self.mqa(tensor, attention_mask=attention_mask, fine_tuning=fine_tuning)
        tensor = tensor + skip_connection                      # model.py:308
        if self.use_moe:
            if self.moe.training:
                # training mode has no backward pass for the folded LayerNorm
                return self.moe(self.norm2(tensor), fine_tuning=fine_tuning, residual=tensor)
            # model.py:311-319 in the block's own kernels
            return self.moe(tensor, fine_tuning=fine_tuning, residual=tensor, norm=self.norm2)
        out = self.ffn(self.norm2(tensor), fine_tuning=fine_tuning) + tensor
        return out, torch.zeros((), dtype=out.dtype, device=out.device)   # no load-balancing loss (model.py:317)
