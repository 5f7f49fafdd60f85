"""The memory step of the reference's ``MemoryTransformerBlock`` (memory_transformer/memory_block.py:468-487,
549-558): ``h + memory_attn(memory_layernorm(h), memory)``, with the submodule and parameter names of that
block so the matching slice of its state dict loads unchanged.  Self-attention and the MLPs of the block are
not part of this package."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import functional as F_moc
from . import ops
from .memory_attention import MemoryCrossAttention


class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, kind, eps):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).float()
        y, stats = ops.norm_fwd(x2, weight.float(), None if bias is None else bias.float(), kind, eps,
                                torch.float32)
        ctx.save_for_backward(x2, weight.float(), stats)
        ctx.cfg = (kind, bias is not None, shape, x.dtype, weight.dtype)
        return y.view(shape).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        x2, w, stats = ctx.saved_tensors
        kind, has_bias, shape, x_dtype, w_dtype = ctx.cfg
        dx, dw, db = ops.norm_bwd(g.reshape(-1, shape[-1]).float(), x2, w, stats, None, kind, has_bias)
        return dx.view(shape).to(x_dtype), dw.to(w_dtype), None if db is None else db.to(w_dtype), None, None


class RMSNorm(nn.Module):
    """x / sqrt(mean(x^2) + eps) * weight (memory_block.py:18-28), on the GPU."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _Norm.apply(x, self.weight, None, "rms", self.eps)


class MemorySubBlock(nn.Module):
    """``forward(hidden_states, memory) -> hidden_states + memory_attn(memory_layernorm(hidden_states), memory)``.

    The normalisation writes the query projection's operand directly and the residual is added in the
    output projection's epilogue, so neither costs a pass over (B, L, d) of its own.
    """

    def __init__(self, hidden_dim: int, num_heads: int, num_kv_heads: Optional[int] = None,
                 memory_dim: Optional[int] = None, use_rms_norm: bool = True, norm_eps: float = 1e-6,
                 wo_init_zero: bool = True, compute_dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.use_rms_norm = use_rms_norm
        self.norm_eps = norm_eps
        self.memory_layernorm = RMSNorm(hidden_dim, eps=norm_eps) if use_rms_norm else nn.LayerNorm(hidden_dim,
                                                                                                    eps=norm_eps)
        self.memory_attn = MemoryCrossAttention(hidden_dim, num_heads, num_kv_heads=num_kv_heads,
                                                memory_dim=memory_dim, wo_init_zero=wo_init_zero,
                                                compute_dtype=compute_dtype)

    def forward(self, hidden_states: torch.Tensor, memory: torch.Tensor) -> torch.Tensor:
        if memory is None:
            raise ValueError("memory must be provided")
        a = self.memory_attn
        return F_moc.cross_attention(
            hidden_states, memory, a.q_proj.weight, a.k_proj.weight, a.v_proj.weight, a.o_proj.weight,
            a.num_heads, a.num_kv_heads, a._compute_dtype(hidden_states),
            pre_norm="rms" if self.use_rms_norm else "layernorm", norm_weight=self.memory_layernorm.weight,
            norm_bias=getattr(self.memory_layernorm, "bias", None), norm_eps=self.norm_eps, add_residual=True)
