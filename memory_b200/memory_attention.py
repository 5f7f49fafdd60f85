"""``MemoryCrossAttention`` with the reference's constructor, parameters and forward contract
(memory_transformer/memory_attention.py:60-146, 320-478), computed by the CUDA kernels."""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import functional as F_moc


class MemoryCrossAttention(nn.Module):
    """Cross attention from hidden states to memory rows that were already gathered and weighted.

    ``forward(hidden_states, memory)`` takes memory of shape (N, d) or (B, N, d) and returns
    ``(output (B, L, d), None)``.  Low-rank and reduced-dimension projection variants of the
    reference are not part of this path and are rejected.  ``use_flash_attention`` and
    ``gradient_checkpointing`` are accepted for signature compatibility; the kernels never
    materialise the score matrix, so neither changes what is computed.
    """

    def __init__(self, hidden_dim: int, num_heads: int, num_kv_heads: Optional[int] = None,
                 memory_dim: Optional[int] = None, use_low_rank_projections: bool = False,
                 projection_rank: Optional[int] = None, reduced_dim_mode: bool = False,
                 reduced_dim: Optional[int] = None, wo_init_zero: bool = True, dropout: float = 0.0,
                 use_flash_attention: bool = True, gradient_checkpointing: bool = False,
                 compute_dtype: Optional[torch.dtype] = None):
        super().__init__()
        if use_low_rank_projections or reduced_dim_mode:
            raise NotImplementedError("low-rank / reduced-dim projections are outside the accelerated path")
        if dropout != 0.0:
            raise NotImplementedError("attention dropout is not supported by the fused kernels")
        self.hidden_dim = hidden_dim
        self.memory_dim = memory_dim if memory_dim is not None else hidden_dim
        self.num_heads = num_heads
        self.num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        if self.num_heads <= 0:
            raise ValueError(f"num_heads must be > 0, got {self.num_heads}")
        if hidden_dim % num_heads != 0:
            raise ValueError(f"hidden_dim ({hidden_dim}) must be divisible by num_heads ({num_heads})")
        if self.num_kv_heads <= 0:
            raise ValueError(f"num_kv_heads must be > 0, got {self.num_kv_heads}")
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(
                f"num_heads ({self.num_heads}) must be divisible by num_kv_heads ({self.num_kv_heads})")
        self.head_dim = hidden_dim // num_heads
        self.kv_hidden_dim = self.num_kv_heads * self.head_dim
        self.num_kv_groups = self.num_heads // self.num_kv_heads
        self.scale = self.head_dim ** -0.5
        self.dropout = dropout
        self.use_flash_attention = use_flash_attention
        self.gradient_checkpointing = gradient_checkpointing
        self.reduced_dim_mode = False
        self.use_low_rank_projections = False
        self.compute_dtype = compute_dtype
        self.q_proj = nn.Linear(self.hidden_dim, self.hidden_dim, bias=False)
        self.k_proj = nn.Linear(self.memory_dim, self.kv_hidden_dim, bias=False)
        self.v_proj = nn.Linear(self.memory_dim, self.kv_hidden_dim, bias=False)
        self.o_proj = nn.Linear(self.hidden_dim, self.hidden_dim, bias=False)
        if wo_init_zero:
            nn.init.zeros_(self.o_proj.weight)

    def forward(self, hidden_states: torch.Tensor, memory: Optional[torch.Tensor] = None,
                token_routing_state: Optional[Dict[str, Any]] = None,
                token_routing_kernel_version: str = "v2", return_attn_weights: bool = False
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        if token_routing_state is not None:
            if return_attn_weights:
                raise ValueError("return_attn_weights=True is not supported for token_routing_state path.")
            return self._forward_token_routed(hidden_states, token_routing_state), None
        if memory is None:
            raise ValueError("memory must be provided when token_routing_state is None.")
        if return_attn_weights:
            raise NotImplementedError("attention weights are never materialised by the fused kernels")
        out = F_moc.cross_attention(hidden_states, memory, self.q_proj.weight, self.k_proj.weight,
                                    self.v_proj.weight, self.o_proj.weight, self.num_heads, self.num_kv_heads,
                                    self._compute_dtype(hidden_states))
        return out, None

    def _forward_token_routed(self, hidden_states: torch.Tensor, state: Dict[str, Any]) -> torch.Tensor:
        """Token-level routing payload of the reference's model (model.py:592-606): dense attention over the
        shared rows plus, per token, its selected chapters (memory_attention.py:480-716), then o_proj.  With
        ``chapter_weights`` every chapter has its own softmax and the outputs are mixed by the weights; without,
        the selected chapters share one softmax.  ``kernel_version`` / ``assume_sorted_topk`` select among the
        reference's Triton variants and have nothing to choose between here."""
        idx = state.get("token_chapter_indices", None)
        if idx is None:
            raise ValueError("token_routing_state must include token_chapter_indices.")
        if idx.dim() != 3:
            raise ValueError(f"token_chapter_indices must be rank-3 [B, T, topk], got shape {tuple(idx.shape)}.")
        if idx.shape[0] != hidden_states.shape[0] or idx.shape[1] != hidden_states.shape[1]:
            raise ValueError(
                "token_chapter_indices shape prefix must match hidden_states [B, T, ...]. "
                f"got hidden_states={tuple(hidden_states.shape)}, token_chapter_indices={tuple(idx.shape)}")
        cd = self._compute_dtype(hidden_states)
        args = dict(num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                    tokens_per_chapter=int(state.get("tokens_per_chapter", 0)),
                    routed_scale=float(state.get("routed_scale", 1.0)), compute_dtype=cd)
        w = (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight, self.o_proj.weight)
        shared, routed = state.get("shared_memory"), state.get("routed_memory")
        if args["tokens_per_chapter"] <= 0:
            routed = None
        weights = state.get("chapter_weights", None)
        if weights is not None:
            return F_moc.token_routed_attention(hidden_states, shared, routed, idx, weights, *w, **args)
        return F_moc.token_routed_attention_joint(hidden_states, shared, routed, idx, *w, **args)

    def _compute_dtype(self, hidden_states: torch.Tensor) -> torch.dtype:
        """Arithmetic type of the projections and the attention.  An explicit ``compute_dtype`` wins; otherwise
        an active CUDA autocast region decides, as it does for the reference's ``nn.Linear`` layers (the trainer
        wraps the model in bf16 autocast, training/trainer.py:100-103, while parameters and the residual
        stream stay fp32) -- autocast never reaches inside a custom autograd function, so it is read here.
        Outside autocast the hidden states' own dtype is used."""
        if self.compute_dtype is not None:
            return self.compute_dtype
        if hidden_states.is_cuda and torch.is_autocast_enabled("cuda"):
            dt = torch.get_autocast_dtype("cuda")
            if dt == torch.bfloat16:
                return dt
            raise NotImplementedError(f"autocast to {dt}: the tensor-core kernels compute in bf16")
        return hidden_states.dtype
