"""``ChapterRouter`` with the reference's constructor, attributes and return contract
(memory_transformer/router.py:15-340), computed by the CUDA router kernels."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import functional as F_moc


class ChapterRouter(nn.Module):
    """Top-k chapter selection with load-balance / auxiliary / z losses.

    Same surface as the reference module: ``.router`` is an ``nn.Linear(hidden_dim, num_chapters)``
    (weight N(0, 0.02), zero bias), ``.top_k`` and ``.routing_strategy`` may be changed by the
    caller between calls, ``forward`` returns ``(indices int64, weights, losses)``.
    Selection order is (weight descending, chapter id ascending).
    """

    def __init__(self, hidden_dim: int, num_chapters: int, top_k: int = 1, routing_strategy: str = "sequence"):
        super().__init__()
        if num_chapters <= 0:
            raise ValueError(f"num_chapters must be > 0, got {num_chapters}")
        if top_k <= 0:
            raise ValueError(f"top_k must be > 0, got {top_k}")
        if top_k > num_chapters:
            raise ValueError(f"top_k ({top_k}) must be <= num_chapters ({num_chapters})")
        self.hidden_dim = hidden_dim
        self.num_chapters = num_chapters
        self.top_k = top_k
        self.routing_strategy = routing_strategy
        self.router = nn.Linear(hidden_dim, num_chapters, bias=True)
        nn.init.normal_(self.router.weight, mean=0.0, std=0.02)
        nn.init.zeros_(self.router.bias)

    def forward(self, hidden_states: torch.Tensor, return_losses: bool = True, exclude_prefix_chapters: int = 0,
                rolling_window_size: Optional[int] = None
                ) -> Tuple[torch.Tensor, torch.Tensor, Dict[str, torch.Tensor]]:
        pos_weight = None
        if self.routing_strategy in ("sequence-rolling", "sequence_rolling"):
            # router.py:100-105, 159-195: the mean over t of the rolling-window means is one coefficient per position
            if hidden_states.dim() != 3:
                raise ValueError(f"hidden_states must be 3D (B, T, D), got shape {tuple(hidden_states.shape)}")
            pos_weight = self._rolling_coefficients(hidden_states.shape[1], rolling_window_size, hidden_states.device)
        elif self.routing_strategy == "token":
            # router.py:106-110 projects every token and averages the logits; the projection is linear, so this is
            # the router applied to the mean state (equal up to rounding)
            pass
        elif self.routing_strategy != "sequence":
            raise ValueError(f"Unknown routing_strategy: {self.routing_strategy}")
        if exclude_prefix_chapters < 0 or exclude_prefix_chapters > self.num_chapters:
            raise ValueError(
                f"exclude_prefix_chapters must be in [0, {self.num_chapters}], got {exclude_prefix_chapters}")
        idx, w, _, _, losses = F_moc.route(hidden_states, self.router.weight, self.router.bias, self.top_k,
                                           exclude_prefix_chapters, 1.0, return_losses, pos_weight=pos_weight)
        return idx, w, losses

    def _rolling_coefficients(self, seq: int, window: Optional[int], device) -> torch.Tensor:
        key = (int(seq), None if window is None else int(window), str(device))
        cache = self.__dict__.setdefault("_rolling_cache", {})
        if key not in cache:
            if len(cache) > 16:
                cache.clear()
            cache[key] = F_moc.ops.rolling_pool_coefficients(seq, window).to(device)
        return cache[key]

    def route_token_level(self, hidden_states: torch.Tensor, return_losses: bool = True,
                          exclude_prefix_chapters: int = 0
                          ) -> Tuple[torch.Tensor, torch.Tensor, Dict[str, torch.Tensor]]:
        """Every token selects its own chapters (router.py:262-340).  Returns (global chapter ids int64
        [B, L, k'], weights [B, L, k'] renormalised over the selection, losses over all B*L routing rows);
        k' = min(top_k, num_chapters - exclude_prefix_chapters), empty tensors when k' <= 0."""
        if hidden_states.dim() != 3:
            raise ValueError(f"hidden_states must be 3D (B, T, D), got shape {tuple(hidden_states.shape)}")
        if exclude_prefix_chapters < 0 or exclude_prefix_chapters > self.num_chapters:
            raise ValueError(
                f"exclude_prefix_chapters must be in [0, {self.num_chapters}], got {exclude_prefix_chapters}")
        return F_moc.route_tokens(hidden_states, self.router.weight, self.router.bias, self.top_k,
                                  exclude_prefix_chapters, return_losses)

    def route_with_shared(self, hidden_states: torch.Tensor, num_shared_chapters: int,
                          routed_scaling_factor: float, return_losses: bool = True):
        """Router plus the model-side shared-prefix step (model.py:356-391) in one launch sequence.
        Returns (indices, weights, combined_indices int32, combined_weights, losses)."""
        return F_moc.route(hidden_states, self.router.weight, self.router.bias, self.top_k,
                           num_shared_chapters, routed_scaling_factor, return_losses)


def compute_total_router_loss(losses: Dict[str, torch.Tensor], load_balance_coef: float = 0.01,
                              auxiliary_coef: float = 0.0, z_loss_coef: float = 0.0,
                              reference_tensor: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Weighted sum of the router losses (router.py:490-527); empty dicts give a zero scalar."""
    if not losses:
        return reference_tensor.new_tensor(0.0) if reference_tensor is not None else torch.tensor(0.0)
    total = next(iter(losses.values())).new_tensor(0.0)
    for key, coef in (("load_balance", load_balance_coef), ("auxiliary", auxiliary_coef), ("z_loss", z_loss_coef)):
        if key in losses and coef > 0:
            total = total + coef * losses[key]
    return total
