"""Optimizer step of the memory bank from the compact gradient the backward pass produces.

The reference hands the bank to ``torch.optim.AdamW`` as its own parameter group (training/trainer.py:338-347,
372-378) and feeds it the dense 262,208 x 768 gradient of ``torch.gather``'s backward.  ``SparseBankAdamW`` applies
the identical update -- every row, bias-corrected moments, decoupled weight decay -- straight from a
``SparseBankGrad`` (chapter ids + rows), in one kernel pass, and can refresh the bf16 working copy of the bank in
the same pass.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops
from .functional import SparseBankGrad


class SparseBankAdamW:
    """AdamW for one bank parameter ([rows, d] fp32) driven by compact gradients.

    ``step(grad)`` takes the ``SparseBankGrad`` a backward pass (or ``GradReducer``) filled; its ``scale`` and the
    optional ``grad_scale`` (e.g. a clipping coefficient) multiply the gradient.  ``state_dict`` / ``load_state_dict``
    use torch.optim.AdamW's per-parameter keys (``step``, ``exp_avg``, ``exp_avg_sq``), so optimizer state moves
    between the two."""

    def __init__(self, param: torch.Tensor, tokens_per_chapter: int, lr: float = 1e-4,
                 betas: Tuple[float, float] = (0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.01,
                 shadow: Optional[torch.Tensor] = None):
        if param.dtype != torch.float32 or param.dim() != 2 or not param.is_contiguous():
            raise TypeError("the bank parameter must be a contiguous fp32 [rows, d] tensor")
        if param.shape[0] % int(tokens_per_chapter) != 0:
            raise ValueError("bank rows must be a whole number of chapters")
        self.param = param
        self.t = int(tokens_per_chapter)
        self.lr, self.betas, self.eps, self.weight_decay = float(lr), tuple(betas), float(eps), float(weight_decay)
        self.exp_avg = torch.zeros_like(param, memory_format=torch.contiguous_format)
        self.exp_avg_sq = torch.zeros_like(param, memory_format=torch.contiguous_format)
        self.step_count = 0
        self.shadow = shadow       # bf16 [rows, d] refreshed by every step, or None
        self._ws = None

    @torch.no_grad()
    def step(self, grad: SparseBankGrad, grad_scale: float = 1.0, lr: Optional[float] = None) -> None:
        if len(grad.entries) != 1:
            raise NotImplementedError(
                "one compact entry per step: sum several layers' entries first (ops.bank_grad_merge)")
        uniq, num_unique, rows, t = grad.entries[0]
        if t != self.t:
            raise ValueError("gradient rows were produced with a different chapter size")
        self.step_count += 1
        if self._ws is None:
            self._ws = torch.empty(4 * (self.param.shape[0] // self.t), dtype=torch.uint8, device=self.param.device)
        ops.bank_adamw_step(self.param.data, self.exp_avg, self.exp_avg_sq, uniq, num_unique,
                            rows if rows.dtype == torch.float32 else rows.float(), self.t,
                            lr=self.lr if lr is None else lr, betas=self.betas, eps=self.eps,
                            weight_decay=self.weight_decay, step=self.step_count,
                            grad_scale=float(grad.scale) * float(grad_scale), shadow=self.shadow, workspace=self._ws)

    def grad_sqnorm(self, grad: SparseBankGrad) -> torch.Tensor:
        """Squared L2 norm of the (scaled) bank gradient as a [1] tensor: the bank's term of a global clip norm."""
        uniq, num_unique, rows, t = grad.entries[0]
        return ops.rows_sqnorm(rows if rows.dtype == torch.float32 else rows.float(), num_unique, t) * (grad.scale ** 2)

    def state_dict(self):
        return {"step": torch.tensor(float(self.step_count)), "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq}

    def load_state_dict(self, state) -> None:
        self.step_count = int(state["step"])
        self.exp_avg.copy_(state["exp_avg"])
        self.exp_avg_sq.copy_(state["exp_avg_sq"])
