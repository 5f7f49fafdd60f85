"""Memory bank modules with the reference's names and parameter keys
(memory_transformer/memory_bank.py:45-76, 176-293)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import functional as F_moc
from . import ops


class StandardMemoryBank(nn.Module):
    """N learnable rows of width ``dim`` (parameter name ``memory``, N(0, init_std))."""

    def __init__(self, num_tokens: int, dim: int, init_std: float = 0.02):
        super().__init__()
        self.num_tokens = num_tokens
        self.dim = dim
        self.init_std = init_std
        self.memory = nn.Parameter(torch.empty(num_tokens, dim))
        nn.init.normal_(self.memory, mean=0.0, std=init_std)

    def get_memory(self) -> torch.Tensor:
        return self.memory

    def forward(self) -> torch.Tensor:
        return self.get_memory()


class ChapteredMemoryBank(nn.Module):
    """Chapter view of a bank: chapter c is rows [c*T, (c+1)*T)."""

    def __init__(self, base_bank: nn.Module, num_chapters: int):
        super().__init__()
        if num_chapters <= 0:
            raise ValueError(f"num_chapters must be > 0, got {num_chapters}")
        if base_bank.num_tokens % num_chapters != 0:
            raise ValueError(
                f"num_tokens ({base_bank.num_tokens}) must be divisible by num_chapters ({num_chapters})")
        self.base_bank = base_bank
        self.num_chapters = num_chapters
        self.tokens_per_chapter = base_bank.num_tokens // num_chapters
        self._bf16_shadow: Optional[torch.Tensor] = None
        self._bf16_version = -1
        self._inv_rms: Optional[torch.Tensor] = None
        self._inv_rms_key = None

    def get_memory(self) -> torch.Tensor:
        return self.base_bank.get_memory()

    def get_chapter(self, chapter_idx: int) -> torch.Tensor:
        t = self.tokens_per_chapter
        return self.get_memory()[chapter_idx * t:(chapter_idx + 1) * t]

    def get_chapters_batched(self, chapter_indices: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """(rows [B, K*T, d], flat row ids [B, K*T]) of the selected chapters; the gradient of the
        rows is scattered only into the touched chapters."""
        memory = self.get_memory()
        rows = F_moc.gather_chapters(memory, chapter_indices, None, self.tokens_per_chapter)
        t = self.tokens_per_chapter
        flat = (chapter_indices.long().unsqueeze(-1) * t
                + torch.arange(t, device=chapter_indices.device).view(1, 1, -1)).view(chapter_indices.shape[0], -1)
        return rows, flat

    def bf16_shadow(self) -> torch.Tensor:
        """bf16 copy of the bank for the TMA-gather projection; refreshed when the parameter changed."""
        memory = self.get_memory()
        if memory.dtype == torch.bfloat16:
            return memory.detach()
        if self._bf16_shadow is None or self._bf16_version != memory._version:
            self._bf16_shadow = ops.cast(memory.detach(), torch.bfloat16)
            self._bf16_version = memory._version
        return self._bf16_shadow

    def row_inv_rms(self, eps: float) -> torch.Tensor:
        """1 / sqrt(mean(row^2) + eps) of every bank row (model.py:423-425 applied to the whole bank), the second
        operand of the fused gather-and-project route under RMS row normalisation; refreshed when the parameter
        changed."""
        memory = self.get_memory()
        key = (memory._version, float(eps))
        if self._inv_rms is None or self._inv_rms_key != key:
            self._inv_rms = ops.row_inv_rms(memory.detach(), eps)
            self._inv_rms_key = key
        return self._inv_rms
