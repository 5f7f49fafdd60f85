"""Decode-time memory layer: cached projected bank rows and the rolling routing state.

The reference's generation loop (inference/generate.py:189-274) calls the model once per token; every memory
layer then routes on a pooled state, re-gathers (S+k)*T bank rows per sequence and re-projects them with Wk / Wv
(model.py:624-692, memory_attention.py:241-243).  While decoding, bank and projections are constant, so

``ProjectedBankCache``  holds ``norm(M) [Wk; Wv]^T`` in bf16 ([C*T, 2*HK*D], 805 MB for the 262,208-row bank);
``RoutingWindow``       is the ``rolling`` / ``hybrid`` routing state of model.py:630-660 (last
                        ``routing_window_size`` layer-input states; prefill pools the whole prompt);
``MemoryDecoder``       runs one step: router on the window -> shared prefix -> query projection -> attention
                        over gathered cache rows scaled by the chapter weight -> output projection.

Results equal ``memory_layer`` on the same inputs up to bf16 rounding of the cached rows.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import functional as F_moc
from . import ops


class ProjectedBankCache:
    """K/V projections of every bank row, built once per weight state."""

    def __init__(self, bank: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, tokens_per_chapter: int,
                 num_shared_chapters: int = 1, norm_type: Optional[str] = None, norm_eps: float = 1e-5,
                 chapters_per_pass: int = 512):
        t = int(tokens_per_chapter)
        rows, d = bank.shape
        if rows % t != 0:
            raise ValueError("bank rows must be a multiple of tokens_per_chapter")
        self.tokens_per_chapter = t
        self.num_chapters = rows // t
        self.kv_dim = wk.shape[0]
        # the reference normalises rows only when a shared and a routed slice both exist (model.py:413-418)
        norm = norm_type if 0 < num_shared_chapters < self.num_chapters else None
        cd = torch.bfloat16
        wkv = ops.cast(torch.cat([wk, wv], dim=0).contiguous(), cd)
        self.kv_bank = torch.empty(rows, 2 * self.kv_dim, dtype=cd, device=bank.device)
        with torch.no_grad():
            for c0 in range(0, self.num_chapters, chapters_per_pass):
                c1 = min(self.num_chapters, c0 + chapters_per_pass)
                idx = torch.arange(c0, c1, dtype=torch.int32, device=bank.device).view(1, -1)
                rows_c, _ = ops.gather_rows_fwd(bank, t, idx, None, norm, norm_eps, cd)     # [1, n*T, d], normalised
                ops.gemm(rows_c.view(-1, d), wkv, out=self.kv_bank[c0 * t:c1 * t], tag="kv_cache")


class RoutingWindow:
    """Routing state of one memory layer during cached generation (model.py:630-660).

    ``prefill(h)`` returns the states the router pools for the prompt and keeps the last ``window`` of them;
    ``step(h)`` appends the new states and returns the window to pool.  ``hybrid`` pools the whole prompt at
    prefill; ``rolling`` pools the window from the start.
    """

    def __init__(self, window_size: int = 128, strategy: str = "hybrid"):
        if strategy not in ("rolling", "hybrid"):
            raise ValueError("strategy must be 'rolling' or 'hybrid'")
        self.window_size = int(window_size)
        self.strategy = strategy
        self.cache: Optional[torch.Tensor] = None

    def reset(self) -> None:
        self.cache = None

    def prefill(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if self.strategy == "rolling":
            return self.step(hidden_states)
        self.cache = hidden_states[:, -self.window_size:].detach()
        return hidden_states

    def step(self, hidden_states: torch.Tensor) -> torch.Tensor:
        combined = hidden_states if self.cache is None else torch.cat([self.cache, hidden_states], dim=1)
        if combined.shape[1] > self.window_size:
            combined = combined[:, -self.window_size:]
        self.cache = combined.detach()
        return combined


class MemoryDecoder:
    """One memory layer in generation mode over a :class:`ProjectedBankCache`."""

    def __init__(self, cache: ProjectedBankCache, router_weight: torch.Tensor, router_bias: Optional[torch.Tensor],
                 wq: torch.Tensor, wo: torch.Tensor, *, num_heads: int, num_kv_heads: Optional[int] = None,
                 top_k: int, num_shared_chapters: int = 1, routed_scaling_factor: float = 2.5):
        self.cache = cache
        self.router_weight, self.router_bias = router_weight, router_bias
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads or num_heads)
        self.top_k, self.num_shared = int(top_k), int(num_shared_chapters)
        self.routed_scale = float(routed_scaling_factor)
        cd = torch.bfloat16
        self.wq_c, self.wo_c = ops.cast(wq.contiguous(), cd), ops.cast(wo.contiguous(), cd)
        self.scale = (wq.shape[0] // self.num_heads) ** -0.5

    @torch.no_grad()
    def step(self, hidden_states: torch.Tensor, routing_states: torch.Tensor) -> Tuple[torch.Tensor, dict]:
        """``hidden_states`` [B, n_q, d]: the tokens being decoded (input of the cross attention);
        ``routing_states`` [B, W, d]: the states the router mean-pools (a :class:`RoutingWindow` result).
        Returns (output [B, n_q, d] in the dtype of ``hidden_states``, routing info)."""
        b, n_q, d = hidden_states.shape
        idx, w, cidx, cw, _ = F_moc.route(routing_states, self.router_weight, self.router_bias, self.top_k,
                                          self.num_shared, self.routed_scale, with_losses=False)
        cd = torch.bfloat16
        q = ops.gemm(ops.cast(hidden_states.reshape(b * n_q, d), cd), self.wq_c, tag="q_proj")
        o = ops.decode_attn(q.view(b, n_q, -1), self.cache.kv_bank, cidx, cw, self.num_heads, self.num_kv_heads,
                            self.cache.tokens_per_chapter, self.scale)
        out_dtype = hidden_states.dtype if hidden_states.dtype in (torch.float32, cd) else cd
        out = ops.gemm(o.view(b * n_q, -1), self.wo_c, out_dtype=out_dtype, tag="o_proj")
        return out.view(b, n_q, d).to(hidden_states.dtype), {"indices": idx, "weights": w, "combined_indices": cidx,
                                                              "combined_weights": cw}
