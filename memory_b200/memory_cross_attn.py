"""``memory_cross_attn`` entry point with the reference's signature and checks
(kernels-final/memory_cross_attn.py:103-112, 1310-1366, 1610-1652)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops


def _check(q, k, v, block_indices, block_size):
    for name, t in (("q", q), ("k", k), ("v", v), ("block_indices", block_indices)):
        if not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor.")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous (expected [B,T,H,D] contiguous). Got strides={t.stride()}.")
    b, tq, hq, kd = q.shape
    bk, tk, h, kk = k.shape
    assert b == bk == v.shape[0], "Batch mismatch"
    assert tk == v.shape[1], "KV length mismatch"
    assert h == v.shape[2], "KV heads mismatch"
    assert kk == kd, "Key dim mismatch"
    assert tuple(block_indices.shape[:3]) == (b, tq, h), "block_indices shape must be [B,TQ,H,S]"
    assert tk % block_size == 0, "TK must be divisible by block_size (chapter size) for clean chapter blocks."
    assert hq % h == 0, "HQ must be multiple of H (GQA grouping)."
    if v.shape[-1] != kd:
        raise ValueError("value head dim must equal key head dim")


def memory_cross_attn_forward(q, k, v, block_indices, block_size: int,
                              scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(o [B,TQ,HQ,D] in v's dtype, lse [B,TQ,HQ] fp32)."""
    _check(q, k, v, block_indices, block_size)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return ops.sparse_attn_fwd(q, k, v, block_indices.to(torch.int32).contiguous(), block_size, scale)


def memory_cross_attn_preprocess_delta(o: torch.Tensor, do: torch.Tensor) -> torch.Tensor:
    """delta[b, t, h] = <o, do> (kernels-final/memory_cross_attn.py:1369-1384); fp32 [B,TQ,HQ]."""
    for name, t in (("o", o), ("do", do)):
        if not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor.")
    assert o.shape == do.shape
    return ops.row_dot(o, do)


def memory_cross_attn_backward(q, k, v, o, lse, do, block_indices, block_size: int, scale: Optional[float] = None,
                               dkv_strategy: str = "b", q_chunk_size: int = 1024, d_chunk_size: int = 256,
                               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dq, dk, dv) in the inputs' dtypes (kernels-final/memory_cross_attn.py:1387-1603).  One backward exists
    here, so ``dkv_strategy`` and the chunk sizes are validated and otherwise unused."""
    if dkv_strategy not in ("a", "b", "c", "d"):
        raise ValueError(f"Unknown dkv_strategy={dkv_strategy}")
    bi = block_indices.to(torch.int32).contiguous()
    _check(q, k, v, bi, block_size)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    dq, dk, dv = ops.sparse_attn_bwd(q, k, v, bi, o, lse, do.contiguous(), block_size, scale)
    return dq, dk.to(k.dtype), dv.to(v.dtype)


class MemoryCrossAttnFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, block_indices, block_size, scale):
        if scale is None:
            scale = q.shape[-1] ** -0.5
        bi = block_indices.to(torch.int32).contiguous()
        _check(q, k, v, bi, block_size)
        o, lse = ops.sparse_attn_fwd(q, k, v, bi, block_size, scale)
        ctx.save_for_backward(q, k, v, o, lse, bi)
        ctx.block_size, ctx.scale = block_size, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, bi = ctx.saved_tensors
        dq, dk, dv = ops.sparse_attn_bwd(q, k, v, bi, o, lse, do.contiguous(), ctx.block_size, ctx.scale)
        return dq, dk.to(k.dtype), dv.to(v.dtype), None, None, None


def memory_cross_attn(q, k, v, block_indices, block_size: int, scale: Optional[float] = None,
                      dkv_strategy: str = "b", q_chunk_size: int = 1024, d_chunk_size: int = 256) -> torch.Tensor:
    """Per-token chapter-sparse attention.  ``dkv_strategy`` / chunk sizes select among the reference's
    Triton backward variants; here one backward exists, so they are validated and otherwise unused."""
    if dkv_strategy not in ("a", "b", "c", "d"):
        raise ValueError(f"Unknown dkv_strategy={dkv_strategy}")
    return MemoryCrossAttnFunction.apply(q, k, v, block_indices, block_size, scale)
