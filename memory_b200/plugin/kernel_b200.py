"""Token-routing kernel plugin with the entry points the reference resolves from ``kernels-final/kernel_<v>.py``
(memory_transformer/token_routing_kernel.py:68-69, 96-142):

    FSA_topk_sparse_attention_bthd            joint softmax over the selected chapters of each token
                                              (kernels-final/kernel_v2.py:3181-3203)
    FSA_topk_sparse_attention_weighted_bthd   exact mixture: a softmax per chapter, outputs mixed by the router
                                              weights, gradients for q, k, v and the weights
                                              (kernels-final/kernel_v4.py:1313-1340)

Both take ``[B, T, H, D]`` tensors and per-(token, kv-head) chapter lists and are called by the reference with
keyword arguments (memory_transformer/memory_attention.py:798-816, 831-853).  The reference finds a plugin as a
FILE named ``kernel_v1.py`` ... ``kernel_v5.py`` in its ``kernels-final`` folder; :func:`install_plugin_files`
writes such files (two lines each, re-exporting this module) so that the stock loader picks these kernels up.
"""
from __future__ import annotations

import os
from typing import Optional, Sequence

import torch

from .. import ops
from ..memory_cross_attn import MemoryCrossAttnFunction

# what the weighted entry point computes: every chapter normalised on its own, then mixed (not the
# "joint_bias" approximation of the reference's kernel_v5)
FSA_WEIGHTED_SEMANTICS = "exact_moe"


def _check_bthd(q, k, v, block_size):
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q/k/v must be rank-4 [B,T,H,D].")
    if k.shape != v.shape:
        raise ValueError("k and v must have identical [B,Tk,H,D] shape.")
    if q.shape[0] != k.shape[0]:
        raise ValueError("q and k/v batch size must match.")
    if q.shape[3] != k.shape[3]:
        raise ValueError("q and k/v head dim must match.")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q/k/v dtype must match.")
    if q.shape[2] % k.shape[2] != 0:
        raise ValueError(f"HQ ({q.shape[2]}) must be divisible by HK ({k.shape[2]}) for GQA.")
    if block_size <= 0 or k.shape[1] % block_size != 0:
        raise ValueError(f"Tk ({k.shape[1]}) must be a positive multiple of block_size ({block_size}).")
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor.")


def _kv_head_indices(block_indices, q, k):
    """[B, Tq, HK, S] int32: lists given per query head are read at the first head of each KV group."""
    if block_indices is None:
        raise ValueError("block_indices_bths is required (topk_idx_hns layouts are not part of this plugin).")
    if block_indices.ndim != 4 or tuple(block_indices.shape[:2]) != tuple(q.shape[:2]):
        raise ValueError("block_indices must be [B, Tq, HK or HQ, topk].")
    hq, hk = q.shape[2], k.shape[2]
    if block_indices.shape[2] == hk:
        bi = block_indices
    elif block_indices.shape[2] == hq:
        bi = block_indices[:, :, :: hq // hk]
    else:
        raise ValueError(f"block_indices head axis must be HK ({hk}) or HQ ({hq}).")
    return bi.to(torch.int32).contiguous()


class _WeightedSparseAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, bi, weights, block_size, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        w32 = weights.float().contiguous()
        mix_ws = None
        if ops.token_mix_supported(q, k, block_size, bi.shape[2]):
            o, lse_slots, mix_ws = ops.token_mix_fwd(q, k, v, bi, w32, scale)      # tcgen05, chapter-stationary
        else:
            o, lse_slots = ops.sparse_attn_weighted_fwd(q, k, v, bi, w32, block_size, scale)
        ctx.save_for_backward(q, k, v, bi, w32, lse_slots)
        ctx.cfg = (block_size, scale, weights.dtype, mix_ws)
        return o

    @staticmethod
    def backward(ctx, g):
        q, k, v, bi, w32, lse_slots = ctx.saved_tensors
        block_size, scale, w_dtype, mix_ws = ctx.cfg
        if mix_ws is not None:
            d_k, d_v = torch.empty_like(k), torch.empty_like(v)      # written in full by the kernel
            d_q, d_w = ops.token_mix_bwd(q, k, v, bi, w32, lse_slots, g.contiguous(), scale, 1.0, mix_ws, d_k, d_v)
            return d_q, d_k, d_v, None, d_w.to(w_dtype), None, None
        d_k = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
        d_v = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
        d_q, d_w = ops.sparse_attn_weighted_bwd(q, k, v, bi, w32, lse_slots, g.contiguous(), block_size, scale, 1.0,
                                                d_k, d_v)
        return d_q, d_k.to(k.dtype), d_v.to(v.dtype), None, d_w.to(w_dtype), None, None


def FSA_topk_sparse_attention_bthd(q_bthd, k_bthd, v_bthd, block_indices_bths, block_size: int,
                                   block_weights_bths=None, softmax_scale: Optional[float] = None,
                                   cu_seqlens_q=None, cu_seqlens_k=None, topk_idx_hns=None, topk_w_hns=None,
                                   assume_sorted_topk: bool = False, disable_causal_mask: bool = False):
    """out [B,Tq,HQ,D]: each token attends to the keys of its selected chapters with one softmax.  Memory rows
    have no positions, so the call must disable the causal mask, as the reference's module does."""
    _check_bthd(q_bthd, k_bthd, v_bthd, int(block_size))
    if not disable_causal_mask:
        raise ValueError("memory chapters are position-free: call with disable_causal_mask=True")
    if block_weights_bths is not None or topk_w_hns is not None:
        raise ValueError("per-chapter weights belong to FSA_topk_sparse_attention_weighted_bthd")
    if cu_seqlens_q is not None or cu_seqlens_k is not None or topk_idx_hns is not None:
        raise ValueError("variable-length / pre-transposed index layouts are not part of this plugin")
    bi = _kv_head_indices(block_indices_bths, q_bthd, k_bthd)
    scale = float(softmax_scale) if softmax_scale is not None else q_bthd.shape[-1] ** -0.5
    return MemoryCrossAttnFunction.apply(q_bthd.contiguous(), k_bthd.contiguous(), v_bthd.contiguous(), bi,
                                         int(block_size), scale)


def FSA_topk_sparse_attention_weighted_bthd(q_bthd, k_bthd, v_bthd, block_indices_bths, chapter_weights_bts,
                                            block_size: int, softmax_scale: Optional[float] = None,
                                            cu_seqlens_q=None, cu_seqlens_k=None, topk_idx_hns=None,
                                            assume_sorted_topk: bool = False, disable_causal_mask: bool = False):
    """out [B,Tq,HQ,D] = sum_s w[b,t,s] * softmax(q K_s^T scale) V_s with a softmax per selected chapter;
    differentiable in q, k, v and the weights."""
    _check_bthd(q_bthd, k_bthd, v_bthd, int(block_size))
    if not disable_causal_mask:
        raise ValueError("memory chapters are position-free: call with disable_causal_mask=True")
    if cu_seqlens_q is not None or cu_seqlens_k is not None or topk_idx_hns is not None:
        raise ValueError("variable-length / pre-transposed index layouts are not part of this plugin")
    bi = _kv_head_indices(block_indices_bths, q_bthd, k_bthd)
    if chapter_weights_bts is None or tuple(chapter_weights_bts.shape) != (q_bthd.shape[0], q_bthd.shape[1], bi.shape[-1]):
        raise ValueError("chapter_weights_bts must be [B, Tq, topk]")
    scale = float(softmax_scale) if softmax_scale is not None else q_bthd.shape[-1] ** -0.5
    return _WeightedSparseAttention.apply(q_bthd, k_bthd, v_bthd, bi, chapter_weights_bts, int(block_size), scale)


_STUB = '''"""Token-routing kernels of memory_b200 under the file name the reference's loader looks for."""
from memory_b200.plugin.kernel_b200 import (FSA_WEIGHTED_SEMANTICS, FSA_topk_sparse_attention_bthd,  # noqa: F401
                                            FSA_topk_sparse_attention_weighted_bthd)
'''


def install_plugin_files(kernels_dir: str, versions: Sequence[str] = ("v2", "v4")) -> list:
    """Writes ``kernel_<v>.py`` re-export files into ``kernels_dir`` (the reference's ``kernels-final`` folder, i.e.
    ``Path(memory_transformer.token_routing_kernel.__file__).parents[1] / "kernels-final"``).  Existing files are
    left alone unless they are such re-export files already.  Returns the paths written."""
    os.makedirs(kernels_dir, exist_ok=True)
    written = []
    for v in versions:
        if v not in ("v1", "v2", "v3", "v4", "v5"):
            raise ValueError(f"unknown kernel version {v!r}")
        path = os.path.join(kernels_dir, f"kernel_{v}.py")
        if os.path.exists(path) and "memory_b200.plugin.kernel_b200" not in open(path).read():
            continue
        with open(path, "w") as f:
            f.write(_STUB)
        written.append(path)
    return written
