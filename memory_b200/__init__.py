"""memory_b200: Mixture-of-Chapters memory cross-attention on B200 (sm_100a).

The operators exist only as CUDA kernels behind ``libmoc_b200.so``; build it with
``python -m memory_b200.build``.  Public surface mirrors the reference's ``memory_transformer``
modules for this path.
"""
from .decode import MemoryDecoder, ProjectedBankCache, RoutingWindow
from .functional import (SparseBankGrad, cross_attention, gather_chapters, memory_layer, route, route_tokens,
                         token_routed_attention, token_routed_attention_joint)
from .memory_attention import MemoryCrossAttention
from .memory_block import MemorySubBlock, RMSNorm
from .memory_bank import ChapteredMemoryBank, StandardMemoryBank
from .memory_cross_attn import (memory_cross_attn, memory_cross_attn_backward, memory_cross_attn_forward,
                                memory_cross_attn_preprocess_delta)
from .optim import SparseBankAdamW
from .router import ChapterRouter, compute_total_router_loss

__all__ = [
    "ChapterRouter", "compute_total_router_loss", "StandardMemoryBank", "ChapteredMemoryBank",
    "MemoryCrossAttention", "MemoryDecoder", "ProjectedBankCache", "RoutingWindow", "MemorySubBlock", "RMSNorm", "memory_cross_attn", "memory_cross_attn_forward", "memory_layer", "route",
    "gather_chapters", "cross_attention", "SparseBankGrad", "SparseBankAdamW", "route_tokens", "token_routed_attention",
    "token_routed_attention_joint", "memory_cross_attn_backward", "memory_cross_attn_preprocess_delta",
]
