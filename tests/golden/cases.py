"""Seeded parity cases shared by the fixture generator and the tests.

Inputs are drawn from numpy's PCG64 generator, so they can be rebuilt anywhere
without storing them; only the reference's outputs live in the ``.npz`` files.
Distributions follow the benchmark configuration list: hidden states N(0,1),
bank rows / projections / router weight N(0,0.02), router bias 0, output
projection N(0,0.02) instead of the model's zero init so outputs are non-zero.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import numpy as np


@dataclass(frozen=True)
class Case:
    name: str
    batch: int
    seq: int
    hidden_dim: int
    num_heads: int
    num_kv_heads: int
    num_chapters: int            # shared prefix included
    tokens_per_chapter: int
    top_k: int
    num_shared_chapters: int = 1
    routed_scaling_factor: float = 2.5
    norm_type: Optional[str] = None
    norm_eps: float = 1e-5
    seed: int = 1234
    separate_router_input: bool = False
    router_scale: float = 0.02       # std of the router weight
    pre_norm: Optional[str] = None   # "rms" / "layernorm": h + attn(norm(h), memory), the block's memory step
    pre_norm_eps: float = 1e-6
    notes: str = ""
    extra: Dict[str, float] = field(default_factory=dict)


# cfg0 is the CPU-runnable configuration of the benchmark list; the rest vary
# one feature each (normalisation, grouped KV heads, two shared chapters, no
# shared chapter, a separate router input, a sharper router so that the same
# chapter is picked by several batch items).
CASES = {
    c.name: c for c in [
        Case("cfg0", 2, 128, 256, 4, 4, 65, 16, 4),
        Case("rms_norm", 2, 64, 128, 2, 2, 33, 16, 4, norm_type="rms", seed=1235),
        Case("layernorm", 2, 64, 128, 2, 2, 33, 16, 4, norm_type="layernorm", seed=1236),
        Case("gqa", 2, 64, 256, 4, 2, 33, 32, 3, seed=1237),
        Case("two_shared", 3, 48, 128, 2, 2, 34, 16, 5, num_shared_chapters=2, seed=1238),
        Case("no_shared", 2, 64, 128, 2, 2, 32, 16, 4, num_shared_chapters=0, seed=1239),
        Case("split_inputs", 2, 64, 128, 2, 2, 33, 16, 4, separate_router_input=True, seed=1240),
        Case("k_exceeds", 2, 32, 128, 2, 2, 5, 16, 5, seed=1241,
             notes="top_k equals the chapter count, so only k = C - S routed chapters exist"),
        Case("head64_t64", 2, 128, 128, 2, 2, 17, 64, 4, seed=1242,
             notes="tensor-core tile shapes: head_dim 64, 64-row chapters"),
        Case("block_rms", 2, 128, 128, 2, 2, 17, 64, 4, seed=1243, pre_norm="rms",
             notes="memory step of the transformer block: RMSNorm, attention, residual add"),
        Case("block_layernorm", 2, 64, 128, 2, 1, 33, 16, 4, seed=1244, pre_norm="layernorm",
             separate_router_input=True,
             notes="LayerNorm variant of the block's memory step, grouped KV heads, router fed separately"),
        Case("head64_t64_rms", 2, 128, 128, 2, 2, 17, 64, 4, norm_type="rms", seed=1245,
             notes="the paper's setting (per-row RMS normalisation of the gathered rows) at tensor-core tile shapes"),
        Case("head64_t64_ln", 2, 128, 128, 2, 1, 17, 64, 4, norm_type="layernorm", seed=1246,
             notes="affine-free LayerNorm of the gathered rows at tensor-core tile shapes, grouped KV heads"),
    ]
}

# cases whose fixtures also hold the reference's outputs under bf16 autocast (head_dim 64: the tensor-core path)
BF16_CASES = ("head64_t64", "block_rms", "head64_t64_rms", "head64_t64_ln")


def make_inputs(case: Case) -> Dict[str, np.ndarray]:
    """Seeded fp32 inputs and parameters of one case."""
    rng = np.random.Generator(np.random.PCG64(case.seed))
    d = case.hidden_dim
    dkv = case.num_kv_heads * (d // case.num_heads)
    n_rows = case.num_chapters * case.tokens_per_chapter

    def normal(shape, std):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)

    out = {
        "h_router": normal((case.batch, case.seq, d), 1.0),
        "bank": normal((n_rows, d), 0.02),
        "router_w": normal((case.num_chapters, d), case.router_scale),
        "router_b": np.zeros((case.num_chapters,), np.float32),
        "wq": normal((d, d), 0.02),
        "wk": normal((dkv, d), 0.02),
        "wv": normal((dkv, d), 0.02),
        "wo": normal((d, d), 0.02),
    }
    out["h_attn"] = normal((case.batch, case.seq, d), 1.0) if case.separate_router_input else out["h_router"]
    if case.pre_norm is not None:
        g2 = np.random.Generator(np.random.PCG64(case.seed + 555))
        out["pre_norm_w"] = (1.0 + 0.1 * g2.standard_normal((d,), dtype=np.float32)).astype(np.float32)
        out["pre_norm_b"] = (0.1 * g2.standard_normal((d,), dtype=np.float32)).astype(np.float32)
    out["d_out"] = np.random.Generator(np.random.PCG64(case.seed + 999)).standard_normal(
        (case.batch, case.seq, d), dtype=np.float32)
    return out


# token-level routing (every token selects its own chapters; model.py:544-606, memory_attention.py:480-716)
TOKEN_CASES = {
    c.name: c for c in [
        Case("token_t16", 2, 32, 128, 2, 2, 9, 16, 3, seed=1250,
             notes="per-token top-3 of 8 routed chapters of 16 rows plus the shared chapter"),
        Case("token_gqa_rms", 2, 32, 128, 2, 1, 9, 64, 3, norm_type="rms", seed=1251,
             notes="64-row chapters, head_dim 64, grouped KV heads, whole-bank RMS normalisation"),
        Case("token_multi_tile", 1, 256, 128, 2, 2, 5, 64, 2, seed=1252,
             notes="256 tokens x top-2 of 4 routed 64-row chapters: chapters with more than 128 (token, slot) pairs, "
                   "i.e. several tiles per chapter in the tensor-core mixture"),
    ]
}
