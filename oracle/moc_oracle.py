"""CPU oracle for the Mixture-of-Chapters memory cross-attention path.

TEST INFRASTRUCTURE ONLY.  This file restates, in plain eager torch-on-CPU, the
arithmetic of the reference's sequence-level memory layer so that the CUDA
product can be checked against it.  Nothing in the shipped package imports it;
only the test-suite, the smoke check and the benchmark's CPU-baseline leg do.

Parity pin: every function below is checked against outputs of the reference's
own modules (``memory_transformer.router.ChapterRouter``,
``memory_transformer.memory_bank.ChapteredMemoryBank``,
``memory_transformer.memory_attention.MemoryCrossAttention`` and the static
helpers of ``memory_transformer.model.MemoryTransformer``) stored as fixtures
under ``tests/golden/`` together with the script that produced them.

Each function cites the reference file:line it follows (paths relative to the
reference project root).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------
# configuration of one memory layer
# --------------------------------------------------------------------------
@dataclass
class LayerShape:
    """Static description of one memory layer (names follow the reference's
    ``MemoryConfig``: memory_transformer/config.py)."""

    hidden_dim: int
    num_heads: int
    num_kv_heads: int
    num_chapters: int          # includes the shared prefix chapters
    tokens_per_chapter: int
    top_k: int
    num_shared_chapters: int = 1
    routed_scaling_factor: float = 2.5
    norm_type: Optional[str] = None   # None | "rms" | "layernorm"
    norm_eps: float = 1e-5
    pre_norm: Optional[str] = None    # None | "rms" | "layernorm": out = h + attn(pre_norm(h), memory)
    pre_norm_eps: float = 1e-6

    @property
    def head_dim(self) -> int:
        return self.hidden_dim // self.num_heads

    @property
    def num_memory_tokens(self) -> int:
        return self.num_chapters * self.tokens_per_chapter


# --------------------------------------------------------------------------
# router
# --------------------------------------------------------------------------
def topk_lower_index_first(probs: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k by (value descending, index ascending).

    The reference calls ``torch.topk`` (router.py:143); its tie order is
    implementation defined, so the oracle fixes the total order the CUDA
    router implements: a stable descending sort keeps the lower index first
    among equal values.
    """
    vals, idx = torch.sort(probs, dim=-1, descending=True, stable=True)
    return vals[..., :k], idx[..., :k]


def router_pool(hidden_states: torch.Tensor) -> torch.Tensor:
    """Mean over the sequence axis (router.py:98), fp32."""
    return hidden_states.float().mean(dim=1)


def router_pool_rolling(hidden_states: torch.Tensor, rolling_window_size: Optional[int] = None) -> torch.Tensor:
    """Mean over t of the rolling-window means mean(h[max(0, t-w+1) .. t]) (router.py:159-195), by prefix sums
    as the reference does."""
    h = hidden_states.float()
    batch, seq, dim = h.shape
    window = seq if rolling_window_size is None else int(rolling_window_size)
    if window <= 0:
        raise ValueError(f"rolling_window_size must be > 0, got {rolling_window_size}")   # router.py:179-180
    window = min(window, seq)
    csum = torch.cat([h.new_zeros((batch, 1, dim)), h.cumsum(dim=1)], dim=1)             # router.py:184-186
    end = torch.arange(seq) + 1
    start = torch.clamp(end - window, min=0)                                             # router.py:188-190
    sums = csum[:, end, :] - csum[:, start, :]                                           # router.py:192
    return (sums / (end - start).to(h.dtype).view(1, seq, 1)).mean(dim=1)                # router.py:193-195


def router_forward(
    hidden_states: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor,
    top_k: int,
    exclude_prefix_chapters: int = 0,
    return_losses: bool = True,
    routing_strategy: str = "sequence",
    rolling_window_size: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor, Dict[str, torch.Tensor], Dict[str, torch.Tensor]]:
    """Sequence-level routing (router.py:94-156); ``routing_strategy`` "sequence" or "sequence-rolling"
    (router.py:96-105).

    Returns (indices (B,k') int64, weights (B,k'), losses, internals).
    """
    num_chapters = weight.shape[0]
    if exclude_prefix_chapters < 0 or exclude_prefix_chapters > num_chapters:
        raise ValueError("exclude_prefix_chapters out of range")        # router.py:117-121
    if routing_strategy in ("sequence-rolling", "sequence_rolling"):
        pooled = router_pool_rolling(hidden_states, rolling_window_size) # router.py:100-104
    else:
        pooled = router_pool(hidden_states)                              # router.py:98
    logits = pooled @ weight.float().t() + bias.float()                  # router.py:99
    probs = F.softmax(logits, dim=-1)                                    # router.py:115
    batch = hidden_states.shape[0]
    if exclude_prefix_chapters > 0:
        select_k = min(int(top_k), num_chapters - exclude_prefix_chapters)
        if select_k <= 0:                                                # router.py:126-137
            idx = torch.empty((batch, 0), dtype=torch.long)
            w = torch.empty((batch, 0), dtype=probs.dtype)
        else:
            masked = probs.clone()                                       # router.py:139-142
            masked[:, :exclude_prefix_chapters] = 0.0
            masked = masked / masked.sum(dim=-1, keepdim=True).clamp_min(1e-12)
            w, idx = topk_lower_index_first(masked, select_k)            # router.py:143
            w = w / w.sum(dim=-1, keepdim=True).clamp_min(1e-12)         # router.py:144
    else:
        w, idx = topk_lower_index_first(probs, int(top_k))               # router.py:146-149
        w = w / w.sum(dim=-1, keepdim=True).clamp_min(1e-12)
    losses: Dict[str, torch.Tensor] = {}
    if return_losses:
        losses = router_losses(logits, probs, idx)
    return idx, w, losses, {"pooled": pooled, "logits": logits, "probs": probs}


def router_losses(logits: torch.Tensor, probs: torch.Tensor, selected: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Auxiliary router losses (router.py:197-260)."""
    num_chapters = probs.shape[-1]
    one_hot = F.one_hot(selected, num_classes=num_chapters).float()      # router.py:225-228
    f = one_hot.sum(dim=1).mean(dim=0)                                   # router.py:231 (no grad)
    p_mean = probs.mean(dim=0)                                           # router.py:234
    out = {"load_balance": num_chapters * (f * p_mean).sum()}            # router.py:237
    p_sq = probs.pow(2).mean(dim=0)                                      # router.py:244
    out["auxiliary"] = F.mse_loss(p_sq, torch.ones_like(p_sq) / num_chapters)   # router.py:245-247
    lse = torch.logsumexp(logits, dim=-1)                                # router.py:251
    out["z_loss"] = (lse ** 2).mean()                                    # router.py:252
    out["entropy"] = -(probs * torch.log(probs.clamp_min(1e-12))).sum(dim=-1).mean()  # router.py:257
    return out


def total_router_loss(losses: Dict[str, torch.Tensor], load_balance_coef: float = 0.01,
                      auxiliary_coef: float = 0.0, z_loss_coef: float = 0.0) -> torch.Tensor:
    """Weighted sum of the auxiliary losses (router.py:490-527)."""
    if not losses:
        return torch.tensor(0.0)
    total = next(iter(losses.values())).new_tensor(0.0)
    if "load_balance" in losses and load_balance_coef > 0:
        total = total + load_balance_coef * losses["load_balance"]
    if "auxiliary" in losses and auxiliary_coef > 0:
        total = total + auxiliary_coef * losses["auxiliary"]
    if "z_loss" in losses and z_loss_coef > 0:
        total = total + z_loss_coef * losses["z_loss"]
    return total


def route_token_level(
    hidden_states: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
    top_k: int, exclude_prefix_chapters: int = 0, return_losses: bool = False,
):
    """Per-token routing (router.py:262-340): global chapter ids and weights; with ``return_losses`` also the
    loss dict over all B*L routing rows (router.py:333-338)."""
    num_chapters = weight.shape[0]
    logits = hidden_states.float() @ weight.float().t() + bias.float()   # router.py:294
    probs = F.softmax(logits, dim=-1)                                    # router.py:295
    select_k = min(int(top_k), num_chapters - exclude_prefix_chapters)
    routed = probs[..., exclude_prefix_chapters:]                        # router.py:322
    routed = routed / routed.sum(dim=-1, keepdim=True).clamp_min(1e-12)
    w, idx_local = topk_lower_index_first(routed, select_k)              # router.py:324-328
    w = w / w.sum(dim=-1, keepdim=True).clamp_min(1e-12)                 # router.py:329
    idx = idx_local + int(exclude_prefix_chapters)                       # router.py:330
    if not return_losses:
        return idx, w
    losses = router_losses(logits.reshape(-1, num_chapters), probs.reshape(-1, num_chapters),
                           idx.reshape(-1, select_k))                    # router.py:333-338
    return idx, w, losses


# --------------------------------------------------------------------------
# model-side glue between router and attention
# --------------------------------------------------------------------------
def prepend_shared_chapters(idx: torch.Tensor, w: torch.Tensor, num_chapters: int,
                            num_shared: int, routed_scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Always-on shared chapters in front, routed weights scaled, renormalised
    (model.py:356-391)."""
    shared = max(0, min(int(num_shared), int(num_chapters)))
    if shared <= 0:
        return idx, w
    batch = idx.shape[0]
    shared_idx = torch.arange(shared, dtype=torch.long).unsqueeze(0).expand(batch, -1)
    shared_w = torch.ones((batch, shared), dtype=w.dtype)
    if idx.shape[1] > 0:
        comb_idx = torch.cat([shared_idx, idx], dim=-1)
        comb_w = torch.cat([shared_w, w * float(routed_scale)], dim=-1)
    else:
        comb_idx, comb_w = shared_idx, shared_w
    comb_w = comb_w / comb_w.sum(dim=-1, keepdim=True).clamp_min(1e-12)
    return comb_idx, comb_w


def gather_chapters(bank: torch.Tensor, chapter_idx: torch.Tensor, tokens_per_chapter: int) -> torch.Tensor:
    """Rows [c*T, (c+1)*T) of every selected chapter c, per batch item
    (memory_bank.py:263-293)."""
    batch, k = chapter_idx.shape
    rows = (chapter_idx.unsqueeze(-1) * tokens_per_chapter
            + torch.arange(tokens_per_chapter).view(1, 1, -1)).reshape(batch, -1)   # memory_bank.py:279-282
    return bank[rows]                                                                # == torch.gather at :291


def normalize_memory_rows(memory: torch.Tensor, num_shared: int, tokens_per_chapter: int,
                          norm_type: str, eps: float) -> torch.Tensor:
    """Per-row normalisation of the shared and routed slices (model.py:393-432)."""
    shared_tokens = min(max(0, int(num_shared)) * int(tokens_per_chapter), memory.shape[1])
    if tokens_per_chapter <= 0 or shared_tokens <= 0 or shared_tokens >= memory.shape[1]:
        return memory                                                    # model.py:413-418
    if norm_type == "rms":
        return memory / memory.pow(2).mean(dim=-1, keepdim=True).add(eps).sqrt()      # model.py:423-425
    if norm_type == "layernorm":
        return F.layer_norm(memory, (memory.shape[-1],), eps=eps)                     # model.py:426-428
    raise ValueError(f"Unsupported norm_type: {norm_type}")


def scale_memory(memory: torch.Tensor, comb_w: torch.Tensor, tokens_per_chapter: int) -> torch.Tensor:
    """Every row of chapter slot s is multiplied by that slot's weight (model.py:689-692)."""
    w = comb_w.unsqueeze(-1).repeat(1, 1, tokens_per_chapter).reshape(memory.shape[0], -1, 1)
    return memory * w


# --------------------------------------------------------------------------
# cross attention
# --------------------------------------------------------------------------
def cross_attention(hidden_states: torch.Tensor, memory: torch.Tensor,
                    wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, wo: torch.Tensor,
                    num_heads: int, num_kv_heads: int) -> torch.Tensor:
    """Eager joint-softmax cross attention over already gathered and scaled
    memory rows (memory_attention.py:209-261, 298-316, 452-478)."""
    batch, seq, hidden = hidden_states.shape
    if memory.dim() == 2:                                                # memory_attention.py:228-230
        memory = memory.unsqueeze(0).expand(batch, -1, -1)
    head_dim = hidden // num_heads
    q = F.linear(hidden_states, wq).view(batch, seq, num_heads, head_dim)            # :241,253
    k = F.linear(memory, wk).view(batch, memory.shape[1], num_kv_heads, head_dim)    # :242,256
    v = F.linear(memory, wv).view(batch, memory.shape[1], num_kv_heads, head_dim)    # :243,257
    groups = num_heads // num_kv_heads
    if groups > 1:                                                       # memory_attention.py:263-267
        k = k.repeat_interleave(groups, dim=2)
        v = v.repeat_interleave(groups, dim=2)
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    scores = torch.matmul(q, k.transpose(-2, -1)) * (head_dim ** -0.5)   # :308
    attn = F.softmax(scores, dim=-1)                                     # :309
    ctx = torch.matmul(attn, v).transpose(1, 2).reshape(batch, seq, hidden)   # :313-316, 470-476
    return F.linear(ctx, wo)                                             # :456


def sparse_chapter_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                             block_indices: torch.Tensor, block_size: int,
                             scale: Optional[float] = None) -> torch.Tensor:
    """Per-token joint softmax over the keys of the selected chapters: the
    contract of ``memory_cross_attn`` (kernels-final/memory_cross_attn.py:1310-1366,
    1639-1652).  q [B,TQ,HQ,D], k/v [B,TK,H,D], block_indices [B,TQ,H,S]."""
    bsz, tq, hq, d = q.shape
    h = k.shape[2]
    g = hq // h
    if scale is None:
        scale = d ** -0.5
    offs = torch.arange(block_size)
    out = torch.zeros(bsz, tq, hq, v.shape[-1], dtype=torch.float32)
    for b in range(bsz):
        for kh in range(h):
            rows = (block_indices[b, :, kh, :].long().unsqueeze(-1) * block_size + offs).reshape(tq, -1)
            kk = k[b, :, kh, :].float()[rows]       # [TQ, S*T, D]
            vv = v[b, :, kh, :].float()[rows]
            for gi in range(g):
                qh = kh * g + gi
                s = (q[b, :, qh, :].float().unsqueeze(1) * kk).sum(-1) * scale
                p = F.softmax(s, dim=-1)
                out[b, :, qh, :] = (p.unsqueeze(-1) * vv).sum(1)
    return out.to(v.dtype)


def attention_heads(hidden_states: torch.Tensor, memory: torch.Tensor, wq, wk, wv,
                    num_heads: int, num_kv_heads: int) -> torch.Tensor:
    """``MemoryCrossAttention._forward_attention`` (memory_attention.py:458-478): joint-softmax attention over the
    given rows, heads concatenated, BEFORE the output projection."""
    batch, seq, hidden = hidden_states.shape
    if memory.dim() == 2:
        memory = memory.unsqueeze(0).expand(batch, -1, -1)
    head_dim = hidden // num_heads
    q = F.linear(hidden_states, wq).view(batch, seq, num_heads, head_dim).transpose(1, 2)
    k = F.linear(memory, wk).view(batch, -1, num_kv_heads, head_dim)
    v = F.linear(memory, wv).view(batch, -1, num_kv_heads, head_dim)
    g = num_heads // num_kv_heads
    k = k.repeat_interleave(g, dim=2).transpose(1, 2)
    v = v.repeat_interleave(g, dim=2).transpose(1, 2)
    attn = F.softmax(torch.matmul(q, k.transpose(-2, -1)) * (head_dim ** -0.5), dim=-1)
    return torch.matmul(attn, v).transpose(1, 2).reshape(batch, seq, hidden)


def weighted_chapter_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, block_indices: torch.Tensor,
                               weights: Optional[torch.Tensor], block_size: int, scale: Optional[float] = None,
                               chunk: int = 256) -> torch.Tensor:
    """The exact mixture rule (kernels-final/kernel_v4.py:298-407; memory_attention.py:667-686 with the emulated
    per-chapter call :856-898): out[b,t] = sum_s w[b,t,s] * softmax(q K_s^T scale) V_s, one softmax per chapter.
    q [B,TQ,HQ,D], k/v [B,TK,H,D], block_indices [B,TQ,H,S], weights [B,TQ,S] (None = all ones)."""
    bsz, tq, hq, d = q.shape
    h = k.shape[2]
    g = hq // h
    if scale is None:
        scale = d ** -0.5
    offs = torch.arange(block_size)
    outs = []
    for b in range(bsz):
        per_b = []
        for t0 in range(0, tq, chunk):
            t1 = min(tq, t0 + chunk)
            acc = []
            for kh in range(h):
                bi = block_indices[b, t0:t1, kh, :].long()                               # [n, S]
                rows = bi.unsqueeze(-1) * block_size + offs                             # [n, S, T]
                kk = k[b, :, kh, :].float()[rows]                                       # [n, S, T, D]
                vv = v[b, :, kh, :].float()[rows]
                qq = q[b, t0:t1, kh * g:(kh + 1) * g, :].float()                        # [n, g, D]
                sc = torch.einsum("ngd,nstd->ngst", qq, kk) * scale
                p = F.softmax(sc, dim=-1)                                               # per chapter
                o = torch.einsum("ngst,nstd->ngsd", p, vv)                              # [n, g, S, D]
                if weights is not None:
                    o = o * weights[b, t0:t1].float().view(t1 - t0, 1, -1, 1)
                acc.append(o.sum(dim=2))                                                # [n, g, D]
            per_b.append(torch.cat(acc, dim=1))                                         # [n, HQ, D]
        outs.append(torch.cat(per_b, dim=0))
    return torch.stack(outs, dim=0)


def token_routed_attention(hidden_states, shared_memory, routed_memory, idx_local, weights, tokens_per_chapter: int,
                           routed_scale: float, wq, wk, wv, wo, num_heads: int, num_kv_heads: int) -> torch.Tensor:
    """``MemoryCrossAttention.forward(token_routing_state=...)`` with chapter weights
    (memory_attention.py:352-400, 480-716, 452-456): dense attention over the shared rows, plus routed_scale times
    the weighted mixture of per-chapter attentions over each token's own chapters, then the output projection.
    ``idx_local`` are chapter ids inside ``routed_memory`` (model.py:583-595)."""
    batch, seq, hidden = hidden_states.shape
    head_dim = hidden // num_heads
    combined = hidden_states.new_zeros(batch, seq, hidden).float()
    if shared_memory is not None and shared_memory.numel() > 0:                          # :550-551
        combined = combined + attention_heads(hidden_states, shared_memory, wq, wk, wv, num_heads, num_kv_heads)
    if routed_memory is not None and routed_memory.numel() > 0 and idx_local.shape[-1] > 0:
        q = F.linear(hidden_states, wq).view(batch, seq, num_heads, head_dim)           # :560
        rm = routed_memory.unsqueeze(0).expand(batch, -1, -1)
        k = F.linear(rm, wk).view(batch, -1, num_kv_heads, head_dim)
        v = F.linear(rm, wv).view(batch, -1, num_kv_heads, head_dim)
        bi = idx_local.unsqueeze(2).expand(batch, seq, num_kv_heads, idx_local.shape[-1])
        routed = weighted_chapter_attention(q, k, v, bi, weights, tokens_per_chapter, head_dim ** -0.5)
        combined = combined + routed.reshape(batch, seq, hidden) * float(routed_scale)   # :707-714
    return F.linear(combined, wo)                                                        # :456


def token_memory_layer(shape: "LayerShape", h_router, h_attn, bank, router_w, router_b, wq, wk, wv, wo,
                       return_losses: bool = True) -> Dict[str, torch.Tensor]:
    """Token-level branch of the model's memory layer (model.py:544-606): per-token routing, bank split into
    shared / routed rows (normalised over the whole bank when configured), token-routed attention."""
    s, t = shape.num_shared_chapters, shape.tokens_per_chapter
    r = route_token_level(h_router, router_w, router_b, shape.top_k, s, return_losses)
    idx, w = r[0], r[1]
    losses = r[2] if return_losses else {}
    shared_tokens = s * t
    shared = bank[:shared_tokens] if shared_tokens > 0 else None                         # model.py:551-563
    routed = bank[shared_tokens:] if shared_tokens < bank.shape[0] else None
    if shape.norm_type is not None and shared is not None and routed is not None:        # model.py:565-581
        merged = normalize_memory_rows(torch.cat([shared, routed], dim=0).unsqueeze(0), s, t, shape.norm_type,
                                       shape.norm_eps).squeeze(0)
        shared, routed = merged[:shared_tokens], merged[shared_tokens:]
    out = token_routed_attention(h_attn, shared, routed, idx - s, w, t, shape.routed_scaling_factor,
                                 wq, wk, wv, wo, shape.num_heads, shape.num_kv_heads)
    return {"out": out, "indices": idx, "weights": w, "losses": losses}


def token_memory_layer_fwd_bwd(shape: "LayerShape", tensors: Dict[str, torch.Tensor], d_out: torch.Tensor,
                               load_balance_coef: float = 0.01, z_loss_coef: float = 0.001) -> Dict[str, torch.Tensor]:
    """Forward + autograd backward of ``(out * d_out).sum() + router loss`` for the token-level layer."""
    names = ["h_router", "bank", "router_w", "router_b", "wq", "wk", "wv", "wo"]
    leaves = {n: tensors[n].detach().clone().float().requires_grad_(True) for n in names}
    res = token_memory_layer(shape, leaves["h_router"], leaves["h_router"], leaves["bank"], leaves["router_w"],
                             leaves["router_b"], leaves["wq"], leaves["wk"], leaves["wv"], leaves["wo"])
    loss = (res["out"].float() * d_out.float()).sum() + total_router_loss(res["losses"], load_balance_coef, 0.0,
                                                                            z_loss_coef)
    loss.backward()
    out = {"out": res["out"].detach(), "indices": res["indices"], "weights": res["weights"].detach(),
           "losses": {k: v.detach() for k, v in res["losses"].items()}, "loss": loss.detach()}
    for n in names:
        out["d_" + n] = leaves[n].grad.detach() if leaves[n].grad is not None else torch.zeros_like(leaves[n])
    return out


# --------------------------------------------------------------------------
# the whole layer (sequence-level routing) and its gradients
# --------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm of the transformer blocks (memory_block.py:26-28): x / sqrt(mean(x^2) + eps) * weight."""
    rms = torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x / rms * weight


def block_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], kind: str,
               eps: float = 1e-6) -> torch.Tensor:
    """``norm_cls`` of a block (memory_block.py:448): RMSNorm when use_rms_norm else torch.nn.LayerNorm."""
    if kind in ("rms", "rmsnorm"):
        return rms_norm(x, weight, eps)
    if kind in ("layernorm", "layer"):
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)
    raise ValueError(f"unknown norm kind {kind!r}")


def memory_sub_block(hidden_states: torch.Tensor, memory: torch.Tensor, norm_weight: torch.Tensor,
                     norm_bias: Optional[torch.Tensor], norm_kind: str, norm_eps: float,
                     wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, wo: torch.Tensor,
                     num_heads: int, num_kv_heads: int) -> torch.Tensor:
    """The memory step of MemoryTransformerBlock.forward (memory_block.py:549-558 and 576-586):
    residual = h; h = memory_layernorm(h); h = residual + memory_attn(h, memory)."""
    normed = block_norm(hidden_states, norm_weight, norm_bias, norm_kind, norm_eps)
    return hidden_states + cross_attention(normed, memory, wq, wk, wv, wo, num_heads, num_kv_heads)


def memory_layer(
    shape: LayerShape,
    h_router: torch.Tensor, h_attn: torch.Tensor, bank: torch.Tensor,
    router_w: torch.Tensor, router_b: torch.Tensor,
    wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, wo: torch.Tensor,
    return_losses: bool = True, autocast_bf16: bool = False,
    pre_norm_w: Optional[torch.Tensor] = None, pre_norm_b: Optional[torch.Tensor] = None,
) -> Dict[str, torch.Tensor]:
    """Router -> shared prefix -> gather -> (norm) -> weight -> cross attention
    (model.py:624-692 followed by memory_block.py:549-558).  With ``shape.pre_norm`` the attention is
    wrapped as the block's memory step, h + attn(norm(h), memory).  With
    ``autocast_bf16`` the attention part runs under CPU bf16 autocast while the
    router stays in fp32, the arrangement the paper-shape configuration asks for."""
    idx, w, losses, internals = router_forward(
        h_router, router_w, router_b, shape.top_k,
        exclude_prefix_chapters=shape.num_shared_chapters, return_losses=return_losses)
    comb_idx, comb_w = prepend_shared_chapters(
        idx, w, shape.num_chapters, shape.num_shared_chapters, shape.routed_scaling_factor)
    memory = gather_chapters(bank, comb_idx, shape.tokens_per_chapter)
    if shape.norm_type is not None:
        memory = normalize_memory_rows(memory, shape.num_shared_chapters, shape.tokens_per_chapter,
                                       shape.norm_type, shape.norm_eps)
    memory = scale_memory(memory, comb_w, shape.tokens_per_chapter)
    def memory_step():
        if shape.pre_norm is None:
            return cross_attention(h_attn, memory, wq, wk, wv, wo, shape.num_heads, shape.num_kv_heads)
        return memory_sub_block(h_attn, memory, pre_norm_w, pre_norm_b, shape.pre_norm, shape.pre_norm_eps,
                                wq, wk, wv, wo, shape.num_heads, shape.num_kv_heads)

    if autocast_bf16:
        with torch.autocast(device_type="cpu", dtype=torch.bfloat16):
            out = memory_step()
    else:
        out = memory_step()
    return {"out": out, "indices": idx, "weights": w, "combined_indices": comb_idx,
            "combined_weights": comb_w, "losses": losses, **internals}


def memory_layer_fwd_bwd(
    shape: LayerShape, tensors: Dict[str, torch.Tensor], d_out: torch.Tensor,
    load_balance_coef: float = 0.01, z_loss_coef: float = 0.001, auxiliary_coef: float = 0.0,
    autocast_bf16: bool = False,
) -> Dict[str, torch.Tensor]:
    """Forward plus autograd backward of ``(out * d_out).sum() + router loss``;
    the loss form mirrors the reference's kernel correctness harness
    (kernels-final/benchmark_kernels_final.py:721-728) with the router terms of
    model.py:776-806 added.  ``tensors`` holds h_router, h_attn, bank, router_w,
    router_b, wq, wk, wv, wo.  Returns outputs and one gradient per input."""
    names = ["h_router", "h_attn", "bank", "router_w", "router_b", "wq", "wk", "wv", "wo"]
    if shape.pre_norm is not None:
        names += ["pre_norm_w"] + (["pre_norm_b"] if shape.pre_norm not in ("rms", "rmsnorm") else [])
    leaves = {}
    shared_h = tensors["h_router"] is tensors["h_attn"]
    for n in names:
        leaves[n] = tensors[n].detach().clone().float().requires_grad_(True)
    if shared_h:
        leaves["h_attn"] = leaves["h_router"]
    res = memory_layer(shape, leaves["h_router"], leaves["h_attn"], leaves["bank"],
                       leaves["router_w"], leaves["router_b"], leaves["wq"], leaves["wk"],
                       leaves["wv"], leaves["wo"], return_losses=True, autocast_bf16=autocast_bf16,
                       pre_norm_w=leaves.get("pre_norm_w"), pre_norm_b=leaves.get("pre_norm_b"))
    loss = (res["out"].float() * d_out.float()).sum()
    loss = loss + total_router_loss(res["losses"], load_balance_coef, auxiliary_coef, z_loss_coef)
    loss.backward()
    out = {k: (v.detach() if torch.is_tensor(v) else v) for k, v in res.items() if k != "losses"}
    out["losses"] = {k: v.detach() for k, v in res["losses"].items()}
    out["loss"] = loss.detach()
    for n in names:
        if shared_h and n == "h_attn":
            continue
        out["d_" + n] = leaves[n].grad.detach() if leaves[n].grad is not None else torch.zeros_like(leaves[n])
    return out


def layer_flops(batch: int, seq: int, shape: LayerShape) -> float:
    """Matmul FLOPs of one forward pass of the layer with the reference's own
    accounting (scripts/estimate_flops.py:353-357,385-417): Q and O
    projections, K and V projections of the selected rows, QK^T and PV, and the
    router GEMV.  Backward is counted as twice the forward
    (scripts/estimate_flops.py:805)."""
    d = shape.hidden_dim
    dkv = shape.num_kv_heads * shape.head_dim
    n_sel = (min(shape.top_k, shape.num_chapters - shape.num_shared_chapters)
             + shape.num_shared_chapters) * shape.tokens_per_chapter
    f = 2.0 * batch * seq * d * d * 2                 # Q and O
    f += 2.0 * batch * n_sel * d * dkv * 2            # K and V
    f += 4.0 * batch * seq * n_sel * d                # QK^T and PV over all heads
    f += 2.0 * batch * d * shape.num_chapters         # router
    return f


__all__ = [
    "LayerShape", "topk_lower_index_first", "router_pool", "router_pool_rolling", "router_forward", "router_losses",
    "total_router_loss", "route_token_level", "prepend_shared_chapters", "gather_chapters",
    "normalize_memory_rows", "scale_memory", "cross_attention", "sparse_chapter_attention", "attention_heads",
    "weighted_chapter_attention", "token_routed_attention", "token_memory_layer", "token_memory_layer_fwd_bwd",
    "memory_layer", "memory_layer_fwd_bwd", "layer_flops",
]
