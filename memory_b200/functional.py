"""Autograd bindings of the CUDA operators.

Three differentiable pieces mirror the reference's sequence-level memory layer
(memory_transformer/model.py:624-692 followed by memory_block.py:549-558):

``route``             router forward/backward (router.py:94-156, 197-260; model.py:356-391)
``gather_chapters``   chapter gather + optional row norm + weight scaling (memory_bank.py:244-293,
                      model.py:393-432, 689-692), backward scatters only into touched chapters
``cross_attention``   Q/K/V/O projections and joint-softmax attention over already gathered rows
                      (memory_attention.py:209-261, 298-316, 452-478)

``memory_layer`` chains them without materialising anything on the host.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from . import ops

LOSS_KEYS = ("load_balance", "auxiliary", "z_loss", "entropy")


class _LossDict(dict):
    """Router loss dict (same keys as the reference) that also carries the raw 4-vector as ``.vector``."""
    vector = None


class SparseBankGrad:
    """Receives bank gradients as (chapter ids, [U*T, d] rows) instead of a dense tensor.

    Attach one to a bank parameter with ``param.moc_sparse_grad = SparseBankGrad()``; backward
    passes then append here and return no dense gradient for the bank.
    """

    def __init__(self, wire_dtype: Optional[torch.dtype] = None, wire_only: bool = False):
        self.entries = []   # list of (uniq int32 [n_pairs], num_unique int32 [1], rows fp32 [n_pairs*T, d], T)
        self.wire = []      # per entry: the same rows in ``wire_dtype`` (what a gradient exchange sends), or None
        self.wire_dtype = wire_dtype   # torch.bfloat16: backward passes also produce the bf16 copy
        # the fused layer then writes ONLY the bf16 rows (they become the entry's rows): for data-parallel steps whose
        # mean gradient is formed from the ranks' bf16 rows anyway, the local fp32 rows would be written for nobody
        self.wire_only = bool(wire_only and wire_dtype == torch.bfloat16)
        self.scale = 1.0    # factor the consumer applies to the summed rows (1 / world after a zero-copy reduction)

    def add(self, uniq, num_unique, rows, tokens_per_chapter, wire=None):
        self.entries.append((uniq, num_unique, rows, int(tokens_per_chapter)))
        self.wire.append(wire)

    def clear(self):
        self.entries.clear()
        self.wire.clear()

    def to_dense(self, like: torch.Tensor) -> torch.Tensor:
        dense = torch.zeros(like.shape, dtype=torch.float32, device=like.device)
        for uniq, num_unique, rows, t in self.entries:
            ops.scatter_bank_grad(rows if rows.dtype == torch.float32 else rows.float(),
                                  {"uniq": uniq, "num_unique": num_unique}, t, dense)
        if self.scale != 1.0:
            dense.mul_(self.scale)
        return dense


# --------------------------------------------------------------------------------------------
# router
# --------------------------------------------------------------------------------------------
class _Route(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, weight, bias, top_k, num_shared, routed_scale, with_losses, pos_weight):
        pooled = ops.pool_weighted_fwd(h, pos_weight) if pos_weight is not None else None
        r = ops.router_fwd(h, weight, bias, top_k, num_shared, routed_scale, with_losses, pooled=pooled)
        ctx.cfg = (tuple(h.shape), h.dtype, int(top_k), int(num_shared), float(routed_scale), bias is not None)
        # Output tensors go through save_for_backward (autograd handles a node's own outputs there without a
        # reference cycle); only tensors that are not outputs stay as attributes, so the node and its buffers
        # are released by reference counting as soon as the graph is.
        ctx.internals = {k: r[k] for k in ("pooled", "probs", "idx", "row_stats", "chapter_stats", "_ws")}
        ctx.pos_weight = pos_weight
        ctx.save_for_backward(weight, r["weights"], r["comb_w"])
        ctx.mark_non_differentiable(r["idx"], r["comb_idx"])
        losses = r["losses"] if with_losses else torch.zeros(4, dtype=torch.float32, device=h.device)
        return r["idx"], r["weights"], r["comb_idx"], r["comb_w"], losses

    @staticmethod
    def backward(ctx, _g_idx, g_w, _g_cidx, g_cw, g_losses):
        weight, weights, comb_w = ctx.saved_tensors
        saved = dict(ctx.internals, weights=weights, comb_w=comb_w)
        h_shape, h_dtype, top_k, num_shared, routed_scale, has_bias = ctx.cfg
        if g_w is not None:
            g_w = g_w.float()
        if g_cw is not None:
            g_cw = g_cw.float()
        if g_losses is not None:
            g_losses = g_losses.float()
        want_dh = ctx.needs_input_grad[0]
        rolling = ctx.pos_weight is not None
        r = ops.router_bwd(h_shape, h_dtype, weight, saved, top_k, num_shared, routed_scale,
                           g_w, g_cw, g_losses, want_dh=want_dh and not rolling)
        d_h = r["d_h"]
        if rolling and want_dh:
            d_h = ops.pool_weighted_bwd(r["d_pooled"], ctx.pos_weight, h_shape, h_dtype)
        d_w = r["d_w"].to(weight.dtype) if ctx.needs_input_grad[1] else None
        d_b = r["d_bias"] if (has_bias and ctx.needs_input_grad[2]) else None
        return d_h, d_w, d_b, None, None, None, None, None


def route(h: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, num_shared: int,
          routed_scale: float = 1.0, with_losses: bool = True, pos_weight: Optional[torch.Tensor] = None):
    """Returns (idx int64 [B,k'], weights [B,k'], comb_idx int32 [B,S+k'], comb_w [B,S+k'], losses dict).
    ``pos_weight`` [L]: pool with these per-position coefficients instead of the plain mean (the
    sequence-rolling rule, see :func:`ops.rolling_pool_coefficients`)."""
    idx, w, cidx, cw, lv = _Route.apply(h, weight, bias, int(top_k), int(num_shared), float(routed_scale),
                                        bool(with_losses), pos_weight)
    losses = {k: lv[i] for i, k in enumerate(LOSS_KEYS)} if with_losses else {}
    if with_losses:
        losses = _LossDict(losses)
        losses.vector = lv          # the four losses as one tensor (order of LOSS_KEYS), for a single backward seed
    return idx, w, cidx, cw, losses


# --------------------------------------------------------------------------------------------
# gather
# --------------------------------------------------------------------------------------------
def _bank_backward(sink, d_mem, bank, t, comb_idx, comb_w, norm, eps, stats, num_chapters, want_dw, want_bank):
    seg = ops.chapter_segments(comb_idx, num_chapters)
    wire = [] if (sink is not None and sink.wire_dtype == torch.bfloat16) else None
    d_cw, rows = ops.gather_rows_bwd(d_mem, bank, t, comb_idx, comb_w, norm, eps, stats, seg,
                                     want_dw=want_dw, want_bank=want_bank, wire_copy=wire)
    d_bank = None
    if want_bank:
        if sink is not None:
            sink.add(seg["uniq"], seg["num_unique"], rows, t, wire=wire[0] if wire else None)
        else:
            d_bank = torch.zeros(bank.shape, dtype=torch.float32, device=bank.device)
            ops.scatter_bank_grad(rows, seg, t, d_bank)
            d_bank = d_bank.to(bank.dtype)
    return d_cw, d_bank


class _GatherChapters(torch.autograd.Function):
    @staticmethod
    def forward(ctx, bank, comb_idx, comb_w, tokens_per_chapter, norm_type, eps, out_dtype, sink):
        out, stats = ops.gather_rows_fwd(bank, tokens_per_chapter, comb_idx, comb_w, norm_type, eps, out_dtype)
        ctx.cfg = (int(tokens_per_chapter), norm_type, float(eps), bank.shape[0] // int(tokens_per_chapter))
        ctx.sink = sink
        ctx.save_for_backward(bank, comb_idx, comb_w, stats)
        return out

    @staticmethod
    def backward(ctx, g):
        bank, comb_idx, comb_w, stats = ctx.saved_tensors
        t, norm, eps, num_chapters = ctx.cfg
        g2 = g.reshape(-1, g.shape[-1])
        d_cw, d_bank = _bank_backward(ctx.sink, g2, bank, t, comb_idx, comb_w, norm, eps, stats, num_chapters,
                                      want_dw=comb_w is not None and ctx.needs_input_grad[2],
                                      want_bank=ctx.needs_input_grad[0])
        return d_bank, None, d_cw, None, None, None, None, None


def gather_chapters(bank: torch.Tensor, comb_idx: torch.Tensor, comb_w: Optional[torch.Tensor],
                    tokens_per_chapter: int, norm_type: Optional[str] = None, eps: float = 1e-5,
                    out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """[B, K*T, d] rows of the selected chapters, normalised and scaled by ``comb_w``."""
    sink = getattr(bank, "moc_sparse_grad", None)
    return _GatherChapters.apply(bank, comb_idx.to(torch.int32), comb_w, int(tokens_per_chapter), norm_type,
                                 float(eps), out_dtype or bank.dtype, sink)


# --------------------------------------------------------------------------------------------
# cross attention over gathered rows
# --------------------------------------------------------------------------------------------
class _CrossAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, memory, wq, wk, wv, wo, norm_w, norm_b, num_heads, num_kv_heads, compute_dtype,
                norm_kind, norm_eps, add_residual):
        b, l, d = h.shape
        cd = compute_dtype
        n_sel = memory.shape[-2]
        mem_shared = memory.dim() == 2
        x2 = h.reshape(b * l, d)
        stats = None
        if norm_kind is not None:
            # the normalisation writes the projection operand in the compute dtype: no separate cast
            x2 = x2.float()
            h2, stats = ops.norm_fwd(x2, norm_w.float(), None if norm_b is None else norm_b.float(), norm_kind,
                                     norm_eps, cd)
        else:
            h2 = ops.cast(x2, cd)
        m2 = ops.cast(memory.reshape(-1, memory.shape[-1]), cd)
        dkv = wk.shape[0]
        wt = None
        if cd == torch.bfloat16 and wq.dtype == wk.dtype == wv.dtype == wo.dtype:
            # one launch: bf16 working copies of the four weights (Wk and Wv stacked) and, for the backward
            # pass, their transposes, so every input-gradient projection has K-major operands
            w_all = torch.empty(2 * d + 2 * dkv, d, dtype=cd, device=h.device)
            wq_c, wkv_c, wo_c = w_all[:d], w_all[d:d + 2 * dkv], w_all[d + 2 * dkv:]
            need_t = any(ctx.needs_input_grad[:6])
            wq_t = torch.empty(d, d, dtype=cd, device=h.device) if need_t else None
            wkv_t = torch.empty(d, 2 * dkv, dtype=cd, device=h.device) if need_t else None
            wo_t = torch.empty(d, d, dtype=cd, device=h.device) if need_t else None
            ops.pack_weights([wq, wk, wv, wo], [wq_c, wkv_c[:dkv], wkv_c[dkv:], wo_c],
                             [wq_t, wkv_t, wkv_t[:, dkv:] if need_t else None, wo_t], [0, 2 * dkv, 2 * dkv, 0])
            wt = (wq_t, wkv_t, wo_t)
        else:
            wq_c, wo_c = ops.cast(wq, cd), ops.cast(wo, cd)
            wkv_c = ops.cast(torch.cat([wk, wv], dim=0), cd)
        q = ops.gemm(h2, wq_c, tag="q_proj")                                   # [B*L, H*D]
        kv = ops.gemm(m2, wkv_c, tag="kv_proj")                                 # [(B*)n_sel, 2*HK*D]
        if mem_shared:
            kv = kv.unsqueeze(0).expand(b, -1, -1).contiguous()
        head_dim = d // num_heads
        scale = head_dim ** -0.5
        kv = kv.view(b, n_sel, -1)
        o, lse = ops.attn_fwd(q.view(b, l, -1), kv, num_heads, num_kv_heads, scale)
        # the output projection writes the caller's dtype; the residual connection of the enclosing block
        # (memory_block.py:558) is added in its epilogue
        res = (x2 if x2.dtype == torch.float32 else x2.float()) if add_residual else None
        out = ops.gemm(o.view(b * l, -1), wo_c, out_dtype=h.dtype if h.dtype in (torch.float32, cd) else cd,
                       residual=res, tag="o_proj")
        ctx.cfg = (num_heads, num_kv_heads, scale, cd, mem_shared, h.dtype, memory.dtype)
        ctx.norm = (norm_kind, norm_b is not None, add_residual,
                    None if norm_w is None else norm_w.dtype, None if norm_b is None else norm_b.dtype)
        ctx.save_for_backward(h2, m2, wq_c, wkv_c, wo_c, q, kv, o, lse,
                              x2 if norm_kind is not None else None, stats,
                              norm_w.float() if norm_kind is not None else None)
        ctx.wt = wt
        ctx.w_dtypes = (wq.dtype, wk.dtype, wv.dtype, wo.dtype)
        return out.view(b, l, -1).to(h.dtype)

    @staticmethod
    def backward(ctx, g):
        h2, m2, wq_c, wkv_c, wo_c, q, kv, o, lse, x2, stats, norm_w = ctx.saved_tensors
        num_heads, num_kv_heads, scale, cd, mem_shared, h_dtype, mem_dtype = ctx.cfg
        norm_kind, norm_has_bias, add_residual, nw_dtype, nb_dtype = ctx.norm
        b, l, _ = o.shape
        d = h2.shape[1]
        g2 = ops.cast(g.reshape(b * l, -1).contiguous(), cd)
        f32 = torch.float32
        # K-splits of the weight-gradient projections: enough (tile, split) items to fill the SMs once
        def splits(rows, out_rows, out_cols):
            if cd == torch.float32:
                return 1
            tiles = -(-out_rows // 128) * -(-out_cols // 256)
            return max(1, min(148 // max(tiles, 1), rows // 512))
        split = splits(b * l, d, d)
        tc = cd == torch.bfloat16

        wt = ctx.wt

        def grad_in(dy, w_c, w_t, tag, out_dtype=None):
            """dX = dY W.  The tensor-core kernel is fastest with both operands K-major, so it takes the
            transposed copy of the small weight; the fp32 kernel takes the strided operand directly."""
            if tc:
                return ops.gemm(dy, w_t if w_t is not None else ops.transpose(w_c), out_dtype=out_dtype, tag=tag)
            return ops.gemm(dy, w_c, b_kmajor=False, tag=tag)

        d_o = grad_in(g2, wo_c, wt[2] if wt else None, "d_attn_out")                                      # [B*L, H*D]
        d_wo = ops.gemm(g2, o.view(b * l, -1), a_kmajor=False, b_kmajor=False, out_dtype=f32, split_k=split,
                        tag="d_wo")
        d_q, d_kv = ops.attn_bwd(q.view(b, l, -1), kv, o, lse, d_o.view(b, l, -1), num_heads, num_kv_heads, scale)
        d_q2 = d_q.view(b * l, -1)
        # gradient of the (normalised) attention input; fp32 when the normalisation's backward consumes it
        d_h = grad_in(d_q2, wq_c, wt[0] if wt else None, "d_h", f32 if norm_kind is not None else None)
        d_nw = d_nb = None
        g_res = g.reshape(b * l, -1) if add_residual else None
        if norm_kind is not None:
            d_h, d_nw, d_nb = ops.norm_bwd(d_h, x2, norm_w, stats, None if g_res is None else g_res.float(),
                                           norm_kind, norm_has_bias)
            d_nw = d_nw.to(nw_dtype)
            d_nb = None if d_nb is None else d_nb.to(nb_dtype)
        elif add_residual:
            d_h = d_h.float() + g_res.float()
        d_wq = ops.gemm(d_q2, h2, a_kmajor=False, b_kmajor=False, out_dtype=f32, split_k=split, tag="d_wq")
        d_kv2 = d_kv.view(-1, d_kv.shape[-1])
        if mem_shared:
            d_kv2 = d_kv.float().sum(dim=0).to(cd)
        rows = d_kv2.shape[0]
        split_kv = splits(rows, wkv_c.shape[0], d)
        d_mem = grad_in(d_kv2, wkv_c, wt[1] if wt else None, "d_mem")
        d_wkv = ops.gemm(d_kv2, m2, a_kmajor=False, b_kmajor=False, out_dtype=f32, split_k=split_kv, tag="d_wkv")
        dkv_dim = wkv_c.shape[0] // 2
        wdt = ctx.w_dtypes
        d_mem = d_mem.view(-1, d_mem.shape[-1]) if mem_shared else d_mem.view(b, -1, d_mem.shape[-1])
        return (d_h.view(b, l, d).to(h_dtype), d_mem.to(mem_dtype), d_wq.to(wdt[0]), d_wkv[:dkv_dim].to(wdt[1]),
                d_wkv[dkv_dim:].to(wdt[2]), d_wo.to(wdt[3]), d_nw, d_nb, None, None, None, None, None, None)


def cross_attention(h: torch.Tensor, memory: torch.Tensor, wq, wk, wv, wo, num_heads: int,
                    num_kv_heads: Optional[int] = None, compute_dtype: Optional[torch.dtype] = None, *,
                    pre_norm: Optional[str] = None, norm_weight: Optional[torch.Tensor] = None,
                    norm_bias: Optional[torch.Tensor] = None, norm_eps: float = 1e-6,
                    add_residual: bool = False) -> torch.Tensor:
    """softmax(Q K^T / sqrt(D)) V over the given memory rows, with the four projections.

    ``pre_norm`` ("rms" or "layernorm") normalises ``h`` first and ``add_residual`` adds ``h`` to the result:
    together they are the memory sub-block of the reference's transformer block, h + attn(norm(h), memory)
    (memory_block.py:549-558), with the normalisation fused into the query projection's operand and the
    residual add into the output projection's epilogue.
    """
    if pre_norm is not None:
        if pre_norm not in ops.NORM_KINDS:
            raise ValueError(f"unknown pre_norm {pre_norm!r}")
        if norm_weight is None:
            raise ValueError("pre_norm needs norm_weight")
        if pre_norm in ("rms", "rmsnorm"):
            norm_bias = None
    return _CrossAttention.apply(h, memory, wq, wk, wv, wo, norm_weight if pre_norm else None,
                                 norm_bias if pre_norm else None, int(num_heads), int(num_kv_heads or num_heads),
                                 compute_dtype or h.dtype, pre_norm, float(norm_eps), bool(add_residual))


# --------------------------------------------------------------------------------------------
# the whole layer as one node with two streams (bf16 path)
# --------------------------------------------------------------------------------------------
_side_streams: Dict[tuple, "torch.cuda.Stream"] = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    """Second stream of the layer, with the priority of the stream it runs beside (a step captured on a
    high-priority stream keeps both of its streams ahead of background work such as a gradient exchange)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    prio = torch.cuda.current_stream(device).priority
    key = (idx, prio)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device, priority=prio)
    return _side_streams[key]


# The dQ kernel runs on the side stream beside the dK/dV kernel (fused route): 768 CTAs over 296 slots leave the last
# of dQ's three rounds 59 % full, and the other kernel's CTAs take the free slots (measured 1.189 -> 1.177 ms per
# step).  MOC_DQ_ON_SIDE_STREAM=0 puts both back on the main stream.
_DQ_ON_SIDE_STREAM = os.environ.get("MOC_DQ_ON_SIDE_STREAM", "1") != "0"


class _MemoryLayerTwoStream(torch.autograd.Function):
    """Router, gather, projections and attention of one layer as a single autograd node, so that the
    bandwidth- and latency-bound kernels (router, chapter bookkeeping, gather backward) run on a second
    stream beside the tensor-core kernels instead of in front of or behind them:

      forward   side: router, chapter segments      | main: weight pack, (norm,) query projection
                join, then gather, K/V projection, attention, output projection on main
      backward  main: dO projection, attention backward, memory-row gradient, bank / chapter-weight
                gradients, router backward           | side: the four weight-gradient and the hidden-state
                                                       projections, normalisation backward

    Both streams fork from and join the caller's stream with events, which a CUDA-graph capture records as
    ordinary dependencies.  Every tensor that crosses streams stays referenced until after the join.
    """

    @staticmethod
    def forward(ctx, h_router, h_attn, bank, router_w, router_b, wq, wk, wv, wo, norm_w, norm_b, cfg, sink,
                fused=None):
        (num_heads, num_kv_heads, t, top_k, num_shared, routed_scale, row_norm, row_eps, with_losses,
         pre_norm, pre_eps, add_residual) = cfg
        cd = torch.bfloat16
        dev = h_attn.device
        b, l, d = h_attn.shape
        dkv = wk.shape[0]
        main, side = torch.cuda.current_stream(dev), _side_stream(dev)
        num_chapters = bank.shape[0] // t

        side.wait_stream(main)
        with torch.cuda.stream(side):
            r = ops.router_fwd(h_router, router_w, router_b, top_k, num_shared, routed_scale, with_losses, parts=1)
            routed = torch.cuda.Event()
            routed.record(side)          # the gather needs nothing after this point of the side stream
            if with_losses:
                ops.router_fwd(h_router, router_w, router_b, top_k, num_shared, routed_scale, with_losses, parts=2,
                               out=r)
            seg = ops.chapter_segments(r["comb_idx"], num_chapters)

        # main stream meanwhile: bf16 weights (+ transposes for the backward pass), query projection
        need_t = any(ctx.needs_input_grad[:11])
        w_all = torch.empty(2 * d + 2 * dkv, d, dtype=cd, device=dev)
        wq_c, wkv_c, wo_c = w_all[:d], w_all[d:d + 2 * dkv], w_all[d + 2 * dkv:]
        wq_t = torch.empty(d, d, dtype=cd, device=dev) if need_t else None
        wkv_t = torch.empty(d, 2 * dkv, dtype=cd, device=dev) if need_t else None
        wo_t = torch.empty(d, d, dtype=cd, device=dev) if need_t else None
        ops.pack_weights([wq, wk, wv, wo], [wq_c, wkv_c[:dkv], wkv_c[dkv:], wo_c],
                         [wq_t, wkv_t, wkv_t[:, dkv:] if need_t else None, wo_t], [0, 2 * dkv, 2 * dkv, 0])
        x2 = h_attn.reshape(b * l, d)
        stats_n = None
        if pre_norm is not None:
            x2 = x2.float()
            h2, stats_n = ops.norm_fwd(x2, norm_w.float(), None if norm_b is None else norm_b.float(), pre_norm,
                                       pre_eps, cd)
        else:
            h2 = ops.cast(x2, cd)
        q = ops.gemm(h2, wq_c, tag="q_proj")

        main.wait_event(routed)
        k_sel = r["idx"].shape[1]
        # the reference only normalises when both a shared and a routed slice exist (model.py:413-418)
        norm = row_norm if (num_shared > 0 and k_sel > 0) else None
        if fused is not None and (norm not in (None, "rms") or (norm == "rms" and fused.get("inv_rms") is None)):
            fused = None                      # affine-free LayerNorm rows are not a row scale: two-pass route
        row_scale = None
        if fused is not None:
            # Gather, normalisation, weight multiply and the K/V projection in one kernel: chapters are read from
            # the bf16 copy of the bank through the TMA gather list, u~ (and 1/rms) is the epilogue row scale.
            n_sel = r["comb_idx"].shape[1] * t
            row_scale = ops.chapter_row_scale(r["comb_idx"], r["comb_w"], fused["inv_rms"] if norm == "rms" else None,
                                              bank.shape[0], t)
            kv = ops.gemm(fused["shadow"], wkv_c, a_row_blocks=r["comb_idx"].reshape(-1), a_block_rows=t,
                          m=b * n_sel, row_scale=row_scale, scale_block_rows=1, tag="kv_proj").view(b, n_sel, -1)
            m2 = stats_m = None
        else:
            memory, stats_m = ops.gather_rows_fwd(bank, t, r["comb_idx"], r["comb_w"], norm, row_eps, cd)
            n_sel = memory.shape[-2]
            m2 = memory.reshape(-1, d)
            kv = ops.gemm(m2, wkv_c, tag="kv_proj").view(b, n_sel, -1)
        scale = (d // num_heads) ** -0.5
        o, lse = ops.attn_fwd(q.view(b, l, -1), kv, num_heads, num_kv_heads, scale)
        res = (x2 if x2.dtype == torch.float32 else x2.float()) if add_residual else None
        out_dtype = h_attn.dtype if h_attn.dtype in (torch.float32, cd) else cd
        out = ops.gemm(o.view(b * l, -1), wo_c, out_dtype=out_dtype, residual=res, tag="o_proj")
        main.wait_stream(side)           # loss terms and chapter segments finished beside the attention

        ctx.cfg = cfg
        ctx.norm_row = norm
        ctx.fused = None if fused is None else dict(fused, row_scale=row_scale)
        ctx.scale = scale
        # outputs of this node (weights, combined weights, losses) are saved through save_for_backward below:
        # kept as attributes they would tie the node to its own outputs in a reference cycle
        ctx.router_saved = {k: r[k] for k in ("pooled", "probs", "idx", "comb_idx", "row_stats", "chapter_stats", "_ws")}
        ctx.seg = seg
        ctx.sink = sink
        ctx.same_h = h_router is h_attn
        ctx.shapes = (tuple(h_router.shape), h_router.dtype, h_attn.dtype, router_b is not None,
                      (wq.dtype, wk.dtype, wv.dtype, wo.dtype), None if norm_w is None else norm_w.dtype,
                      None if norm_b is None else norm_b.dtype)
        ctx.wt = (wq_t, wkv_t, wo_t)
        ctx.save_for_backward(h2, m2, wq_c, wkv_c, wo_c, q, kv, o, lse, bank, router_w, stats_m,
                              x2 if pre_norm is not None else None, stats_n,
                              norm_w.float() if pre_norm is not None else None, r["weights"], r["comb_w"])
        ctx.mark_non_differentiable(r["idx"], r["comb_idx"])
        losses = r["losses"] if with_losses else torch.zeros(4, dtype=torch.float32, device=dev)
        return out.view(b, l, -1).to(h_attn.dtype), r["idx"], r["weights"], r["comb_idx"], r["comb_w"], losses

    @staticmethod
    def backward(ctx, g, _g_idx, g_w, _g_cidx, g_cw, g_losses):
        (h2, m2, wq_c, wkv_c, wo_c, q, kv, o, lse, bank, router_w, stats_m, x2, stats_n,
         norm_w, r_weights, r_comb_w) = ctx.saved_tensors
        (num_heads, num_kv_heads, t, top_k, num_shared, routed_scale, _row_norm, row_eps, _with_losses,
         pre_norm, _pre_eps, add_residual) = ctx.cfg
        hr_shape, hr_dtype, ha_dtype, has_rbias, wdt, nw_dtype, nb_dtype = ctx.shapes
        wq_t, wkv_t, wo_t = ctx.wt
        r, seg = dict(ctx.router_saved, weights=r_weights, comb_w=r_comb_w), ctx.seg
        cd, f32 = torch.bfloat16, torch.float32
        dev = q.device
        b, l, _ = o.shape
        d = h2.shape[1]
        main, side = torch.cuda.current_stream(dev), _side_stream(dev)
        need = ctx.needs_input_grad
        num_chapters = bank.shape[0] // t

        def splits(rows, out_rows, out_cols):
            tiles = -(-out_rows // 128) * -(-out_cols // 256)
            return max(1, min(148 // max(tiles, 1), rows // 512))

        g2f = g.reshape(b * l, -1)
        g2 = ops.cast(g2f.contiguous(), cd)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            d_wo = ops.gemm(g2, o.view(b * l, -1), a_kmajor=False, b_kmajor=False, out_dtype=f32,
                            split_k=splits(b * l, d, d), tag="d_wo")
        d_o = ops.gemm(g2, wo_t, tag="d_attn_out")
        fused = ctx.fused
        # 64-row chapters: the chapter-weight gradient is taken in the dK/dV epilogue, where K and V are still in
        # shared memory, instead of by a pass over the memory-row gradient and the bank rows
        kv_dot = None
        if fused is not None and t == 64:
            kv_dot = torch.empty(b, kv.shape[1] // 64, num_kv_heads, dtype=f32, device=dev)
        split_bwd = _DQ_ON_SIDE_STREAM and fused is not None
        if split_bwd:
            # per-row constants here, then the dQ kernel on the side stream (its consumers follow it there) beside
            # the dK/dV kernel on this one: each fills the tail of the other's last round of CTAs
            q3, do3 = q.view(b, l, -1), d_o.view(b, l, -1)
            bufs = (torch.empty_like(q3), torch.empty_like(kv),
                    torch.empty(6, b, num_heads, l, dtype=f32, device=dev))
            akw = dict(buffers=bufs, kv_row_scale=fused["row_scale"], kv_dot=kv_dot)
            ops.attn_bwd(q3, kv, o, lse, do3, num_heads, num_kv_heads, ctx.scale, parts=1, **akw)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                ops.attn_bwd(q3, kv, o, lse, do3, num_heads, num_kv_heads, ctx.scale, parts=2, **akw)
            ops.attn_bwd(q3, kv, o, lse, do3, num_heads, num_kv_heads, ctx.scale, parts=4, **akw)
            d_q, d_kv = bufs[0], bufs[1]
        else:
            d_q, d_kv = ops.attn_bwd(q.view(b, l, -1), kv, o, lse, d_o.view(b, l, -1), num_heads, num_kv_heads,
                                     ctx.scale, kv_row_scale=None if fused is None else fused["row_scale"],
                                     kv_dot=kv_dot)
        d_q2 = d_q.view(b * l, -1)
        d_kv2 = d_kv.view(-1, d_kv.shape[-1])

        if not split_bwd:
            side.wait_stream(main)
        with torch.cuda.stream(side):
            d_wq = ops.gemm(d_q2, h2, a_kmajor=False, b_kmajor=False, out_dtype=f32, split_k=splits(b * l, d, d),
                            tag="d_wq")
            # gradient of the (normalised) attention input, in the hidden-state dtype so that the router's
            # gradient can be added into it
            d_h = ops.gemm(d_q2, wq_t, out_dtype=f32 if (pre_norm is not None or ha_dtype == f32) else cd, tag="d_h")
            d_nw = d_nb = None
            g_res = g2f if add_residual else None
            if pre_norm is not None:
                d_h, d_nw, d_nb = ops.norm_bwd(d_h, x2, norm_w, stats_n, None if g_res is None else g_res.float(),
                                               pre_norm, nb_dtype is not None)
                d_nw = d_nw.to(nw_dtype)
                d_nb = None if d_nb is None else d_nb.to(nb_dtype)
            elif add_residual:
                d_h = d_h.float() + g_res.float()
            d_h = d_h.view(b, l, d).to(ha_dtype)
            ev_dh = torch.cuda.Event()
            ev_dh.record(side)              # the router's hidden-state gradient is added into d_h later
            if split_bwd:
                side.wait_stream(main)      # dK/dV was issued on the main stream
            if fused is None:
                d_wkv = ops.gemm(d_kv2, m2, a_kmajor=False, b_kmajor=False, out_dtype=f32,
                                 split_k=splits(d_kv2.shape[0], wkv_c.shape[0], d), tag="d_wkv")
            elif fused.get("wkv_grad_in_place"):
                # dKV' already carries the row scale, so the weight gradient can read the raw bank rows in place
                # through the gather list on its B operand
                d_wkv = ops.gemm(d_kv2, fused["shadow"], a_kmajor=False, b_kmajor=False, out_dtype=f32,
                                 split_k=splits(d_kv2.shape[0], wkv_c.shape[0], d), tag="d_wkv",
                                 b_row_blocks=r["comb_idx"].reshape(-1), b_block_rows=t, k=d_kv2.shape[0])
            else:
                # ... but with the contraction running over chapters, every K step of that projection lands in
                # another chapter of the 403 MB copy and it measured twice as slow as over contiguous rows.  This
                # stream has slack, so the raw selected rows (no norm, no weight: dKV' carries both) are copied out
                # once here, off the critical path, and the projection runs over the contiguous copy.
                m_raw, _ = ops.gather_rows_fwd(fused["shadow"], t, r["comb_idx"], None, None, row_eps, cd)
                d_wkv = ops.gemm(d_kv2, m_raw.view(-1, d), a_kmajor=False, b_kmajor=False, out_dtype=f32,
                                 split_k=splits(d_kv2.shape[0], wkv_c.shape[0], d), tag="d_wkv")

        d_mem = ops.gemm(d_kv2, wkv_t, tag="d_mem")
        want_bank = need[2]
        wire = [] if (ctx.sink is not None and ctx.sink.wire_dtype == torch.bfloat16) else None
        d_bank = None

        def emit_bank(rows):
            nonlocal d_bank
            if not want_bank:
                return
            if ctx.sink is not None:
                ctx.sink.add(seg["uniq"], seg["num_unique"], rows, t, wire=wire[0] if wire else None)
            else:
                d_bank = torch.zeros(bank.shape, dtype=f32, device=dev)
                ops.scatter_bank_grad(rows, seg, t, d_bank)
                d_bank = d_bank.to(bank.dtype)

        if fused is None:
            d_cw, rows = ops.gather_rows_bwd(d_mem, bank, t, r["comb_idx"], r["comb_w"], ctx.norm_row, row_eps,
                                             stats_m, seg, want_dw=True, want_bank=want_bank, wire_copy=wire)
            emit_bank(rows)
        else:
            pre = dict(want_bank=want_bank, wire_copy=wire,
                       wire_only=ctx.sink is not None and getattr(ctx.sink, "wire_only", False))
            pargs = (d_mem, fused["shadow"], t, r["comb_idx"], r["comb_w"],
                     fused["inv_rms"] if ctx.norm_row == "rms" else None, seg)
            if kv_dot is not None:
                # the chapter-weight gradient came out of the dK/dV epilogue, so nothing downstream reads the bank
                # gradient: its kernel runs on the side stream, off the path to the router's backward
                d_cw = kv_dot.sum(dim=2) / r["comb_w"].clamp_min(1e-30)
                ev_mem = torch.cuda.Event()
                ev_mem.record(main)
                with torch.cuda.stream(side):
                    side.wait_event(ev_mem)
                    _, rows = ops.gather_rows_bwd_prescaled(*pargs, want_dw=False, **pre)
                    emit_bank(rows if rows is not None else (wire[0] if wire else None))
            else:
                d_cw, rows = ops.gather_rows_bwd_prescaled(*pargs, want_dw=True, **pre)
                emit_bank(rows if rows is not None else (wire[0] if wire else None))
        if g_cw is not None:
            d_cw = d_cw + g_cw.float()
        fuse_dh = ctx.same_h and need[0] and hr_dtype == ha_dtype
        if fuse_dh:
            main.wait_event(ev_dh)      # the attention branch's d_h must be complete before the router adds to it
        # logit gradient on the main stream; the router-weight gradient (nothing downstream reads it) on the side
        # stream beside the pooled / hidden-state gradient
        rargs = (hr_shape, hr_dtype, router_w, r, top_k, num_shared, routed_scale,
                 None if g_w is None else g_w.float(), d_cw, None if g_losses is None else g_losses.float())
        rb = ops.router_bwd(*rargs, want_dh=need[0], parts=1)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            ops.router_bwd(*rargs, want_dh=need[0], parts=2, out=rb)
        ops.router_bwd(*rargs, want_dh=need[0], d_h_accum=d_h if fuse_dh else None, parts=4, out=rb)
        main.wait_stream(side)
        d_rw = rb["d_w"].to(router_w.dtype) if need[3] else None
        d_rb = rb["d_bias"] if (has_rbias and need[4]) else None
        dkv_dim = wkv_c.shape[0] // 2
        if fuse_dh:
            d_hr, d_ha = rb["d_h"], None
        else:
            d_hr, d_ha = rb["d_h"], d_h
        return (d_hr, d_ha, d_bank, d_rw, d_rb, d_wq.to(wdt[0]), d_wkv[:dkv_dim].to(wdt[1]),
                d_wkv[dkv_dim:].to(wdt[2]), d_wo.to(wdt[3]), d_nw, d_nb, None, None, None)


# --------------------------------------------------------------------------------------------
# the fused layer
# --------------------------------------------------------------------------------------------
def memory_layer(h_router: torch.Tensor, h_attn: torch.Tensor, bank: torch.Tensor,
                 router_weight: torch.Tensor, router_bias: Optional[torch.Tensor],
                 wq, wk, wv, wo, *, num_heads: int, num_kv_heads: Optional[int], tokens_per_chapter: int,
                 top_k: int, num_shared_chapters: int = 1, routed_scaling_factor: float = 2.5,
                 norm_type: Optional[str] = None, norm_eps: float = 1e-5, with_losses: bool = True,
                 compute_dtype: Optional[torch.dtype] = None, pre_norm: Optional[str] = None,
                 pre_norm_weight: Optional[torch.Tensor] = None, pre_norm_bias: Optional[torch.Tensor] = None,
                 pre_norm_eps: float = 1e-6, add_residual: bool = False,
                 two_stream: bool = True, bank_shadow: Optional[torch.Tensor] = None,
                 bank_inv_rms: Optional[torch.Tensor] = None,
                 wkv_grad_in_place: bool = False) -> Tuple[torch.Tensor, Dict[str, torch.Tensor], Dict]:
    """Sequence-level Mixture-of-Chapters memory layer on the GPU.

    Returns (out [B,L,d], router losses, info) with info = indices / weights of the routing.
    ``norm_type`` normalises the gathered bank rows; ``pre_norm`` / ``add_residual`` wrap the attention as
    h_attn + attn(pre_norm(h_attn), memory) (see :func:`cross_attention`).  With bf16 compute the layer runs as
    one autograd node that overlaps its small kernels with the tensor-core kernels on a second stream
    (``two_stream=False`` chains the three separate nodes instead; results are the same).

    ``bank_shadow`` (bf16 copy of ``bank``, e.g. ``ChapteredMemoryBank.bf16_shadow()`` or the copy
    ``SparseBankAdamW`` refreshes) switches the bf16 layer to the fused gather-and-project route: the K/V projection
    reads the selected chapters straight from that copy and no gathered rows are materialised, forward or
    backward.  With ``norm_type="rms"`` it also needs ``bank_inv_rms`` (``ops.row_inv_rms`` of the bank with
    ``norm_eps``); ``norm_type="layernorm"`` keeps the two-pass route.  ``wkv_grad_in_place`` lets the Wk / Wv
    gradient read the bank through a gather list as well instead of copying the raw selected rows out on the side
    stream first (no gathered copy at all, but slower at the paper shape).
    """
    cd = compute_dtype or h_attn.dtype
    if (cd == torch.bfloat16 and two_stream and wq.dtype == wk.dtype == wv.dtype == wo.dtype
            and bank.shape[1] == h_attn.shape[-1]):
        cfg = (int(num_heads), int(num_kv_heads or num_heads), int(tokens_per_chapter), int(top_k),
               int(num_shared_chapters), float(routed_scaling_factor), norm_type, float(norm_eps), bool(with_losses),
               pre_norm, float(pre_norm_eps), bool(add_residual))
        if pre_norm is not None and pre_norm not in ops.NORM_KINDS:
            raise ValueError(f"unknown pre_norm {pre_norm!r}")
        if pre_norm in ("rms", "rmsnorm"):
            pre_norm_bias = None
        out, idx, w, cidx, cw, lv = _MemoryLayerTwoStream.apply(
            h_router, h_attn, bank, router_weight, router_bias, wq, wk, wv, wo,
            pre_norm_weight if pre_norm else None, pre_norm_bias if pre_norm else None, cfg,
            getattr(bank, "moc_sparse_grad", None),
            None if bank_shadow is None else {"shadow": bank_shadow, "inv_rms": bank_inv_rms,
                                              "wkv_grad_in_place": wkv_grad_in_place})
        losses = {}
        if with_losses:
            losses = _LossDict({k: lv[i] for i, k in enumerate(LOSS_KEYS)})
            losses.vector = lv
        return out, losses, {"indices": idx, "weights": w, "combined_indices": cidx, "combined_weights": cw}
    idx, w, cidx, cw, losses = route(h_router, router_weight, router_bias, top_k, num_shared_chapters,
                                     routed_scaling_factor, with_losses)
    k_sel = idx.shape[1]
    # the reference only normalises when both a shared and a routed slice exist (model.py:413-418)
    norm = norm_type if (num_shared_chapters > 0 and k_sel > 0) else None
    memory = gather_chapters(bank, cidx, cw, tokens_per_chapter, norm, norm_eps, out_dtype=cd)
    out = cross_attention(h_attn, memory, wq, wk, wv, wo, num_heads, num_kv_heads, cd, pre_norm=pre_norm,
                          norm_weight=pre_norm_weight, norm_bias=pre_norm_bias, norm_eps=pre_norm_eps,
                          add_residual=add_residual)
    return out, losses, {"indices": idx, "weights": w, "combined_indices": cidx, "combined_weights": cw}


# --------------------------------------------------------------------------------------------
# token-level routing (every token selects its own chapters)
# --------------------------------------------------------------------------------------------
def _weight_grad_splits(cd, rows: int, out_rows: int, out_cols: int) -> int:
    """K-splits of a weight-gradient projection dW[out_rows, out_cols] = dY^T X over ``rows``: enough (tile, split)
    items to fill the SMs once (tensor-core kernel only; the splits add into a zeroed fp32 output)."""
    if cd != torch.bfloat16:
        return 1
    tiles = -(-out_rows // 128) * -(-out_cols // 256)
    return max(1, min(148 // max(tiles, 1), rows // 512))


# rows * chapters * hidden above which a bf16 model's token router projects on the tensor cores (split fp32 weight)
_SPLIT_ROUTER_MIN_WORK = 1 << 27


class _RouteTokens(torch.autograd.Function):
    """ChapterRouter.route_token_level (router.py:262-340): logits of every token by an fp32 projection, then the
    same softmax / prefix mask / top-k / renormalisation / loss kernels as the sequence router with one routing
    row per token."""

    @staticmethod
    def forward(ctx, h, weight, bias, top_k, num_shared, with_losses):
        b, l, d = h.shape
        rows = b * l
        h2 = h.reshape(rows, d).contiguous()
        h32 = ops.cast(h2, torch.float32)
        w32 = weight.float().contiguous()
        c = w32.shape[0]
        split = None
        if h.dtype == torch.bfloat16 and d % 8 == 0 and rows * c * d >= _SPLIT_ROUTER_MIN_WORK:
            # bf16 activations are exact bf16 numbers: logits = h (w0 + w1 + w2)^T as three tensor-core products
            # accumulated in fp32 (smallest term first) carry the fp32 weight's 24 mantissa bits
            cp = -(-c // 8) * 8
            w_terms = ops.split_bf16(w32 if cp == c else torch.nn.functional.pad(w32, (0, 0, 0, cp - c)), 3)
            parts = ops.gemm(h2, w_terms.view(3 * cp, d), out_dtype=torch.float32, tag="token_router_logits")
            logits = ops.sum_terms(parts, c, 3, bias=None if bias is None else bias.float())
            del parts
            split = (h2, w_terms, cp)
        else:
            logits = ops.gemm(h32, w32, tag="token_router_logits")                 # [rows, C] fp32, no bias yet
        ctx.split = split
        r = ops.router_fwd(h32.view(rows, 1, d), w32, None if split is not None else bias, top_k, num_shared, 1.0,
                           with_losses, pooled=h32, logits=logits)      # (the split path has added the bias)
        k = r["idx"].shape[1]
        ctx.cfg = ((b, l, d), h.dtype, int(top_k), int(num_shared), bias is not None)
        ctx.internals = {n: r[n] for n in ("pooled", "probs", "idx", "row_stats", "chapter_stats", "_ws", "comb_w")}
        ctx.save_for_backward(w32, r["weights"])
        idx = r["idx"].view(b, l, k)
        ctx.mark_non_differentiable(idx)
        losses = r["losses"] if with_losses else torch.zeros(4, dtype=torch.float32, device=h.device)
        return idx, r["weights"].view(b, l, k), losses

    @staticmethod
    def backward(ctx, _g_idx, g_w, g_losses):
        w32, weights = ctx.saved_tensors
        (b, l, d), h_dtype, top_k, num_shared, has_bias = ctx.cfg
        rows = b * l
        saved = dict(ctx.internals, weights=weights)
        g_w = None if g_w is None else g_w.reshape(rows, -1).float().contiguous()
        g_losses = None if g_losses is None else g_losses.float()
        r = ops.router_bwd((rows, 1, d), torch.float32, w32, saved, top_k, num_shared, 1.0, g_w, None, g_losses,
                           want_dh=False, parts=1, logits_only=True)
        d_logits = r["d_logits"]
        h32 = saved["pooled"]
        d_h = d_w = d_b = None
        if ctx.split is not None:
            h2, w_terms, cp = ctx.split
            c = w32.shape[0]
            dl = d_logits if cp == c else torch.nn.functional.pad(d_logits, (0, cp - c))
            dl_terms = ops.split_bf16(dl, 3)                                       # [3, rows, cp]
            if ctx.needs_input_grad[0]:
                # the gradient leaves in bf16: one product of the leading terms
                d_h = ops.gemm(dl_terms[0], w_terms[0], b_kmajor=False, tag="token_router_dh").view(b, l, d)
            if ctx.needs_input_grad[1]:
                for t in (2, 1, 0):
                    d_w = ops.gemm(dl_terms[t], h2, a_kmajor=False, b_kmajor=False, out=d_w, out_dtype=torch.float32,
                                   accumulate=d_w is not None, tag="token_router_dw")
                d_w = d_w[:c]
        else:
            if ctx.needs_input_grad[0]:
                d_h = ops.gemm(d_logits, w32, b_kmajor=False, tag="token_router_dh").view(b, l, d).to(h_dtype)
            if ctx.needs_input_grad[1]:
                d_w = ops.gemm(d_logits, h32, a_kmajor=False, b_kmajor=False, tag="token_router_dw")
        if has_bias and ctx.needs_input_grad[2]:
            d_b = ops.col_sum(d_logits)
        return d_h, d_w, d_b, None, None, None


def route_tokens(h: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, num_shared: int,
                 with_losses: bool = True):
    """Returns (global chapter ids int64 [B,L,k'], weights [B,L,k'], losses dict); k' = min(k, C - num_shared)."""
    idx, w, lv = _RouteTokens.apply(h, weight, bias, int(top_k), int(num_shared), bool(with_losses))
    losses = {}
    if with_losses:
        losses = _LossDict({k: lv[i] for i, k in enumerate(LOSS_KEYS)})
        losses.vector = lv
    return idx, w, losses


class _TokenRoutedAttention(torch.autograd.Function):
    """MemoryCrossAttention._forward_token_routed_attention + o_proj (memory_attention.py:480-716, 452-456) with
    per-token chapter weights:

        out = Wo [ attn(q, shared rows)  +  rho * sum_s w[t,s] softmax(q K_{c(t,s)}^T) V_{c(t,s)} ]

    The routed bank is projected once (the reference projects it once per batch item); the shared branch is the
    dense attention kernel over the S*T shared rows with all B*L tokens as one sequence."""

    @staticmethod
    def forward(ctx, h, shared_mem, routed_mem, idx_local, weights, wq, wk, wv, wo, cfg):
        num_heads, num_kv_heads, t, rho, cd = cfg
        b, l, d = h.shape
        rows = b * l
        dkv = wk.shape[0]
        head_dim = d // num_heads
        scale = head_dim ** -0.5
        h2 = ops.cast(h.reshape(rows, d).contiguous(), cd)
        wq_c, wo_c = ops.cast(wq, cd), ops.cast(wo, cd)
        wkv_c = ops.cast(torch.cat([wk, wv], dim=0), cd)
        q = ops.gemm(h2, wq_c, tag="q_proj")                                            # [rows, H*D]
        comb = None
        sh = None
        if shared_mem is not None and shared_mem.numel() > 0:
            sm2 = ops.cast(shared_mem.contiguous(), cd)
            kv_sh = ops.gemm(sm2, wkv_c, tag="kv_proj_shared")                          # [S*T, 2*dkv]
            # bf16 attention backward wants the query count in multiples of 64: pad with zero rows
            pad = (-rows) % 64 if cd == torch.bfloat16 else 0
            q_sh = q if pad == 0 else torch.cat([q, q.new_zeros(pad, q.shape[1])], dim=0)
            o_sh, lse_sh = ops.attn_fwd(q_sh.view(1, rows + pad, -1), kv_sh.view(1, kv_sh.shape[0], -1), num_heads,
                                        num_kv_heads, scale)
            sh = (sm2, kv_sh, q_sh, o_sh, lse_sh, pad)
            comb = o_sh.view(rows + pad, -1)[:rows]
        rt = None
        k_sel = idx_local.shape[-1]
        if routed_mem is not None and routed_mem.numel() > 0 and k_sel > 0:
            rm2 = ops.cast(routed_mem.contiguous(), cd)
            kv_rt = ops.gemm(rm2, wkv_c, tag="kv_proj_routed")                          # [(C-S)*T, 2*dkv]
            n_rt = kv_rt.shape[0]
            k4 = kv_rt[:, :dkv].unflatten(1, (num_kv_heads, head_dim)).unsqueeze(0)
            v4 = kv_rt[:, dkv:].unflatten(1, (num_kv_heads, head_dim)).unsqueeze(0)
            w2 = weights.reshape(1, rows, k_sel).float().contiguous()
            q4 = q.view(1, rows, num_heads, head_dim)
            base = None if comb is None else comb.contiguous().view(1, rows, num_heads, head_dim)
            mix_ws = None
            if ops.token_mix_supported(q4, k4, t, 1):
                # tensor cores: every chapter's K / V tile stationary under the tokens that selected it
                bidx = idx_local.reshape(1, rows, 1, k_sel).to(torch.int32).contiguous()
                comb4, lse_slots, mix_ws = ops.token_mix_fwd(q4, k4, v4, bidx, w2, scale, base=base, out_scale=rho)
            else:
                bidx = idx_local.reshape(1, rows, 1, k_sel).expand(1, rows, num_kv_heads, k_sel).to(torch.int32).contiguous()
                comb4, lse_slots = ops.sparse_attn_weighted_fwd(q4, k4, v4, bidx, w2, t, scale, base=base,
                                                                out_scale=rho)
            comb = comb4.view(rows, -1)
            rt = (rm2, kv_rt, bidx, w2, lse_slots, n_rt, mix_ws)
        if comb is None:
            comb = q.new_zeros(rows, d)
        out = ops.gemm(comb.contiguous(), wo_c, out_dtype=h.dtype if h.dtype in (torch.float32, cd) else cd, tag="o_proj")
        ctx.cfg = cfg
        ctx.meta = (b, l, d, dkv, scale, h.dtype, None if shared_mem is None else shared_mem.dtype,
                    None if routed_mem is None else routed_mem.dtype, weights.dtype,
                    (wq.dtype, wk.dtype, wv.dtype, wo.dtype))
        ctx.sh, ctx.rt = sh, rt
        ctx.save_for_backward(h2, q, comb, wq_c, wkv_c, wo_c)
        return out.view(b, l, -1).to(h.dtype)

    @staticmethod
    def backward(ctx, g):
        h2, q, comb, wq_c, wkv_c, wo_c = ctx.saved_tensors
        num_heads, num_kv_heads, t, rho, cd = ctx.cfg
        b, l, d, dkv, scale, h_dtype, sh_dtype, rt_dtype, w_dtype, wdt = ctx.meta
        rows = b * l
        head_dim = d // num_heads
        f32 = torch.float32
        g2 = ops.cast(g.reshape(rows, -1).contiguous(), cd)
        d_comb = ops.gemm(g2, wo_c, b_kmajor=False, tag="d_attn_out")                   # [rows, H*D]
        d_wo = ops.gemm(g2, comb, a_kmajor=False, b_kmajor=False, out_dtype=f32,
                        split_k=_weight_grad_splits(cd, rows, wo_c.shape[0], wo_c.shape[1]), tag="d_wo")
        d_q = None
        d_wkv = None
        d_shared = d_routed = d_weights = None
        if ctx.sh is not None:
            sm2, kv_sh, q_sh, o_sh, lse_sh, pad = ctx.sh
            dc = d_comb if pad == 0 else torch.cat([d_comb, d_comb.new_zeros(pad, d_comb.shape[1])], dim=0)
            d_q_sh, d_kv_sh = ops.attn_bwd(q_sh.view(1, rows + pad, -1), kv_sh.view(1, kv_sh.shape[0], -1), o_sh, lse_sh,
                                           dc.view(1, rows + pad, -1), num_heads, num_kv_heads, scale)
            d_q = d_q_sh.view(rows + pad, -1)[:rows].contiguous()
            d_kv_sh2 = d_kv_sh.view(kv_sh.shape[0], -1)
            d_shared = ops.gemm(d_kv_sh2, wkv_c, b_kmajor=False, out_dtype=sh_dtype if sh_dtype in (f32, cd) else cd,
                                tag="d_shared_mem").to(sh_dtype)
            d_wkv = ops.gemm(d_kv_sh2, sm2, a_kmajor=False, b_kmajor=False, out_dtype=f32,
                             split_k=_weight_grad_splits(cd, sm2.shape[0], 2 * dkv, d), tag="d_wkv_shared")
        if ctx.rt is not None:
            rm2, kv_rt, bidx, w2, lse_slots, n_rt, mix_ws = ctx.rt
            k4 = kv_rt[:, :dkv].unflatten(1, (num_kv_heads, head_dim)).unsqueeze(0)
            v4 = kv_rt[:, dkv:].unflatten(1, (num_kv_heads, head_dim)).unsqueeze(0)
            # (the tensor-core mixture writes every row itself; the CUDA-core one adds into zeros)
            d_kv_rt = (torch.zeros(n_rt, 2 * dkv, dtype=f32, device=q.device) if mix_ws is None
                       else torch.empty(n_rt, 2 * dkv, dtype=cd, device=q.device))
            dk4 = d_kv_rt[:, :dkv].unflatten(1, (num_kv_heads, head_dim)).unsqueeze(0)
            dv4 = d_kv_rt[:, dkv:].unflatten(1, (num_kv_heads, head_dim)).unsqueeze(0)
            q4, dc4 = q.view(1, rows, num_heads, head_dim), d_comb.view(1, rows, num_heads, head_dim)
            d_q4 = None if d_q is None else d_q.view(1, rows, num_heads, head_dim)
            if mix_ws is not None:
                d_q, d_w = ops.token_mix_bwd(q4, k4, v4, bidx, w2, lse_slots, dc4, scale, rho, mix_ws, dk4, dv4,
                                             d_q_base=d_q4)
                d_kv_c = d_kv_rt
            else:
                d_q, d_w = ops.sparse_attn_weighted_bwd(q4, k4, v4, bidx, w2, lse_slots, dc4, t, scale, rho, dk4, dv4,
                                                        d_q_accum=d_q4)
                d_kv_c = ops.cast(d_kv_rt, cd)
            d_q = d_q.view(rows, -1)
            d_weights = d_w.view(b, l, -1).to(w_dtype)
            # written in the bank's dtype by the projection's epilogue (an fp32 master bank: no conversion pass
            # over 805 MB afterwards)
            d_routed = ops.gemm(d_kv_c, wkv_c, b_kmajor=False, out_dtype=rt_dtype if rt_dtype in (f32, cd) else cd,
                                tag="d_routed_mem").to(rt_dtype)
            g_wkv = ops.gemm(d_kv_c, rm2, a_kmajor=False, b_kmajor=False, out_dtype=f32,
                             split_k=_weight_grad_splits(cd, n_rt, 2 * dkv, d), tag="d_wkv_routed")
            d_wkv = g_wkv if d_wkv is None else d_wkv + g_wkv
        if d_q is None:
            d_q = q.new_zeros(rows, d)
        d_h = ops.gemm(d_q, wq_c, b_kmajor=False, tag="d_h").view(b, l, d).to(h_dtype)
        d_wq = ops.gemm(d_q, h2, a_kmajor=False, b_kmajor=False, out_dtype=f32,
                        split_k=_weight_grad_splits(cd, rows, d, d), tag="d_wq")
        if d_wkv is None:
            d_wkv = torch.zeros(2 * dkv, d, dtype=f32, device=q.device)
        return (d_h, d_shared, d_routed, None, d_weights, d_wq.to(wdt[0]), d_wkv[:dkv].to(wdt[1]),
                d_wkv[dkv:].to(wdt[2]), d_wo.to(wdt[3]), None)


def token_routed_attention(h: torch.Tensor, shared_memory: Optional[torch.Tensor],
                           routed_memory: Optional[torch.Tensor], token_chapter_indices: torch.Tensor,
                           chapter_weights: torch.Tensor, wq, wk, wv, wo, *, num_heads: int,
                           num_kv_heads: Optional[int], tokens_per_chapter: int, routed_scale: float = 1.0,
                           compute_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Token-routed memory cross-attention with router-weighted chapters, output projection included.
    ``token_chapter_indices`` [B,L,k] are ids LOCAL to ``routed_memory`` (global id minus the shared prefix,
    model.py:583-595); ``chapter_weights`` [B,L,k] carry the router's gradient."""
    cfg = (int(num_heads), int(num_kv_heads or num_heads), int(tokens_per_chapter), float(routed_scale),
           compute_dtype or h.dtype)
    return _TokenRoutedAttention.apply(h, shared_memory, routed_memory, token_chapter_indices, chapter_weights,
                                       wq, wk, wv, wo, cfg)


class _Linear(torch.autograd.Function):
    """y = x W^T by the projection kernels (nn.Linear without bias), differentiable in x and W."""

    @staticmethod
    def forward(ctx, x, w, cd):
        x2 = ops.cast(x.reshape(-1, x.shape[-1]).contiguous(), cd)
        wc = ops.cast(w.contiguous(), cd)
        ctx.save_for_backward(x2, wc)
        ctx.meta = (x.shape, x.dtype, w.dtype, cd)
        return ops.gemm(x2, wc).view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, g):
        x2, wc = ctx.saved_tensors
        shape, x_dtype, w_dtype, cd = ctx.meta
        g2 = ops.cast(g.reshape(-1, g.shape[-1]).contiguous(), cd)
        d_x = ops.gemm(g2, wc, b_kmajor=False).view(shape).to(x_dtype) if ctx.needs_input_grad[0] else None
        d_w = (ops.gemm(g2, x2, a_kmajor=False, b_kmajor=False, out_dtype=torch.float32).to(w_dtype)
               if ctx.needs_input_grad[1] else None)
        return d_x, d_w, None


def linear(x: torch.Tensor, w: torch.Tensor, compute_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    return _Linear.apply(x, w, compute_dtype or x.dtype)


class _DenseAttention(torch.autograd.Function):
    """softmax(q K^T scale) V for q [B, L, H*D] and kv [B, N, 2*HK*D] (K heads then V heads per row)."""

    @staticmethod
    def forward(ctx, q, kv, num_heads, num_kv_heads, scale):
        o, lse = ops.attn_fwd(q, kv, num_heads, num_kv_heads, scale)
        ctx.save_for_backward(q, kv, o, lse)
        ctx.cfg = (num_heads, num_kv_heads, scale)
        return o

    @staticmethod
    def backward(ctx, g):
        q, kv, o, lse = ctx.saved_tensors
        d_q, d_kv = ops.attn_bwd(q, kv, o, lse, g.contiguous(), *ctx.cfg)
        return d_q, d_kv, None, None, None


def token_routed_attention_joint(h, shared_memory, routed_memory, token_chapter_indices, wq, wk, wv, wo, *,
                                 num_heads: int, num_kv_heads: Optional[int], tokens_per_chapter: int,
                                 routed_scale: float = 1.0, compute_dtype: Optional[torch.dtype] = None):
    """Token-routed attention WITHOUT chapter weights (memory_attention.py:688-704): the selected chapters of a
    token share one softmax; out = Wo [ attn(q, shared) + rho * attn(q, selected chapters) ].  Composed from the
    differentiable projection, dense-attention and per-token sparse-attention operators."""
    from .memory_cross_attn import MemoryCrossAttnFunction
    cd = compute_dtype or h.dtype
    hk = int(num_kv_heads or num_heads)
    b, l, d = h.shape
    rows = b * l
    head_dim = d // num_heads
    scale = head_dim ** -0.5
    q = linear(h.reshape(1, rows, d), wq, cd)                                        # [1, rows, H*D]
    comb = None
    if shared_memory is not None and shared_memory.numel() > 0:
        kv_sh = torch.cat([linear(shared_memory, wk, cd), linear(shared_memory, wv, cd)], dim=-1).unsqueeze(0)
        pad = (-rows) % 64 if cd == torch.bfloat16 else 0
        q_sh = q if pad == 0 else torch.cat([q, q.new_zeros(1, pad, q.shape[-1])], dim=1)
        comb = _DenseAttention.apply(q_sh, kv_sh, num_heads, hk, scale)[:, :rows]
    k_sel = token_chapter_indices.shape[-1]
    if routed_memory is not None and routed_memory.numel() > 0 and k_sel > 0 and tokens_per_chapter > 0:
        k4 = linear(routed_memory, wk, cd).view(1, -1, hk, head_dim)
        v4 = linear(routed_memory, wv, cd).view(1, -1, hk, head_dim)
        bidx = token_chapter_indices.reshape(1, rows, 1, k_sel).expand(1, rows, hk, k_sel).to(torch.int32).contiguous()
        routed = MemoryCrossAttnFunction.apply(q.view(1, rows, num_heads, head_dim).contiguous(), k4.contiguous(),
                                               v4.contiguous(), bidx, int(tokens_per_chapter), scale)
        routed = routed.view(1, rows, -1) * float(routed_scale)
        comb = routed if comb is None else comb + routed
    if comb is None:
        comb = q.new_zeros(1, rows, d)
    return linear(comb, wo, cd).view(b, l, -1).to(h.dtype)
