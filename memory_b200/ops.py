"""Tensor-level wrappers of the C-ABI entry points: allocate outputs, pass raw pointers.

Every function requires CUDA tensors; nothing here computes on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from . import _lib as L


def _contig(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else (t if t.is_contiguous() else t.contiguous())


# Kernel-launch accounting and optional per-call CUDA-event timing (used by the benchmark).
LAUNCHES = 0
TIMER = None   # when a dict: name -> list of (start_event, end_event) on the current stream
LAUNCH_HOOK = None   # when callable: called with "<operator>:<bf16|f32|...>" for every operator call (tests use it to
                     # assert which arithmetic path ran)

_DTYPE_TAG = {torch.bfloat16: "bf16", torch.float32: "f32", torch.float16: "f16"}


def _instrument(name: str, launches):
    """Counts the kernels a wrapper launches (``launches`` is an int or a callable on the call's
    arguments) and, when ``TIMER`` is set, brackets the call with CUDA events."""
    def deco(fn):
        def wrapped(*args, **kwargs):
            global LAUNCHES
            n = launches(*args, **kwargs) if callable(launches) else launches
            LAUNCHES += n
            if LAUNCH_HOOK is not None:
                base = (name(*args, **kwargs) if callable(name) else name).split(":")[0]
                first = next((a for a in args if torch.is_tensor(a)), None)
                LAUNCH_HOOK(base + ":" + (_DTYPE_TAG.get(first.dtype, str(first.dtype)) if first is not None else "-"))
            if TIMER is None:
                return fn(*args, **kwargs)
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*args, **kwargs)
            e1.record()
            label = name(*args, **kwargs) if callable(name) else name
            TIMER.setdefault(label, []).append((e0, e1))
            return out
        wrapped.__name__ = fn.__name__
        wrapped.__doc__ = fn.__doc__
        return wrapped
    return deco


# --------------------------------------------------------------------------------------------
# router
# --------------------------------------------------------------------------------------------
def _router_shape(h: torch.Tensor, num_chapters: int, top_k: int, num_shared: int, routed_scale: float):
    b, l, d = h.shape
    return L.RouterShape(b, l, d, num_chapters, top_k, num_shared, float(routed_scale), L.dtype_code(h.dtype))


def router_selected_k(num_chapters: int, top_k: int, num_shared: int) -> int:
    return max(0, min(int(top_k), int(num_chapters) - int(num_shared)))


def _router_fwd_launches(*a, **k):
    parts = k.get("parts", 3)
    with_losses = a[6] if len(a) > 6 else k.get("with_losses")
    return (4 if parts & 1 else 0) + (2 if (parts & 2) and with_losses else 0)


@_instrument(lambda *a, **k: "router_fwd" if k.get("parts", 3) == 3 else "router_fwd:parts%d" % k["parts"],
             _router_fwd_launches)
def router_fwd(h: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], top_k: int,
               num_shared: int, routed_scale: float, with_losses: bool, parts: int = 3,
               out: Optional[Dict[str, torch.Tensor]] = None,
               pooled: Optional[torch.Tensor] = None,
               logits: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
    """``parts`` (1 = pooling, logits, selection; 2 = loss terms) runs a subset on the current stream; pass the dict
    returned by the first call as ``out`` to the second.  ``pooled`` ([B, d] fp32): pooled states computed by
    another rule (see :func:`pool_weighted_fwd`); the mean-pool is then skipped.  ``logits`` ([B, C] fp32, without
    the bias): pooled x W^T already computed by a projection kernel; only the bias is added (in place)."""
    L.require_cuda(h, weight, bias)
    if h.dim() != 3:
        raise ValueError(f"hidden_states must be 3D (B, T, D), got shape {tuple(h.shape)}")
    h = _contig(h)
    weight = _contig(weight.float())
    bias = _contig(bias.float()) if bias is not None else None
    b, l, d = h.shape
    c = weight.shape[0]
    k = router_selected_k(c, top_k, num_shared)
    dev = h.device
    s = _router_shape(h, c, top_k, num_shared, routed_scale)
    f32 = dict(dtype=torch.float32, device=dev)
    lib = L.lib()
    if pooled is not None and logits is not None:
        ws_bytes = lib.moc_router_workspace_bytes_parts(C.byref(s), 1 | 2 | 8 | 16, 0)   # loss partials only
    else:
        ws_bytes = lib.moc_router_workspace_bytes(C.byref(s))
    if out is None:
        out = {
            "pooled": torch.empty(b, d, **f32), "logits": torch.empty(b, c, **f32), "probs": torch.empty(b, c, **f32),
            "idx": torch.empty(b, k, dtype=torch.int64, device=dev), "weights": torch.empty(b, k, **f32),
            "comb_idx": torch.empty(b, num_shared + k, dtype=torch.int32, device=dev),
            "comb_w": torch.empty(b, num_shared + k, **f32),
            "row_stats": torch.empty(b, 4, **f32), "chapter_stats": torch.empty(2, c, **f32),
            "losses": torch.empty(4, **f32) if with_losses else None,
            "_ws": torch.empty(ws_bytes, dtype=torch.uint8, device=dev),
        }
    ws_bytes = out["_ws"].numel()
    if pooled is not None:
        out["pooled"] = _contig(pooled.float())
        parts = int(parts) | 8
    if logits is not None:
        if logits.dtype != torch.float32 or tuple(logits.shape) != (b, c) or not logits.is_contiguous():
            raise ValueError("logits must be a contiguous fp32 [rows, num_chapters] tensor")
        out["logits"] = logits
        parts = int(parts) | 16
    rc = lib.moc_router_fwd_parts(C.byref(s), L.ptr(h), L.ptr(weight), L.ptr(bias), L.ptr(out["pooled"]),
                                  L.ptr(out["logits"]), L.ptr(out["probs"]), L.ptr(out["idx"]), L.ptr(out["weights"]),
                                  L.ptr(out["comb_idx"]), L.ptr(out["comb_w"]), L.ptr(out["row_stats"]),
                                  L.ptr(out["chapter_stats"]), L.ptr(out["losses"]), L.ptr(out["_ws"]), ws_bytes,
                                  int(parts), L.ptr(L.status_word(dev)), L.stream_ptr(dev))
    L.check(rc, "moc_router_fwd_parts")
    return out


def _router_bwd_launches(*a, **k):
    parts = k.get("parts", 7)
    want_dh = a[-1] if len(a) > 10 else k.get("want_dh")
    return (1 if parts & 1 else 0) + (1 if parts & 2 else 0) + ((3 if want_dh else 2) if parts & 4 else 0)


@_instrument(lambda *a, **k: "router_bwd" if k.get("parts", 7) == 7 else "router_bwd:parts%d" % k["parts"],
             _router_bwd_launches)
def router_bwd(h_shape, h_dtype, weight: torch.Tensor, saved: Dict[str, torch.Tensor], top_k: int,
               num_shared: int, routed_scale: float, d_weights: Optional[torch.Tensor],
               d_comb_w: Optional[torch.Tensor], d_losses: Optional[torch.Tensor],
               want_dh: bool, d_h_accum: Optional[torch.Tensor] = None, parts: int = 7,
               out: Optional[Dict[str, torch.Tensor]] = None, logits_only: bool = False) -> Dict[str, torch.Tensor]:
    """``d_h_accum`` ([B, L, d] of the hidden-state dtype): the hidden-state gradient is added into it instead
    of being written to a fresh tensor (the attention branch's gradient of the same hidden states).
    ``parts`` (1 = d_logits, 2 = d_w / d_bias, 4 = d_pooled / d_h) runs a subset on the current stream; pass the
    dict returned by the first call as ``out`` to the later ones so they share buffers.  ``logits_only`` (with
    parts = 1): no later part will run on these buffers, so no batch-sized scratch is allocated."""
    if logits_only and parts != 1:
        raise ValueError("logits_only goes with parts=1")
    b, l, d = h_shape
    c = weight.shape[0]
    dev = weight.device
    s = L.RouterShape(b, l, d, c, top_k, num_shared, float(routed_scale), L.dtype_code(h_dtype))
    f32 = dict(dtype=torch.float32, device=dev)
    weight = _contig(weight.float())
    lib = L.lib()
    if out is None:
        if logits_only:
            # logit gradient only (the token-level path finishes with projection kernels): no batch-sized scratch
            ws_bytes = max(16, lib.moc_router_workspace_bytes_parts(C.byref(s), 0, 1))
            out = {"d_logits": torch.empty(b, c, **f32), "d_w": torch.empty(1, **f32), "d_bias": torch.empty(1, **f32),
                   "d_pooled": torch.empty(1, **f32), "d_h": None,
                   "_ws": torch.empty(ws_bytes, dtype=torch.uint8, device=dev)}
        else:
            ws_bytes = lib.moc_router_workspace_bytes(C.byref(s))
            out = {"d_logits": torch.empty(b, c, **f32), "d_w": torch.empty(c, d, **f32),
                   "d_bias": torch.empty(c, **f32), "d_pooled": torch.empty(b, d, **f32), "d_h": None,
                   "_ws": torch.empty(ws_bytes, dtype=torch.uint8, device=dev)}
    ws_bytes = out["_ws"].numel()
    accumulate = 0
    if want_dh and (parts & 4):
        if d_h_accum is not None:
            if d_h_accum.dtype != h_dtype or tuple(d_h_accum.shape) != (b, l, d) or not d_h_accum.is_contiguous():
                raise ValueError("d_h_accum must be a contiguous [B, L, d] tensor of the hidden-state dtype")
            out["d_h"], accumulate = d_h_accum, 1
        else:
            out["d_h"] = torch.empty(b, l, d, dtype=h_dtype, device=dev)
    rc = lib.moc_router_bwd_parts(C.byref(s), L.ptr(weight), L.ptr(saved["pooled"]), L.ptr(saved["probs"]),
                                  L.ptr(saved["idx"]), L.ptr(saved["weights"]), L.ptr(saved["comb_w"]),
                                  L.ptr(saved["row_stats"]), L.ptr(saved["chapter_stats"]),
                                  L.ptr(_contig(d_weights)), L.ptr(_contig(d_comb_w)), L.ptr(_contig(d_losses)),
                                  L.ptr(out["d_logits"]), L.ptr(out["d_w"]), L.ptr(out["d_bias"]),
                                  L.ptr(out["d_pooled"]), L.ptr(out["d_h"]) if (parts & 4) else None, accumulate,
                                  L.ptr(out["_ws"]), ws_bytes, int(parts), L.ptr(L.status_word(dev)),
                                  L.stream_ptr(dev))
    L.check(rc, "moc_router_bwd_parts")
    return out


def rolling_pool_coefficients(seq: int, window) -> torch.Tensor:
    """c[s] such that sum_s c[s] h[:, s] equals the reference's ``_sequence_rolling_pool`` (router.py:159-195):
    the mean over t of mean(h[max(0, t-w+1) .. t]).  Position s belongs to the windows ending at t = s .. s+w-1
    (clipped to the sequence), each contributing 1 / (L * window_length(t)).  Host arithmetic in fp64."""
    if seq <= 0:
        raise ValueError("sequence length must be > 0")
    w = seq if window is None else int(window)
    if w <= 0:
        raise ValueError(f"rolling_window_size must be > 0, got {window}")
    w = min(w, seq)
    t = torch.arange(seq, dtype=torch.float64)
    inv_len = 1.0 / torch.clamp(t + 1, max=w)                  # window ending at t holds min(t + 1, w) positions
    csum = torch.cat([torch.zeros(1, dtype=torch.float64), inv_len.cumsum(0)])
    hi = torch.clamp(torch.arange(seq) + w, max=seq)            # windows ending at s .. min(s + w, L) - 1 cover s
    return ((csum[hi] - csum[torch.arange(seq)]) / seq).float()


@_instrument("pool_weighted_fwd", 2)
def pool_weighted_fwd(h: torch.Tensor, pos_weight: torch.Tensor) -> torch.Tensor:
    L.require_cuda(h, pos_weight)
    h = _contig(h)
    b, l, d = h.shape
    pooled = torch.empty(b, d, dtype=torch.float32, device=h.device)
    ws = torch.empty(b * 32 * d, dtype=torch.float32, device=h.device)
    rc = L.lib().moc_pool_weighted_fwd(L.ptr(h), L.dtype_code(h.dtype), L.ptr(_contig(pos_weight.float())),
                                       L.ptr(pooled), b, l, d, L.ptr(ws), ws.numel() * 4, L.stream_ptr(h.device))
    L.check(rc, "moc_pool_weighted_fwd")
    return pooled


@_instrument("pool_weighted_bwd", 1)
def pool_weighted_bwd(d_pooled: torch.Tensor, pos_weight: torch.Tensor, h_shape, h_dtype,
                      d_h_accum: Optional[torch.Tensor] = None) -> torch.Tensor:
    b, l, d = h_shape
    d_h = d_h_accum if d_h_accum is not None else torch.empty(b, l, d, dtype=h_dtype, device=d_pooled.device)
    rc = L.lib().moc_pool_weighted_bwd(L.ptr(_contig(d_pooled)), L.ptr(_contig(pos_weight.float())), L.ptr(d_h),
                                       L.dtype_code(h_dtype), b, l, d, 1 if d_h_accum is not None else 0,
                                       L.stream_ptr(d_pooled.device))
    L.check(rc, "moc_pool_weighted_bwd")
    return d_h


def peer_barrier(flag_arrays, rank: int, epoch: int, poll_limit: int = 1 << 22) -> None:
    """Barrier over flag words in the ranks' (peer-mapped) memory on the current stream; ``flag_arrays[r]`` is rank
    r's uint32/int32 [world] array, ``epoch`` grows by one per call.  Bounded: a peer that never arrives leaves
    MOC_DEV_TIMEOUT in the status word instead of a hung kernel."""
    world = len(flag_arrays)
    dev = flag_arrays[rank].device
    arr = (C.c_void_p * world)(*[t.data_ptr() for t in flag_arrays])
    rc = L.lib().moc_peer_barrier(arr, int(rank), world, int(epoch) & 0xFFFFFFFF, int(poll_limit),
                                  L.ptr(L.status_word(dev)), L.stream_ptr(dev))
    L.check(rc, "moc_peer_barrier")


def wait_probe(device, expected: int, arrivals: int, poll_limit: int):
    """Runs the bounded-wait self-test kernel; returns (wait succeeded, second wait result, abort flag)."""
    out = torch.zeros(3, dtype=torch.int32, device=device)
    rc = L.lib().moc_wait_probe(int(expected), int(arrivals), int(poll_limit), L.ptr(L.status_word(device)),
                                L.ptr(out), L.stream_ptr(device))
    L.check(rc, "moc_wait_probe")
    return tuple(int(v) for v in out.tolist())


# --------------------------------------------------------------------------------------------
# gather
# --------------------------------------------------------------------------------------------
@_instrument("gather_rows_fwd", 1)
def gather_rows_fwd(bank: torch.Tensor, tokens_per_chapter: int, comb_idx: torch.Tensor,
                    comb_w: Optional[torch.Tensor], norm_type: Optional[str], eps: float,
                    out_dtype: torch.dtype) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    L.require_cuda(bank, comb_idx, comb_w)
    bank = _contig(bank)
    comb_idx = _contig(comb_idx.to(torch.int32))
    b, k = comb_idx.shape
    n_rows, d = bank.shape
    t = int(tokens_per_chapter)
    out = torch.empty(b, k * t, d, dtype=out_dtype, device=bank.device)
    code = L.NORM_CODES[norm_type]
    stats = torch.empty(b * k * t, 2, dtype=torch.float32, device=bank.device) if code != 0 else None
    rc = L.lib().moc_gather_rows_fwd(L.ptr(bank), L.dtype_code(bank.dtype), n_rows, d, t, L.ptr(comb_idx),
                                     L.ptr(_contig(comb_w)), b, k, code, float(eps), L.ptr(out),
                                     L.dtype_code(out_dtype), L.ptr(stats), L.ptr(L.status_word(bank.device)),
                                     L.stream_ptr(bank.device))
    L.check(rc, "moc_gather_rows_fwd")
    return out, stats


@_instrument("chapter_segments", 1)
def chapter_segments(comb_idx: torch.Tensor, num_chapters: int) -> Dict[str, torch.Tensor]:
    comb_idx = _contig(comb_idx.to(torch.int32))
    n = comb_idx.numel()
    dev = comb_idx.device
    i32 = dict(dtype=torch.int32, device=dev)
    seg = {"uniq": torch.empty(n, **i32), "seg_offsets": torch.empty(n + 1, **i32),
           "seg_pairs": torch.empty(n, **i32), "pair_to_uniq": torch.empty(n, **i32),
           "num_unique": torch.empty(1, **i32)}
    rc = L.lib().moc_chapter_segments(L.ptr(comb_idx), n, int(num_chapters), L.ptr(seg["uniq"]),
                                      L.ptr(seg["seg_offsets"]), L.ptr(seg["seg_pairs"]),
                                      L.ptr(seg["pair_to_uniq"]), L.ptr(seg["num_unique"]),
                                      L.ptr(L.status_word(dev)), L.stream_ptr(dev))
    L.check(rc, "moc_chapter_segments")
    return seg


@_instrument("gather_rows_bwd", 2)
def gather_rows_bwd(d_mem: torch.Tensor, bank: torch.Tensor, tokens_per_chapter: int, comb_idx: torch.Tensor,
                    comb_w: Optional[torch.Tensor], norm_type: Optional[str], eps: float,
                    row_stats: Optional[torch.Tensor], seg: Dict[str, torch.Tensor],
                    want_dw: bool = True, want_bank: bool = True, wire_copy: Optional[list] = None
                    ) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """``wire_copy``: pass an empty list to also get the compact rows in bf16 (appended to it): the copy a
    gradient exchange sends when it is asked to halve its volume."""
    bank = _contig(bank)
    d_mem = _contig(d_mem)
    comb_idx = _contig(comb_idx.to(torch.int32))
    b, k = comb_idx.shape
    n_rows, d = bank.shape
    t = int(tokens_per_chapter)
    dev = bank.device
    d_comb_w = torch.empty(b, k, dtype=torch.float32, device=dev) if want_dw else None
    bank_grad = torch.empty(b * k * t, d, dtype=torch.float32, device=dev) if want_bank else None
    wire = None
    if want_bank and wire_copy is not None:
        wire = torch.empty(b * k * t, d, dtype=torch.bfloat16, device=dev)
        wire_copy.append(wire)
    rc = L.lib().moc_gather_rows_bwd(L.ptr(d_mem), L.dtype_code(d_mem.dtype), L.ptr(bank), L.dtype_code(bank.dtype),
                                     n_rows, d, t, L.ptr(comb_idx), L.ptr(_contig(comb_w)), b, k,
                                     L.NORM_CODES[norm_type], float(eps), L.ptr(row_stats), L.ptr(seg["uniq"]),
                                     L.ptr(seg["seg_offsets"]), L.ptr(seg["seg_pairs"]), L.ptr(seg["num_unique"]),
                                     L.ptr(d_comb_w), L.ptr(bank_grad), L.ptr(wire), L.ptr(L.status_word(dev)),
                                     L.stream_ptr(dev))
    L.check(rc, "moc_gather_rows_bwd")
    return d_comb_w, bank_grad


@_instrument("row_inv_rms", 1)
def row_inv_rms(bank: torch.Tensor, eps: float) -> torch.Tensor:
    """1 / sqrt(mean(row^2) + eps) of every bank row (fp32 [rows])."""
    L.require_cuda(bank)
    bank = _contig(bank)
    out = torch.empty(bank.shape[0], dtype=torch.float32, device=bank.device)
    rc = L.lib().moc_row_inv_rms(L.ptr(bank), L.dtype_code(bank.dtype), bank.shape[0], bank.shape[1], float(eps),
                                 L.ptr(out), L.stream_ptr(bank.device))
    L.check(rc, "moc_row_inv_rms")
    return out


@_instrument("chapter_row_scale", 1)
def chapter_row_scale(comb_idx: torch.Tensor, comb_w: Optional[torch.Tensor], inv_rms: Optional[torch.Tensor],
                      bank_rows: int, tokens_per_chapter: int) -> torch.Tensor:
    """scale[pair*T + r] = comb_w[pair] * inv_rms[row] (inv_rms None: no normalisation); fp32 [n_pairs*T]."""
    comb_idx = _contig(comb_idx.to(torch.int32))
    n = comb_idx.numel()
    t = int(tokens_per_chapter)
    out = torch.empty(n * t, dtype=torch.float32, device=comb_idx.device)
    rc = L.lib().moc_chapter_row_scale(L.ptr(comb_idx), L.ptr(_contig(comb_w)), L.ptr(_contig(inv_rms)), int(bank_rows),
                                       n, t, L.ptr(out), L.ptr(L.status_word(comb_idx.device)),
                                       L.stream_ptr(comb_idx.device))
    L.check(rc, "moc_chapter_row_scale")
    return out


@_instrument("gather_rows_bwd_prescaled", 2)
def gather_rows_bwd_prescaled(g: torch.Tensor, bank: torch.Tensor, tokens_per_chapter: int, comb_idx: torch.Tensor,
                              comb_w: Optional[torch.Tensor], inv_rms: Optional[torch.Tensor],
                              seg: Dict[str, torch.Tensor], want_dw: bool = True, want_bank: bool = True,
                              wire_copy: Optional[list] = None, wire_only: bool = False):
    """Chapter-weight gradient and compact bank gradient from g = (row scale) * dM~ (see ``moc_row_inv_rms``).
    ``wire_copy`` (a list) receives the same rows in bf16; with ``wire_only`` the fp32 rows are not written at all
    (returned as None): a data-parallel step forms its mean gradient from the ranks' bf16 rows."""
    bank, g = _contig(bank), _contig(g)
    comb_idx = _contig(comb_idx.to(torch.int32))
    n = comb_idx.numel()
    n_rows, d = bank.shape
    t = int(tokens_per_chapter)
    dev = bank.device
    d_comb_w = torch.empty(comb_idx.shape, dtype=torch.float32, device=dev) if want_dw else None
    wire_only = bool(wire_only and want_bank and wire_copy is not None and d % 8 == 0 and d <= 1024)
    bank_grad = torch.empty(n * t, d, dtype=torch.float32, device=dev) if (want_bank and not wire_only) else None
    wire = None
    if want_bank and wire_copy is not None:
        wire = torch.empty(n * t, d, dtype=torch.bfloat16, device=dev)
        wire_copy.append(wire)
    rc = L.lib().moc_gather_rows_bwd_prescaled(L.ptr(g), L.dtype_code(g.dtype), L.ptr(bank), L.dtype_code(bank.dtype),
                                               n_rows, d, t, L.ptr(comb_idx), L.ptr(_contig(comb_w)), n,
                                               L.ptr(_contig(inv_rms)), L.ptr(seg["uniq"]), L.ptr(seg["seg_offsets"]),
                                               L.ptr(seg["seg_pairs"]), L.ptr(seg["num_unique"]), L.ptr(d_comb_w),
                                               L.ptr(bank_grad), L.ptr(wire), L.ptr(L.status_word(dev)),
                                               L.stream_ptr(dev))
    L.check(rc, "moc_gather_rows_bwd_prescaled")
    return d_comb_w, bank_grad


@_instrument("bank_grad_merge", 2)
def bank_grad_merge(rank_rows, ids_all: torch.Tensor, counts: torch.Tensor, tokens_per_chapter: int,
                    num_chapters: int, scale: float = 1.0, out: Optional[Dict[str, torch.Tensor]] = None,
                    out_dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """Sum of the ranks' compact gradient rows over the union of their chapter lists.

    ``rank_rows``: one [per_rank*T, d] tensor per rank (all fp32 or all bf16); ``ids_all`` int32 [world, per_rank];
    ``counts`` int32 [world].  Returns {"uniq", "num_unique", "rows" [cap*T, d] in ``out_dtype`` (sums are formed in
    fp32), scratch...}; pass the dict back as ``out`` to reuse its buffers."""
    world, per_rank = ids_all.shape
    t, d = int(tokens_per_chapter), rank_rows[0].shape[1]
    dev = ids_all.device
    L.require_cuda(ids_all, counts, *rank_rows)
    if any(r.dtype != rank_rows[0].dtype or not r.is_contiguous() for r in rank_rows):
        raise ValueError("rank_rows must be contiguous tensors of one dtype")
    n = world * per_rank
    cap = min(n, int(num_chapters))
    if out is None:
        i32 = dict(dtype=torch.int32, device=dev)
        out = {"uniq": torch.empty(n, **i32), "seg_offsets": torch.empty(n + 1, **i32),
               "seg_pairs": torch.empty(n, **i32), "pair_to_uniq": torch.empty(n, **i32),
               "num_unique": torch.empty(1, **i32),
               "rows": torch.empty(cap * t, d, dtype=out_dtype, device=dev)}
    arr = (C.c_void_p * world)(*[r.data_ptr() for r in rank_rows])
    rc = L.lib().moc_bank_grad_merge_to(arr, L.dtype_code(rank_rows[0].dtype), world, L.ptr(_contig(ids_all)),
                                        L.ptr(_contig(counts)), per_rank, t, d, int(num_chapters), float(scale),
                                        L.ptr(out["uniq"]), L.ptr(out["seg_offsets"]), L.ptr(out["seg_pairs"]),
                                        L.ptr(out["pair_to_uniq"]), L.ptr(out["num_unique"]), L.ptr(out["rows"]),
                                        L.dtype_code(out["rows"].dtype), out["rows"].shape[0],
                                        L.ptr(L.status_word(dev)), L.stream_ptr(dev))
    L.check(rc, "moc_bank_grad_merge_to")
    return out


@_instrument("bank_adamw_step", 2)
def bank_adamw_step(param: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, uniq: torch.Tensor,
                    num_unique: torch.Tensor, grad_rows: torch.Tensor, tokens_per_chapter: int, *, lr: float,
                    betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01, step: int = 1,
                    grad_scale: float = 1.0, shadow: Optional[torch.Tensor] = None,
                    workspace: Optional[torch.Tensor] = None) -> None:
    """In-place AdamW update of every bank row from a compact gradient (see ``moc_bank_adamw_step``)."""
    L.require_cuda(param, exp_avg, exp_avg_sq, uniq, num_unique, grad_rows, shadow)
    for t in (param, exp_avg, exp_avg_sq, grad_rows):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError("parameter, moments and gradient rows must be contiguous fp32 tensors")
    if shadow is not None and (shadow.dtype != torch.bfloat16 or shadow.shape != param.shape or not shadow.is_contiguous()):
        raise TypeError("shadow must be a contiguous bf16 tensor shaped like the parameter")
    rows, d = param.shape
    c = rows // int(tokens_per_chapter)
    lib = L.lib()
    need = lib.moc_bank_adamw_workspace_bytes(c)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=param.device)
    rc = lib.moc_bank_adamw_step(L.ptr(param), L.ptr(exp_avg), L.ptr(exp_avg_sq), rows, d, int(tokens_per_chapter),
                                 L.ptr(uniq), L.ptr(num_unique), uniq.numel(), L.ptr(grad_rows), float(grad_scale),
                                 float(lr), float(betas[0]), float(betas[1]), float(eps), float(weight_decay),
                                 int(step), L.ptr(shadow), L.ptr(workspace), workspace.numel(),
                                 L.ptr(L.status_word(param.device)), L.stream_ptr(param.device))
    L.check(rc, "moc_bank_adamw_step")


@_instrument("rows_sqnorm", 2)
def rows_sqnorm(rows: torch.Tensor, num_unique: torch.Tensor, tokens_per_chapter: int) -> torch.Tensor:
    """Sum of squares of the valid part of a compact gradient ([1] fp32, no host synchronisation)."""
    L.require_cuda(rows, num_unique)
    out = torch.empty(1, dtype=torch.float32, device=rows.device)
    ws = torch.empty(592, dtype=torch.float32, device=rows.device)
    rc = L.lib().moc_rows_sqnorm(L.ptr(_contig(rows)), L.ptr(num_unique), int(tokens_per_chapter), rows.shape[1],
                                 L.ptr(out), L.ptr(ws), ws.numel() * 4, L.stream_ptr(rows.device))
    L.check(rc, "moc_rows_sqnorm")
    return out


@_instrument("scatter_bank_grad", 1)
def scatter_bank_grad(bank_grad: torch.Tensor, seg: Dict[str, torch.Tensor], tokens_per_chapter: int,
                      dense: torch.Tensor) -> None:
    """dense[uniq[u]*T + r] += bank_grad[u*T + r] for the chapters listed in ``seg``."""
    n_rows, d = dense.shape
    rc = L.lib().moc_scatter_bank_grad(L.ptr(bank_grad), L.ptr(seg["uniq"]), L.ptr(seg["num_unique"]),
                                       seg["uniq"].numel(), int(tokens_per_chapter), d, L.ptr(dense), n_rows,
                                       L.ptr(L.status_word(dense.device)), L.stream_ptr(dense.device))
    L.check(rc, "moc_scatter_bank_grad")


# --------------------------------------------------------------------------------------------
# projections
# --------------------------------------------------------------------------------------------
def _gemm_label(a, b, **k):
    tag = k.get("tag")
    return "gemm:" + tag if tag else "gemm"


@_instrument(_gemm_label, 1)
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_kmajor: bool = True, b_kmajor: bool = True,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, accumulate: bool = False,
         split_k: int = 1, row_scale: Optional[torch.Tensor] = None, scale_block_rows: int = 1,
         a_row_blocks: Optional[torch.Tensor] = None, a_block_rows: int = 0, m: Optional[int] = None,
         residual: Optional[torch.Tensor] = None, tag: Optional[str] = None,
         b_row_blocks: Optional[torch.Tensor] = None, b_block_rows: int = 0, k: Optional[int] = None) -> torch.Tensor:
    """C[M,N] (+)= op(A) op(B) (+ residual).  a_kmajor: A stored [M,K] else [K,M]; b_kmajor: B stored [N,K]
    else [K,N]; residual: fp32 [M,N] added in the epilogue.  ``a_row_blocks`` / ``b_row_blocks``: gather lists over
    the rows of a K-major A / the K rows of an MN-major B (blocks of ``*_block_rows`` rows, e.g. chapters of the
    bank); ``m`` / ``k`` give the gathered extent."""
    L.require_cuda(a, b)
    if a.dtype != b.dtype:
        raise TypeError("projection operands must share a dtype")
    a, b = _contig(a), _contig(b)
    if a_row_blocks is not None:
        mm, kk = int(m), a.shape[1]
    elif a_kmajor:
        mm, kk = a.shape
    else:
        kk, mm = a.shape
    if b_kmajor:
        nn, kb = b.shape
    else:
        kb, nn = b.shape
    if b_row_blocks is not None:
        if b_kmajor or a_row_blocks is not None or k is None:
            raise ValueError("b_row_blocks needs b_kmajor=False, no a_row_blocks and the gathered extent k")
        kb = int(k)
    if kk != kb:
        raise ValueError(f"inner dimensions differ: {kk} vs {kb}")
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else a.dtype
    if out is None:
        out = (torch.zeros if (split_k > 1 and not accumulate) else torch.empty)(mm, nn, dtype=out_dtype, device=a.device)
    g = L.GemmDesc(L.dtype_code(a.dtype), L.dtype_code(out_dtype), mm, nn, kk, int(a_kmajor), int(b_kmajor),
                   a.stride(0), b.stride(0), out.stride(0), int(accumulate), int(split_k), int(scale_block_rows),
                   int(a_block_rows), a.shape[0], None, 0)
    if residual is not None:
        if residual.dtype != torch.float32 or tuple(residual.shape) != (mm, nn) or residual.stride(1) != 1:
            raise ValueError("residual must be fp32 [M, N] with unit column stride")
        L.require_cuda(residual)
        g.residual, g.ldr = L.ptr(residual), residual.stride(0)
    if b_row_blocks is not None:
        rc = L.lib().moc_gemm_gather_b(C.byref(g), L.ptr(a), L.ptr(b), L.ptr(out), L.ptr(_contig(row_scale)),
                                       L.ptr(_contig(b_row_blocks)), int(b_block_rows), b.shape[0],
                                       L.ptr(L.status_word(a.device)), L.stream_ptr(a.device))
        L.check(rc, "moc_gemm_gather_b")
        return out
    rc = L.lib().moc_gemm(C.byref(g), L.ptr(a), L.ptr(b), L.ptr(out), L.ptr(_contig(row_scale)),
                          L.ptr(_contig(a_row_blocks)), L.ptr(L.status_word(a.device)), L.stream_ptr(a.device))
    L.check(rc, "moc_gemm")
    return out


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
def _attn_shape(q: torch.Tensor, kv: torch.Tensor, num_heads: int, num_kv_heads: int, scale: float):
    b, l, hd = q.shape
    n_sel = kv.shape[1]
    d = hd // num_heads
    if kv.shape[2] != 2 * num_kv_heads * d:
        raise ValueError("kv must be [B, n_sel, 2 * num_kv_heads * head_dim]")
    return L.AttnShape(b, l, n_sel, num_heads, num_kv_heads, d, float(scale), L.dtype_code(q.dtype))


@_instrument("attn_fwd", 1)
def attn_fwd(q: torch.Tensor, kv: torch.Tensor, num_heads: int, num_kv_heads: int,
             scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    L.require_cuda(q, kv)
    q, kv = _contig(q), _contig(kv)
    s = _attn_shape(q, kv, num_heads, num_kv_heads, scale)
    o = torch.empty_like(q)
    lse = torch.empty(s.batch, num_heads, s.seq, dtype=torch.float32, device=q.device)
    rc = L.lib().moc_attn_fwd(C.byref(s), L.ptr(q), L.ptr(kv), L.ptr(o), L.ptr(lse),
                              L.ptr(L.status_word(q.device)), L.stream_ptr(q.device))
    L.check(rc, "moc_attn_fwd")
    return o, lse


def _attn_bwd_launches(*a, **k):
    parts = k.get("parts")
    if parts is not None:
        return bin(int(parts)).count("1")
    return 3 if a[0].dtype == torch.bfloat16 else 4


@_instrument(lambda *a, **k: "attn_bwd" if k.get("parts") is None else "attn_bwd:parts%d" % k["parts"],
             _attn_bwd_launches)
def attn_bwd(q: torch.Tensor, kv: torch.Tensor, o: torch.Tensor, lse: torch.Tensor, d_o: torch.Tensor,
             num_heads: int, num_kv_heads: int, scale: float, parts: Optional[int] = None,
             buffers=None, kv_row_scale: Optional[torch.Tensor] = None,
             kv_dot: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """dQ and dKV.  ``parts`` (bf16 only) restricts the call to some of its kernels for timing;
    ``buffers`` = (d_q, d_kv, scratch) reuses outputs between such calls.  ``kv_row_scale`` [B*n_sel] fp32 (bf16
    only): dK / dV rows leave multiplied by it (the fused gather-and-project path); ``kv_dot`` fp32
    [B, n_sel/64, HK] then receives per 64-key block and KV head sum_rows(<dK, K> + <dV, V>)."""
    q, kv, o, d_o = _contig(q), _contig(kv), _contig(o), _contig(d_o)
    s = _attn_shape(q, kv, num_heads, num_kv_heads, scale)
    if buffers is None:
        d_q = torch.empty_like(q)
        d_kv = torch.empty_like(kv)
        scratch = torch.empty(6, s.batch, num_heads, s.seq, dtype=torch.float32, device=q.device)
    else:
        d_q, d_kv, scratch = buffers
    if kv_row_scale is not None and parts is not None:
        rc = L.lib().moc_attn_bwd_scaled_parts(C.byref(s), L.ptr(q), L.ptr(kv), L.ptr(o), L.ptr(lse), L.ptr(d_o),
                                               L.ptr(d_q), L.ptr(d_kv), L.ptr(scratch), L.ptr(_contig(kv_row_scale)),
                                               L.ptr(kv_dot), int(parts), L.ptr(L.status_word(q.device)),
                                               L.stream_ptr(q.device))
    elif kv_row_scale is not None:
        rc = L.lib().moc_attn_bwd_scaled(C.byref(s), L.ptr(q), L.ptr(kv), L.ptr(o), L.ptr(lse), L.ptr(d_o),
                                         L.ptr(d_q), L.ptr(d_kv), L.ptr(scratch), L.ptr(_contig(kv_row_scale)),
                                         L.ptr(kv_dot), L.ptr(L.status_word(q.device)), L.stream_ptr(q.device))
    elif parts is None:
        rc = L.lib().moc_attn_bwd(C.byref(s), L.ptr(q), L.ptr(kv), L.ptr(o), L.ptr(lse), L.ptr(d_o), L.ptr(d_q),
                                  L.ptr(d_kv), L.ptr(scratch), L.ptr(L.status_word(q.device)),
                                  L.stream_ptr(q.device))
    else:
        rc = L.lib().moc_attn_bwd_parts(C.byref(s), L.ptr(q), L.ptr(kv), L.ptr(o), L.ptr(lse), L.ptr(d_o),
                                        L.ptr(d_q), L.ptr(d_kv), L.ptr(scratch), int(parts),
                                        L.ptr(L.status_word(q.device)), L.stream_ptr(q.device))
    L.check(rc, "moc_attn_bwd")
    return d_q, d_kv


@_instrument("attn_bwd_static", _attn_bwd_launches)
def attn_bwd_static(q: torch.Tensor, kv: torch.Tensor, o: torch.Tensor, lse: torch.Tensor, d_o: torch.Tensor,
                    num_heads: int, num_kv_heads: int, scale: float, out=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """dQ and dKV through the entry point that allocates nothing: its scratch is a fixed array inside
    the library (6*B*H*L must not exceed ``_lib.ATTN_BWD_STATIC_MAX_FLOATS``).  Pass ``out`` =
    (d_q, d_kv) to keep this wrapper from allocating the outputs either.  Calls that may overlap on
    the GPU must be serialised by the caller, because they share that array."""
    q, kv, o, d_o = _contig(q), _contig(kv), _contig(o), _contig(d_o)
    s = _attn_shape(q, kv, num_heads, num_kv_heads, scale)
    d_q, d_kv = out if out is not None else (torch.empty_like(q), torch.empty_like(kv))
    rc = L.lib().moc_attn_bwd_static(C.byref(s), L.ptr(q), L.ptr(kv), L.ptr(o), L.ptr(lse), L.ptr(d_o),
                                     L.ptr(d_q), L.ptr(d_kv), L.ptr(L.status_word(q.device)),
                                     L.stream_ptr(q.device))
    L.check(rc, "moc_attn_bwd_static")
    return d_q, d_kv


@_instrument("sparse_attn_fwd", 1)
def sparse_attn_fwd(q, k, v, block_indices, block_size: int, scale: float):
    L.require_cuda(q, k, v, block_indices)
    b, tq, hq, d = q.shape
    _, tk, h, _ = k.shape
    s = L.SparseAttnShape(b, tq, tk, hq, h, d, block_indices.shape[-1], int(block_size), float(scale),
                          L.dtype_code(q.dtype))
    o = torch.empty(b, tq, hq, v.shape[-1], dtype=v.dtype, device=q.device)
    lse = torch.empty(b, tq, hq, dtype=torch.float32, device=q.device)
    rc = L.lib().moc_sparse_attn_fwd(C.byref(s), L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(block_indices), L.ptr(o),
                                     L.ptr(lse), L.ptr(L.status_word(q.device)), L.stream_ptr(q.device))
    L.check(rc, "moc_sparse_attn_fwd")
    return o, lse


@_instrument("sparse_attn_bwd", 1)
def sparse_attn_bwd(q, k, v, block_indices, o, lse, d_o, block_size: int, scale: float):
    b, tq, hq, d = q.shape
    _, tk, h, _ = k.shape
    s = L.SparseAttnShape(b, tq, tk, hq, h, d, block_indices.shape[-1], int(block_size), float(scale),
                          L.dtype_code(q.dtype))
    d_q = torch.empty_like(q)
    d_k = torch.empty(k.shape, dtype=torch.float32, device=q.device)
    d_v = torch.empty(v.shape, dtype=torch.float32, device=q.device)
    rc = L.lib().moc_sparse_attn_bwd(C.byref(s), L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(block_indices), L.ptr(o),
                                     L.ptr(lse), L.ptr(_contig(d_o)), L.ptr(d_q), L.ptr(d_k), L.ptr(d_v),
                                     L.ptr(L.status_word(q.device)), L.stream_ptr(q.device))
    L.check(rc, "moc_sparse_attn_bwd")
    return d_q, d_k, d_v


@_instrument("sparse_attn_weighted_fwd", 1)
def sparse_attn_weighted_fwd(q, k, v, block_indices, weights, block_size: int, scale: float,
                             base: Optional[torch.Tensor] = None, out_scale: float = 1.0):
    """Per-chapter softmax, outputs mixed by ``weights``: o = base + out_scale * sum_s w_s softmax(q K_s^T) V_s.
    q [B,TQ,HQ,D]; k / v [B,TK,H,D] views whose rows may be strided (unit stride over (H, D));
    block_indices int32 [B,TQ,H,S]; weights [B,TQ,S].  Returns (o like q, lse_slots fp32 [B,TQ,HQ,S])."""
    L.require_cuda(q, k, v, block_indices, weights)
    b, tq, hq, d = q.shape
    _, tk, h, _ = k.shape
    q = _contig(q)
    ld = _kv_row_stride(k, v)
    s = L.SparseAttnShape(b, tq, tk, hq, h, d, block_indices.shape[-1], int(block_size), float(scale),
                          L.dtype_code(q.dtype))
    o = torch.empty_like(q)
    lse = torch.empty(b, tq, hq, block_indices.shape[-1], dtype=torch.float32, device=q.device)
    rc = L.lib().moc_sparse_attn_weighted_fwd(C.byref(s), L.ptr(q), L.ptr(k), L.ptr(v), ld,
                                              L.ptr(_contig(block_indices)), L.ptr(_contig(weights.float())),
                                              L.ptr(_contig(base)), float(out_scale), L.ptr(o), L.ptr(lse),
                                              L.ptr(L.status_word(q.device)), L.stream_ptr(q.device))
    L.check(rc, "moc_sparse_attn_weighted_fwd")
    return o, lse


@_instrument("sparse_attn_weighted_bwd", 1)
def sparse_attn_weighted_bwd(q, k, v, block_indices, weights, lse_slots, d_o, block_size: int, scale: float,
                             out_scale: float, d_k: torch.Tensor, d_v: torch.Tensor,
                             d_q_accum: Optional[torch.Tensor] = None):
    """Gradients of :func:`sparse_attn_weighted_fwd`.  ``d_k`` / ``d_v`` are zeroed fp32 accumulators shaped like
    k / v (row-strided views allowed); returns (d_q, d_w [B,TQ,S])."""
    b, tq, hq, d = q.shape
    _, tk, h, _ = k.shape
    q, d_o = _contig(q), _contig(d_o)
    ld, ldg = _kv_row_stride(k, v), _kv_row_stride(d_k, d_v)
    n_sel = block_indices.shape[-1]
    s = L.SparseAttnShape(b, tq, tk, hq, h, d, n_sel, int(block_size), float(scale), L.dtype_code(q.dtype))
    d_q = d_q_accum if d_q_accum is not None else torch.empty_like(q)
    d_w_heads = torch.empty(b, tq, hq, n_sel, dtype=torch.float32, device=q.device)
    rc = L.lib().moc_sparse_attn_weighted_bwd(C.byref(s), L.ptr(q), L.ptr(k), L.ptr(v), ld,
                                              L.ptr(_contig(block_indices)), L.ptr(_contig(weights.float())),
                                              float(out_scale), L.ptr(lse_slots), L.ptr(d_o), L.ptr(d_q),
                                              1 if d_q_accum is not None else 0, L.ptr(d_k), L.ptr(d_v), ldg,
                                              L.ptr(d_w_heads), L.ptr(L.status_word(q.device)),
                                              L.stream_ptr(q.device))
    L.check(rc, "moc_sparse_attn_weighted_bwd")
    return d_q, d_w_heads.sum(dim=2)


def token_mix_supported(q: torch.Tensor, k: torch.Tensor, block_size: int, index_heads: int) -> bool:
    """Whether the tensor-core chapter-stationary mixture takes this problem: bf16, head_dim 64, 64-row chapters,
    whole chapters, and one chapter list per token (``index_heads`` 1) or per KV head."""
    return (q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q.shape[-1] == 64 and int(block_size) == 64
            and k.shape[1] % 64 == 0 and index_heads in (1, k.shape[2]) and q.shape[2] % k.shape[2] == 0)


def _token_mix_shape(q, k, block_indices, scale):
    b, tq, hq, d = q.shape
    _, tk, h, _ = k.shape
    return L.SparseAttnShape(b, tq, tk, hq, h, d, block_indices.shape[-1], 64, float(scale), L.dtype_code(q.dtype))


@_instrument("token_mix_fwd", 7)
def token_mix_fwd(q, k, v, block_indices, weights, scale: float, base: Optional[torch.Tensor] = None,
                  out_scale: float = 1.0):
    """o = base + out_scale * sum_s w_s softmax(q K_s^T) V_s with every chapter's K / V tile stationary under the
    query rows that selected it.  q [B,TQ,HQ,64] bf16; k / v [B,TK,H,64] (row-strided views allowed);
    block_indices int32 [B,TQ,1 or H,S]; weights [B,TQ,S].
    Returns (o, lse_slots fp32 [B,TQ,HQ,S], index workspace for :func:`token_mix_bwd`)."""
    L.require_cuda(q, k, v, block_indices, weights)
    b, tq, hq, d = q.shape
    hi, n_sel = block_indices.shape[2], block_indices.shape[3]
    q = _contig(q)
    bi = _contig(block_indices)
    ld = _kv_row_stride(k, v)
    s = _token_mix_shape(q, k, bi, scale)
    ws = torch.empty(L.lib().moc_token_mix_workspace_bytes(C.byref(s), hi) // 4, dtype=torch.int32, device=q.device)
    status, stream = L.ptr(L.status_word(q.device)), L.stream_ptr(q.device)
    L.check(L.lib().moc_token_mix_index(C.byref(s), hi, L.ptr(bi), L.ptr(ws), status, stream), "moc_token_mix_index")
    partial = torch.empty(b * tq * n_sel * hq * d, dtype=q.dtype, device=q.device)
    o = torch.empty_like(q)
    lse = torch.empty(b, tq, hq, n_sel, dtype=torch.float32, device=q.device)
    rc = L.lib().moc_token_mix_fwd(C.byref(s), hi, L.ptr(q), L.ptr(k), L.ptr(v), ld, L.ptr(bi),
                                   L.ptr(_contig(weights.float())), L.ptr(_contig(base)), float(out_scale), L.ptr(ws),
                                   L.ptr(partial), L.ptr(o), L.ptr(lse), status, stream)
    L.check(rc, "moc_token_mix_fwd")
    return o, lse, ws


@_instrument("token_mix_bwd", 2)
def token_mix_bwd(q, k, v, block_indices, weights, lse_slots, d_o, scale: float, out_scale: float,
                  workspace: torch.Tensor, d_k: torch.Tensor, d_v: torch.Tensor,
                  d_q_base: Optional[torch.Tensor] = None):
    """Gradients of :func:`token_mix_fwd`.  ``d_k`` / ``d_v`` are bf16 tensors shaped like k / v (row-strided views
    allowed, uninitialised is fine) that the call writes in full -- zeros for chapters nobody selected; returns
    (d_q = d_q_base + routed part, d_w [B,TQ,S])."""
    b, tq, hq, d = q.shape
    hi, n_sel = block_indices.shape[2], block_indices.shape[3]
    q, d_o = _contig(q), _contig(d_o)
    bi = _contig(block_indices)
    ld, ldg = _kv_row_stride(k, v), _kv_row_stride(d_k, d_v)
    s = _token_mix_shape(q, k, bi, scale)
    partial = torch.empty(b * tq * n_sel * hq * d, dtype=q.dtype, device=q.device)
    d_q = torch.empty_like(q)
    d_w_heads = torch.zeros(b, tq, hq, n_sel, dtype=torch.float32, device=q.device)
    rc = L.lib().moc_token_mix_bwd(C.byref(s), hi, L.ptr(q), L.ptr(k), L.ptr(v), ld, L.ptr(bi),
                                   L.ptr(_contig(weights.float())), float(out_scale), L.ptr(lse_slots), L.ptr(d_o),
                                   L.ptr(workspace), L.ptr(partial), L.ptr(_contig(d_q_base)), L.ptr(d_q), L.ptr(d_k),
                                   L.ptr(d_v), ldg, L.ptr(d_w_heads), L.ptr(L.status_word(q.device)),
                                   L.stream_ptr(q.device))
    L.check(rc, "moc_token_mix_bwd")
    return d_q, d_w_heads.sum(dim=2)


def _kv_row_stride(k: torch.Tensor, v: torch.Tensor) -> int:
    """Elements between consecutive rows of a [B,TK,H,D] key / value view whose (H, D) part is dense."""
    b, tk, h, d = k.shape
    for t in (k, v):
        if t.stride(3) != 1 or t.stride(2) != d or (b > 1 and t.stride(0) != tk * t.stride(1)):
            raise ValueError("k / v must be dense over (heads, head_dim) with uniformly strided rows")
    if k.stride(1) != v.stride(1):
        raise ValueError("k and v must share a row stride")
    return int(k.stride(1))


@_instrument("row_dot", 1)
def row_dot(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """<a[..., :], b[..., :]> over the last axis, fp32, shaped like ``a.shape[:-1]``."""
    L.require_cuda(a, b)
    if a.dtype != b.dtype or a.shape != b.shape:
        raise ValueError("row_dot operands must share shape and dtype")
    a, b = _contig(a), _contig(b)
    dim = a.shape[-1]
    out = torch.empty(a.shape[:-1], dtype=torch.float32, device=a.device)
    rc = L.lib().moc_row_dot(L.ptr(a), L.ptr(b), L.dtype_code(a.dtype), L.ptr(out), a.numel() // dim, dim,
                             L.stream_ptr(a.device))
    L.check(rc, "moc_row_dot")
    return out


@_instrument("col_sum", 1)
def col_sum(x: torch.Tensor) -> torch.Tensor:
    """Sum over the rows of a contiguous fp32 [rows, cols] matrix."""
    L.require_cuda(x)
    x = _contig(x.float())
    out = torch.empty(x.shape[1], dtype=torch.float32, device=x.device)
    rc = L.lib().moc_col_sum(L.ptr(x), L.ptr(out), x.shape[0], x.shape[1], L.stream_ptr(x.device))
    L.check(rc, "moc_col_sum")
    return out


def cast(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """fp32 <-> bf16 conversion on the device (identity when the dtype already matches)."""
    if t.dtype == dtype:
        return t
    return _cast(t, dtype)


@_instrument("split_bf16", 1)
def split_bf16(t: torch.Tensor, terms: int = 3) -> torch.Tensor:
    """bf16 [terms, *t.shape] with t == sum of the terms to 2^-24 relative (terms = 3): successive roundings of the
    residual.  Sums of bf16 tensor-core products over the terms reproduce an fp32 product to fp32-grade accuracy."""
    L.require_cuda(t)
    if t.dtype != torch.float32:
        raise TypeError("split_bf16 takes an fp32 tensor")
    t = _contig(t)
    out = torch.empty((terms,) + tuple(t.shape), dtype=torch.bfloat16, device=t.device)
    L.check(L.lib().moc_split_bf16(L.ptr(t), L.ptr(out), t.numel(), int(terms), L.stream_ptr(t.device)),
            "moc_split_bf16")
    return out


@_instrument("sum_terms", 1)
def sum_terms(src: torch.Tensor, cols: int, terms: int, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dst[r, c] = bias[c] + sum_t src[r, t * ld + c] for fp32 src [rows, terms * ld] (smallest term, highest t,
    first)."""
    L.require_cuda(src)
    src = _contig(src)
    rows, ld = src.shape[0], src.shape[1] // terms
    out = torch.empty(rows, cols, dtype=torch.float32, device=src.device)
    L.check(L.lib().moc_sum_terms(L.ptr(src), L.ptr(_contig(bias)), L.ptr(out), rows, int(cols), ld, int(terms),
                                  L.stream_ptr(src.device)), "moc_sum_terms")
    return out


def gemm_split(a: torch.Tensor, b: torch.Tensor, *, a_kmajor: bool = True, b_kmajor: bool = True,
               out_dtype: torch.dtype = torch.float32, tag: Optional[str] = None) -> torch.Tensor:
    """fp32-grade C = op(A) op(B) on the tensor cores: an fp32 operand is split into three bf16 terms, a bf16 operand
    is taken as it is, and the partial products (smallest first) accumulate in one fp32 output.  Pairs of terms whose
    product lies below 2^-24 of the leading one are left out."""
    ta = split_bf16(a, 3) if a.dtype == torch.float32 else a.unsqueeze(0)
    tb = split_bf16(b, 3) if b.dtype == torch.float32 else b.unsqueeze(0)
    pairs = sorted(((i, j) for i in range(ta.shape[0]) for j in range(tb.shape[0]) if i + j <= 2),
                   key=lambda ij: -(ij[0] + ij[1]))
    out = None
    for i, j in pairs:
        out = gemm(ta[i], tb[j], a_kmajor=a_kmajor, b_kmajor=b_kmajor, out=out, out_dtype=torch.float32,
                   accumulate=out is not None, tag=tag)
    return out if out_dtype == torch.float32 else cast(out, out_dtype)


@_instrument("cast", 1)
def _cast(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    L.require_cuda(t)
    t = _contig(t)
    out = torch.empty(t.shape, dtype=dtype, device=t.device)
    lib = L.lib()
    if t.dtype == torch.float32 and dtype == torch.bfloat16:
        rc = lib.moc_cast_f32_to_bf16(L.ptr(t), L.ptr(out), t.numel(), L.stream_ptr(t.device))
    elif t.dtype == torch.bfloat16 and dtype == torch.float32:
        rc = lib.moc_cast_bf16_to_f32(L.ptr(t), L.ptr(out), t.numel(), L.stream_ptr(t.device))
    else:
        raise TypeError(f"unsupported cast {t.dtype} -> {dtype}")
    L.check(rc, "moc_cast")
    return out


@_instrument("transpose", 1)
def transpose(t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """[R, C] -> contiguous [C, R] in ``dtype`` (default: same dtype)."""
    L.require_cuda(t)
    t = _contig(t)
    dtype = dtype or t.dtype
    r, c = t.shape
    out = torch.empty(c, r, dtype=dtype, device=t.device)
    rc = L.lib().moc_transpose(L.ptr(t), L.dtype_code(t.dtype), L.ptr(out), L.dtype_code(dtype), r, c,
                               L.stream_ptr(t.device))
    L.check(rc, "moc_transpose")
    return out


@_instrument("pack_weights", 1)
def pack_weights(mats, outs, outs_t, ldt=None) -> None:
    """bf16 copies (``outs[i]``, may be None) and bf16 transposes (``outs_t[i]``, may be None; row stride
    ``ldt[i]``, 0 = dense) of up to four same-dtype row-major matrices, in one launch."""
    n = len(mats)
    L.require_cuda(*mats)
    mats = [_contig(m) for m in mats]
    arr = C.c_void_p * n
    iarr = C.c_int32 * n
    rc = L.lib().moc_pack_weights(
        n, arr(*[m.data_ptr() for m in mats]), L.dtype_code(mats[0].dtype),
        arr(*[(o.data_ptr() if o is not None else None) for o in outs]),
        arr(*[(o.data_ptr() if o is not None else None) for o in outs_t]),
        iarr(*[m.shape[0] for m in mats]), iarr(*[m.shape[1] for m in mats]),
        iarr(*(ldt if ldt is not None else [0] * n)), L.stream_ptr(mats[0].device))
    L.check(rc, "moc_pack_weights")


# --------------------------------------------------------------------------------------------
# normalisation in front of the memory cross-attention
# --------------------------------------------------------------------------------------------
NORM_KINDS = {"rms": 1, "rmsnorm": 1, "layernorm": 2, "layer": 2}


@_instrument("norm_fwd", 1)
def norm_fwd(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], kind: str, eps: float,
             out_dtype: torch.dtype):
    """Rows of ``x`` [rows, dim] (fp32) normalised; returns (y in ``out_dtype``, stats [rows, 2])."""
    L.require_cuda(x, weight)
    if x.dtype != torch.float32 or weight.dtype != torch.float32:
        raise TypeError("normalisation runs on fp32 rows and fp32 weights")
    x = _contig(x)
    rows, dim = x.shape
    y = torch.empty(rows, dim, dtype=out_dtype, device=x.device)
    stats = torch.empty(rows, 2, dtype=torch.float32, device=x.device)
    f32 = out_dtype == torch.float32
    rc = L.lib().moc_norm_fwd(L.ptr(x), L.ptr(_contig(weight)), L.ptr(_contig(bias)), NORM_KINDS[kind], float(eps),
                              rows, dim, L.ptr(y) if f32 else None, None if f32 else L.ptr(y), L.ptr(stats),
                              L.stream_ptr(x.device))
    L.check(rc, "moc_norm_fwd")
    return y, stats


@_instrument("norm_bwd", 2)
def norm_bwd(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, stats: torch.Tensor,
             residual_grad: Optional[torch.Tensor], kind: str, with_bias: bool):
    """Gradients of :func:`norm_fwd`: (dx [+ residual_grad], dweight, dbias or None)."""
    L.require_cuda(dy, x, weight, stats)
    dy, x = _contig(dy), _contig(x)
    rows, dim = x.shape
    dx = torch.empty_like(x)
    dweight = torch.empty(dim, dtype=torch.float32, device=x.device)
    dbias = torch.empty(dim, dtype=torch.float32, device=x.device) if with_bias else None
    ws = torch.empty(L.lib().moc_norm_bwd_workspace_bytes(rows, dim), dtype=torch.uint8, device=x.device)
    rc = L.lib().moc_norm_bwd(L.ptr(dy), L.ptr(x), L.ptr(_contig(weight)), L.ptr(stats),
                              L.ptr(_contig(residual_grad)), NORM_KINDS[kind], rows, dim, L.ptr(dx), L.ptr(dweight),
                              L.ptr(dbias), L.ptr(ws), L.stream_ptr(x.device))
    L.check(rc, "moc_norm_bwd")
    return dx, dweight, dbias


# --------------------------------------------------------------------------------------------
# decode-time attention over cached projected bank rows
# --------------------------------------------------------------------------------------------
@_instrument("decode_attn", 1)
def decode_attn(q: torch.Tensor, kv_bank: torch.Tensor, comb_idx: torch.Tensor, comb_w: torch.Tensor,
                num_heads: int, num_kv_heads: int, tokens_per_chapter: int, scale: float, want_lse: bool = False):
    """q [B, n_q, H*64] bf16, kv_bank [C*T, 2*HK*64] bf16, comb_idx / comb_w [B, S+k] -> out like q (and lse)."""
    L.require_cuda(q, kv_bank, comb_idx, comb_w)
    if q.dtype != torch.bfloat16 or kv_bank.dtype != torch.bfloat16:
        raise TypeError("decode attention runs on a bf16 query and a bf16 K/V cache")
    q, kv_bank = _contig(q), _contig(kv_bank)
    b, n_q, hd = q.shape
    d = hd // num_heads
    if kv_bank.shape[1] != 2 * num_kv_heads * d:
        raise ValueError("kv_bank must be [rows, 2 * num_kv_heads * head_dim]")
    comb_idx = _contig(comb_idx.to(torch.int32))
    comb_w = _contig(comb_w.float())
    if tuple(comb_idx.shape) != tuple(comb_w.shape) or comb_idx.shape[0] != b:
        raise ValueError("comb_idx and comb_w must both be [B, S+k]")
    s = L.DecodeShape(b, n_q, num_heads, num_kv_heads, d, comb_idx.shape[1], int(tokens_per_chapter), float(scale))
    out = torch.empty_like(q)
    lse = torch.empty(b, n_q, num_heads, dtype=torch.float32, device=q.device) if want_lse else None
    rc = L.lib().moc_decode_attn(C.byref(s), L.ptr(q), L.ptr(kv_bank), kv_bank.shape[0], L.ptr(comb_idx),
                                 L.ptr(comb_w), L.ptr(out), L.ptr(lse), L.ptr(L.status_word(q.device)),
                                 L.stream_ptr(q.device))
    L.check(rc, "moc_decode_attn")
    return (out, lse) if want_lse else out
