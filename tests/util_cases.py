"""Helpers shared by the GPU parity tests."""
import os

import numpy as np
import torch

from cases import BF16_CASES, CASES, make_inputs  # noqa: F401  (tests/golden is on sys.path via conftest)
from oracle import moc_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def shape_of(case):
    return O.LayerShape(case.hidden_dim, case.num_heads, case.num_kv_heads, case.num_chapters,
                        case.tokens_per_chapter, case.top_k, case.num_shared_chapters,
                        case.routed_scaling_factor, case.norm_type, case.norm_eps, case.pre_norm,
                        case.pre_norm_eps)


def load_gold(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a-b| / max |b| -- the tolerance form the parity bars are stated in."""
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    return float((a - b).abs().max() / (b.abs().max() + 1e-30))


def close_stats(a: torch.Tensor, b: torch.Tensor, tol: float) -> dict:
    """The three forms a tolerance is checked in.

    ``max_rel``   max |a-b| / max |b|            (one number per tensor)
    ``l2_rel``    ||a-b||_2 / ||b||_2            (catches errors spread over many small entries)
    ``bad``       entries failing |a-b| <= tol + tol |b|, the element-wise form of the reference's kernel
                  harness (kernels-final/benchmark_kernels_final.py:676-682), with the worst one's index
    """
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    diff = (a - b).abs()
    viol = diff > (tol + tol * b.abs())
    n_bad = int(viol.sum())
    worst = None
    if n_bad:
        flat = int((diff - tol * b.abs()).reshape(-1).argmax())
        worst = (flat, float(a.reshape(-1)[flat]), float(b.reshape(-1)[flat]))
    return {"max_rel": float(diff.max() / (b.abs().max() + 1e-30)),
            "l2_rel": float(diff.double().pow(2).sum().sqrt() / (b.double().pow(2).sum().sqrt() + 1e-30)),
            "bad": n_bad, "numel": b.numel(), "worst": worst}


def assert_close_all_forms(a, b, tol, what=""):
    s = close_stats(a, b, tol)
    assert s["max_rel"] < tol and s["l2_rel"] < tol and s["bad"] == 0, (what, s)
    return s


def run_layer_gpu(case, compute_dtype, dev, inputs=None, lb=0.01, z=0.001, fused=False, in_place=False, sink=None):
    """``fused``: the bf16 layer reads the chapters from a bf16 copy of the bank inside the K/V projection (no
    gathered rows), forward and backward."""
    import memory_b200 as M
    from memory_b200 import ops
    inp = inputs or {k: torch.from_numpy(v) for k, v in make_inputs(case).items()}
    inp = {k: v.to(dev) for k, v in inp.items()}
    names = ("h_router", "bank", "router_w", "router_b", "wq", "wk", "wv", "wo")
    P = {k: inp[k].clone().requires_grad_(True) for k in names}
    if sink is not None:
        P["bank"].moc_sparse_grad = sink
    P["h_attn"] = inp["h_attn"].clone().requires_grad_(True) if case.separate_router_input else P["h_router"]
    extra = {}
    if case.pre_norm is not None:
        P["pre_norm_w"] = inp["pre_norm_w"].clone().requires_grad_(True)
        if case.pre_norm != "rms":
            P["pre_norm_b"] = inp["pre_norm_b"].clone().requires_grad_(True)
        extra = dict(pre_norm=case.pre_norm, pre_norm_weight=P["pre_norm_w"], pre_norm_bias=P.get("pre_norm_b"),
                     pre_norm_eps=case.pre_norm_eps, add_residual=True)
    if fused:
        extra = dict(extra, bank_shadow=ops.cast(inp["bank"].contiguous(), torch.bfloat16),
                     bank_inv_rms=ops.row_inv_rms(inp["bank"].contiguous(), case.norm_eps),
                     wkv_grad_in_place=in_place)
    out, losses, info = M.memory_layer(
        P["h_router"], P["h_attn"], P["bank"], P["router_w"], P["router_b"], P["wq"], P["wk"], P["wv"], P["wo"],
        num_heads=case.num_heads, num_kv_heads=case.num_kv_heads, tokens_per_chapter=case.tokens_per_chapter,
        top_k=case.top_k, num_shared_chapters=case.num_shared_chapters,
        routed_scaling_factor=case.routed_scaling_factor, norm_type=case.norm_type, norm_eps=case.norm_eps,
        compute_dtype=compute_dtype, **extra)
    loss = (out.float() * inp["d_out"]).sum() + lb * losses["load_balance"] + z * losses["z_loss"]
    loss.backward()
    return out, losses, info, P


def attn_reference(q, kv, H, HK, D):
    """Dense torch attention over q [B,L,H*D], kv [B,N,2*HK*D] (K heads then V heads)."""
    B, L, _ = q.shape
    N = kv.shape[1]
    qq = q.view(B, L, H, D).transpose(1, 2)
    k = kv[..., :HK * D].view(B, N, HK, D).transpose(1, 2).repeat_interleave(H // HK, 1)
    v = kv[..., HK * D:].view(B, N, HK, D).transpose(1, 2).repeat_interleave(H // HK, 1)
    s = qq @ k.transpose(-1, -2) * D ** -0.5
    return (s.softmax(-1) @ v).transpose(1, 2).reshape(B, L, H * D), torch.logsumexp(s, -1)
