"""Parity at the benchmarked configuration: B 8, L 1024, d 768, 12 x 64 heads, 4,097 chapters of 64 rows,
top-64 routed plus one shared chapter, routed scale 2.5, bf16 activations, fp32 router.

The CPU oracle (fp32, eager) runs the same layer on the same tensors; the CUDA layer runs through the C ABI.
Two parameter sets are used:

* ``paper`` -- router weight N(0, 1): the top-65 probabilities of every sequence are separated by > 64 fp32
  ulps (recomputed in fp64 below), so "indices bit-exact" is a meaningful statement and is asserted.
* ``paper_flat`` -- router weight N(0, 0.02), the distribution the benchmark itself draws: the logits differ by
  ~1e-2 and several adjacent ranks sit within a few ulps of each other, where no two fp32 summation orders agree.
  There the selection is checked against fp64: it must be the exact top-k up to ties below 16 ulps.
"""
import numpy as np
import pytest
import torch

from cases import Case, make_inputs
from util_cases import assert_close_all_forms, close_stats, rel_err, run_layer_gpu, shape_of
from oracle import moc_oracle as O

pytestmark = pytest.mark.gpu
BF16 = 2e-2
ULP = float(np.finfo(np.float32).eps)

PAPER = Case("paper", 8, 1024, 768, 12, 12, 4097, 64, 64, seed=2000, router_scale=1.0)
PAPER_RMS = Case("paper_rms", 8, 1024, 768, 12, 12, 4097, 64, 64, seed=2000, router_scale=1.0, norm_type="rms")
PAPER_FLAT = Case("paper_flat", 8, 1024, 768, 12, 12, 4097, 64, 64, seed=2001, router_scale=0.02)


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


_cache = {}


def paper_inputs(case):
    """Seeded tensors of the case with the hidden states rounded to bf16 (what the layer is fed)."""
    key = (case.seed, case.router_scale)
    if key not in _cache:
        for k_ in [k_ for k_ in _cache if not (isinstance(k_, tuple) and k_[-1] == "ref")]:
            del _cache[k_]
        inp = {k: torch.from_numpy(v) for k, v in make_inputs(case).items()}
        inp["h_router"] = inp["h_router"].bfloat16().float()
        inp["h_attn"] = inp["h_router"]
        _cache[key] = inp
    return _cache[key]


def fp64_masked_probs(inp, num_shared):
    pooled = inp["h_router"].double().mean(1)
    z = pooled @ inp["router_w"].double().t() + inp["router_b"].double()
    p = torch.softmax(z, -1)
    p[:, :num_shared] = 0
    return p / p.sum(-1, keepdim=True)


def test_rank_gaps_of_the_paper_case_are_wide():
    inp = paper_inputs(PAPER)
    p = fp64_masked_probs(inp, 1)
    srt = torch.sort(p, -1, descending=True).values
    rel = ((srt[:, :64] - srt[:, 1:65]) / srt[:, :64]).min().item()
    assert rel > 64 * ULP, rel / ULP


def test_router_paper_shape_indices_bit_exact_and_gradients(dev):
    """4,097-way selection with k = 64: radix select, rank sort, weights, the four losses and every gradient."""
    import memory_b200 as M
    from memory_b200 import _lib as L
    inp = paper_inputs(PAPER)
    hr = inp["h_router"].clone().requires_grad_(True)
    wr = inp["router_w"].clone().requires_grad_(True)
    br = inp["router_b"].clone().requires_grad_(True)
    idx, w, losses, _ = O.router_forward(hr, wr, br, 64, 1)
    cidx, cw = O.prepend_shared_chapters(idx, w, 4097, 1, 2.5)
    g = torch.Generator().manual_seed(5)
    g_w, g_cw = torch.randn(w.shape, generator=g), torch.randn(cw.shape, generator=g)
    coef = {"load_balance": 0.3, "auxiliary": 700.0, "z_loss": 0.2, "entropy": 0.1}
    (sum(coef[k] * losses[k] for k in coef) + (w * g_w).sum() + (cw * g_cw).sum()).backward()

    h = inp["h_router"].bfloat16().to(dev).requires_grad_(True)      # bf16 activations, fp32 router
    W = inp["router_w"].to(dev).requires_grad_(True)
    b = inp["router_b"].to(dev).requires_grad_(True)
    gi, gw, gci, gcw, gl = M.route(h, W, b, 64, 1, 2.5, True)
    (sum(coef[k] * gl[k] for k in coef) + (gw * g_w.to(dev)).sum() + (gcw * g_cw.to(dev)).sum()).backward()
    L.check_device_status(dev)
    assert torch.equal(gi.cpu(), idx), "routed chapter ids must be bit-exact, in order"
    assert torch.equal(gci.cpu().long(), cidx)
    assert rel_err(gw, w) < 1e-5 and rel_err(gcw, cw) < 1e-5
    for k in coef:
        np.testing.assert_allclose(gl[k].item(), losses[k].item(), rtol=1e-5, atol=1e-8, err_msg=k)
    assert_close_all_forms(W.grad, wr.grad, 1e-4, "d_router_w")
    assert_close_all_forms(b.grad, br.grad, 1e-4, "d_router_b")
    # the hidden-state gradient leaves in bf16 (the activation dtype)
    assert rel_err(h.grad, hr.grad) < 1e-2


def test_router_flat_logits_selection_is_exact_up_to_ulp_ties(dev):
    """The benchmark's own parameter distribution: adjacent ranks closer than fp32 rounding exist, so the
    selection is held to fp64: descending order and the top-k property up to 16-ulp ties, and every
    difference from the fp32 oracle's ids sits on such a tie."""
    import memory_b200 as M
    inp = paper_inputs(PAPER_FLAT)
    p = fp64_masked_probs(inp, 1)
    gi, gw, _, _, _ = M.route(inp["h_router"].bfloat16().to(dev), inp["router_w"].to(dev), inp["router_b"].to(dev),
                              64, 1, 2.5, False)
    gi = gi.cpu()
    tau = 16 * ULP
    sel = torch.gather(p, 1, gi)
    assert (sel[:, :-1] >= sel[:, 1:] * (1 - tau)).all(), "selection must be in descending order"
    rest = p.clone()
    rest.scatter_(1, gi, 0.0)
    assert (rest.max(-1).values <= sel[:, -1] * (1 + tau)).all(), "an unselected chapter outranks a selected one"
    assert all(len(set(r.tolist())) == 64 for r in gi)
    oi, ow, _, _ = O.router_forward(inp["h_router"], inp["router_w"], inp["router_b"], 64, 1, False)
    diff = gi != oi
    if diff.any():
        a, b = torch.gather(p, 1, gi)[diff], torch.gather(p, 1, oi)[diff]
        assert ((a - b).abs() <= tau * b).all(), "a difference from the fp32 oracle that is not an ulp-level tie"
    w64 = sel / sel.sum(-1, keepdim=True)
    assert rel_err(gw, w64) < 1e-5


@pytest.mark.parametrize("fused", [False, True], ids=["two_pass", "fused_gather"])
@pytest.mark.parametrize("case", [PAPER, PAPER_RMS], ids=["norm_off", "norm_rms"])
def test_layer_paper_shape_bf16_against_fp32_oracle(case, fused, dev):
    """The whole bf16 layer, forward and backward, against the fp32 oracle: output, every parameter and input
    gradient, bank gradient on the touched rows and exactly zero elsewhere."""
    from memory_b200 import _lib as L
    inp = paper_inputs(case)
    tensors = {k: inp[k] for k in ("h_router", "h_attn", "bank", "router_w", "router_b", "wq", "wk", "wv", "wo")}
    key = (case.name, "ref")
    if key not in _cache:
        _cache[key] = O.memory_layer_fwd_bwd(shape_of(case), tensors, inp["d_out"], 0.01, 0.001)
    ref = _cache[key]
    gpu_in = dict(inp)
    gpu_in["h_router"] = inp["h_router"].bfloat16()
    gpu_in["h_attn"] = gpu_in["h_router"]
    out, losses, info, P = run_layer_gpu(case, torch.bfloat16, dev, inputs=gpu_in, fused=fused)
    L.check_device_status(dev)
    assert out.dtype == torch.bfloat16
    assert torch.equal(info["indices"].cpu(), ref["indices"])
    assert torch.equal(info["combined_indices"].cpu().long(), ref["combined_indices"])
    assert rel_err(info["combined_weights"], ref["combined_weights"]) < 1e-5
    for k in ("load_balance", "z_loss", "auxiliary", "entropy"):
        np.testing.assert_allclose(losses[k].item(), ref["losses"][k].item(), rtol=1e-5, atol=1e-8, err_msg=k)
    report = {"out": assert_close_all_forms(out, ref["out"], BF16, "out")}
    for g, p in (("d_h_router", "h_router"), ("d_wq", "wq"), ("d_wk", "wk"), ("d_wv", "wv"), ("d_wo", "wo"),
                 ("d_router_w", "router_w"), ("d_router_b", "router_b")):
        report[g] = assert_close_all_forms(P[p].grad, ref[g], BF16, g)
    T = case.tokens_per_chapter
    touched = torch.unique(ref["combined_indices"].reshape(-1))
    rows = (touched[:, None] * T + torch.arange(T)[None]).reshape(-1)
    bg = P["bank"].grad
    report["d_bank"] = assert_close_all_forms(bg[rows.to(dev)], ref["d_bank"][rows], BF16, "d_bank")
    mask = torch.ones(bg.shape[0], dtype=torch.bool, device=dev)
    mask[rows.to(dev)] = False
    assert not bg[mask].any(), "bank gradient must be zero outside the touched chapters"
    print({k: (round(v["max_rel"], 5), round(v["l2_rel"], 5)) for k, v in report.items()})


def test_chapter_segments_at_520_pairs_with_shared_duplicates(dev):
    """8 x 65 (batch, slot) pairs: the shared chapter is picked by every sequence and routed ones by several."""
    from memory_b200 import ops
    g = torch.Generator().manual_seed(3)
    idx = torch.stack([torch.cat([torch.zeros(1, dtype=torch.long), 1 + torch.randperm(300, generator=g)[:64]])
                       for _ in range(8)]).int()
    seg = ops.chapter_segments(idx.to(dev), 4097)
    n = int(seg["num_unique"].item())
    uniq = seg["uniq"][:n].cpu()
    ref_u, inv = torch.unique(idx.reshape(-1), return_inverse=True)
    assert torch.equal(uniq.long(), ref_u.long())
    assert torch.equal(seg["pair_to_uniq"].cpu().long(), inv)
    off = seg["seg_offsets"][:n + 1].cpu().long()
    pairs = seg["seg_pairs"].cpu().long()
    for u in range(n):
        mine = pairs[off[u]:off[u + 1]]
        assert torch.equal(torch.sort(mine).values, torch.nonzero(inv == u).reshape(-1))
        assert torch.equal(mine, torch.sort(mine).values), "pairs of a chapter are summed in a fixed (ascending) order"
