"""Token-level routing on the GPU: every token selects its own chapters (BASELINE configuration 3 semantics).

Checked against fixtures made by the reference's own modules (``ChapterRouter.route_token_level``,
``MemoryCrossAttention.forward(token_routing_state=...)``, tests/golden/make_golden.py) and against the CPU oracle's
restatement of the exact mixture rule; the kernel plugin is additionally loaded through the reference's own
file-path loader and called by the reference's own attention module.
"""
import os

import numpy as np
import pytest
import torch

from cases import TOKEN_CASES, make_inputs
from util_cases import assert_close_all_forms, load_gold, rel_err
from oracle import install_reference as ref_install
from oracle import moc_oracle as O

pytestmark = pytest.mark.gpu
FP32_FWD, FP32_BWD, BF16_FWD, BF16_BWD = 1e-4, 5e-4, 2e-2, 3e-2


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _split_bank(bank, case):
    """model.py:551-581: shared / routed rows, normalised over the whole bank when the case says so."""
    s, t = case.num_shared_chapters, case.tokens_per_chapter
    shared, routed = bank[:s * t].contiguous(), bank[s * t:].contiguous()
    if case.norm_type == "rms":
        shared = shared / shared.pow(2).mean(-1, keepdim=True).add(case.norm_eps).sqrt()
        routed = routed / routed.pow(2).mean(-1, keepdim=True).add(case.norm_eps).sqrt()
    elif case.norm_type == "layernorm":
        shared = torch.nn.functional.layer_norm(shared, (shared.shape[-1],), eps=case.norm_eps)
        routed = torch.nn.functional.layer_norm(routed, (routed.shape[-1],), eps=case.norm_eps)
    return shared.contiguous(), routed.contiguous()


def run_token_layer_gpu(case, compute_dtype, dev):
    import memory_b200 as M
    inp = {k: torch.from_numpy(v).to(dev) for k, v in make_inputs(case).items()}
    router = M.ChapterRouter(case.hidden_dim, case.num_chapters, top_k=case.top_k, routing_strategy="token").to(dev)
    attn = M.MemoryCrossAttention(case.hidden_dim, case.num_heads, num_kv_heads=case.num_kv_heads,
                                  wo_init_zero=False, compute_dtype=compute_dtype).to(dev)
    bank = inp["bank"].clone().requires_grad_(True)
    with torch.no_grad():
        router.router.weight.copy_(inp["router_w"]); router.router.bias.copy_(inp["router_b"])
        attn.q_proj.weight.copy_(inp["wq"]); attn.k_proj.weight.copy_(inp["wk"])
        attn.v_proj.weight.copy_(inp["wv"]); attn.o_proj.weight.copy_(inp["wo"])
    h = inp["h_router"].clone().requires_grad_(True)
    s = case.num_shared_chapters
    idx, w, losses = router.route_token_level(hidden_states=h, return_losses=True, exclude_prefix_chapters=s)
    shared, routed = _split_bank(bank, case)
    state = {"shared_memory": shared, "routed_memory": routed, "token_chapter_indices": (idx - s).to(torch.int32),
             "tokens_per_chapter": case.tokens_per_chapter, "routed_scale": float(case.routed_scaling_factor),
             "kernel_version": "v2", "chapter_weights": w}
    out, none = attn(h, None, token_routing_state=state, token_routing_kernel_version="v2")
    assert none is None
    loss = (out.float() * inp["d_out"]).sum() + 0.01 * losses["load_balance"] + 0.001 * losses["z_loss"]
    loss.backward()
    grads = {"d_h_router": h.grad, "d_router_w": router.router.weight.grad, "d_router_b": router.router.bias.grad,
             "d_wq": attn.q_proj.weight.grad, "d_wk": attn.k_proj.weight.grad, "d_wv": attn.v_proj.weight.grad,
             "d_wo": attn.o_proj.weight.grad, "d_bank": bank.grad}
    return idx, w, losses, out, grads


@pytest.mark.parametrize("name", list(TOKEN_CASES))
def test_token_layer_fp32_matches_reference_golden(name, dev):
    from memory_b200 import _lib as L
    case, gold = TOKEN_CASES[name], load_gold(name)
    idx, w, losses, out, grads = run_token_layer_gpu(case, torch.float32, dev)
    L.check_device_status(dev)
    assert idx.dtype == torch.int64 and np.array_equal(idx.cpu().numpy(), gold["indices"])
    assert rel_err(w, torch.from_numpy(gold["weights"])) < 1e-5
    for k in ("load_balance", "auxiliary", "z_loss", "entropy"):
        np.testing.assert_allclose(losses[k].item(), float(gold["loss_" + k]), rtol=1e-5, atol=1e-8, err_msg=k)
    assert_close_all_forms(out, torch.from_numpy(gold["out"]), FP32_FWD, "out")
    for k, g in grads.items():
        assert_close_all_forms(g, torch.from_numpy(gold[k]), FP32_BWD, k)


@pytest.mark.parametrize("name", ["token_gqa_rms", "token_multi_tile"])
def test_token_layer_bf16_matches_reference_golden(name, dev):
    """64-row chapters and head_dim 64: projections, the shared branch and the per-token mixture on the tensor-core
    kernels (``token_multi_tile``: chapters selected by more than 128 (token, slot) pairs)."""
    from memory_b200 import _lib as L
    case, gold = TOKEN_CASES[name], load_gold(name)
    idx, w, losses, out, grads = run_token_layer_gpu(case, torch.bfloat16, dev)
    L.check_device_status(dev)
    assert np.array_equal(idx.cpu().numpy(), gold["indices"])
    assert_close_all_forms(out, torch.from_numpy(gold["out"]), BF16_FWD, "out")
    for k, g in grads.items():
        assert_close_all_forms(g, torch.from_numpy(gold[k]), BF16_BWD, k)


def test_token_router_split_weight_projection_on_the_tensor_cores(dev):
    """bf16 activations, fp32 router, large enough for the split-weight tensor-core projection (4,097-style odd
    chapter count: padded operands).  Selection is held to fp64 (exact top-k up to 16-ulp ties), weights and losses
    to fp32 tolerances, the weight gradient to 1e-4 and the bf16 hidden-state gradient to 1e-2."""
    import memory_b200 as M
    from memory_b200 import _lib as L
    from memory_b200 import ops
    g = torch.Generator().manual_seed(77)
    B, Lq, d, C, k, S = 2, 512, 256, 1025, 8, 1
    h = torch.randn(B, Lq, d, generator=g).bfloat16()
    W = torch.randn(C, d, generator=g) * 0.05
    bias = torch.randn(C, generator=g) * 0.1
    hc, wc, bc = h.float().clone().requires_grad_(True), W.clone().requires_grad_(True), bias.clone().requires_grad_(True)
    idx, w, losses = O.route_token_level(hc, wc, bc, k, S, True)
    g_w = torch.randn(w.shape, generator=g)
    coef = {"load_balance": 0.3, "auxiliary": 50.0, "z_loss": 0.2, "entropy": 0.1}
    (sum(coef[n] * losses[n] for n in coef) + (w * g_w).sum()).backward()

    hg = h.to(dev).requires_grad_(True)
    wg, bg = W.to(dev).requires_grad_(True), bias.to(dev).requires_grad_(True)
    seen = []
    ops.LAUNCH_HOOK = seen.append
    try:
        gi, gw, gl = M.route_tokens(hg, wg, bg, k, S, True)
        (sum(coef[n] * gl[n] for n in coef) + (gw * g_w.to(dev)).sum()).backward()
    finally:
        ops.LAUNCH_HOOK = None
    L.check_device_status(dev)
    assert "split_bf16:f32" in seen and "gemm:bf16" in seen and "gemm:f32" not in seen, sorted(set(seen))
    # selection against fp64
    z = h.double().reshape(-1, d) @ W.double().t() + bias.double()
    p = torch.softmax(z, -1)
    p[:, :S] = 0
    gi2 = gi.reshape(-1, k).cpu()
    sel = torch.gather(p, 1, gi2)
    tau = 16 * float(np.finfo(np.float32).eps)
    assert (sel[:, :-1] >= sel[:, 1:] * (1 - tau)).all()
    rest = p.clone()
    rest.scatter_(1, gi2, 0.0)
    assert (rest.max(-1).values <= sel[:, -1] * (1 + tau)).all(), "an unselected chapter outranks a selected one"
    # rows whose top-(k+1) probabilities are more than 64 fp32 ulps apart: there "bit-exact" is meaningful, and the
    # ids must be the fp64 top-k in order
    srt, order = torch.sort(p, -1, descending=True)
    gap = ((srt[:, :k] - srt[:, 1:k + 1]) / srt[:, :k]).min(-1).values
    clear = gap > 64 * float(np.finfo(np.float32).eps)
    assert clear.float().mean() > 0.5, "the seed leaves too few gap-checked rows"
    assert torch.equal(gi2[clear], order[clear][:, :k]), "ids on gap-checked rows must be bit-exact"
    same = (gi.cpu() == idx).all(-1).reshape(-1)
    assert same.float().mean() > 0.999, "ids differ from the fp32 oracle beyond rare ulp-level ties"
    assert rel_err(gw.reshape(-1, k)[same.to(dev)], w.reshape(-1, k)[same]) < 1e-5
    for n in coef:
        np.testing.assert_allclose(gl[n].item(), losses[n].item(), rtol=2e-5, atol=1e-8, err_msg=n)
    assert_close_all_forms(wg.grad, wc.grad, 1e-4, "d_router_w")
    assert_close_all_forms(bg.grad, bc.grad, 1e-4, "d_router_b")
    assert rel_err(hg.grad, hc.grad) < 1e-2


def test_token_router_empty_selection_and_errors(dev):
    import memory_b200 as M
    router = M.ChapterRouter(32, 4, top_k=2).to(dev)
    h = torch.randn(2, 5, 32, device=dev)
    idx, w, losses = router.route_token_level(h, return_losses=False, exclude_prefix_chapters=4)
    assert idx.shape == (2, 5, 0) and w.shape == (2, 5, 0) and losses == {}
    with pytest.raises(ValueError):
        router.route_token_level(h[0])
    with pytest.raises(ValueError):
        router.route_token_level(h, exclude_prefix_chapters=5)
    attn = M.MemoryCrossAttention(32, 2, wo_init_zero=False).to(dev)
    with pytest.raises(ValueError):
        attn(h, None, token_routing_state={"routed_memory": None})
    with pytest.raises(ValueError):
        attn(h, None, token_routing_state={"token_chapter_indices": torch.zeros(2, 5, dtype=torch.int32, device=dev)})
    with pytest.raises(ValueError):
        attn(h, None, token_routing_state={"token_chapter_indices": torch.zeros(2, 4, 1, dtype=torch.int32, device=dev)})
    with pytest.raises(ValueError):
        attn(h, None, token_routing_state={}, return_attn_weights=True)


def _plugin_problem(dev, dtype, B=2, TQ=40, TK=128, HQ=4, H=2, D=64, S=3, BS=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, TQ, HQ, D, generator=g).to(dtype)
    k = torch.randn(B, TK, H, D, generator=g).to(dtype)
    v = torch.randn(B, TK, H, D, generator=g).to(dtype)
    bi = torch.stack([torch.randperm(TK // BS, generator=g)[:S] for _ in range(B * TQ * H)]).view(B, TQ, H, S).int()
    w = torch.rand(B, TQ, S, generator=g) + 0.1
    w = (w / w.sum(-1, keepdim=True)).to(dtype)
    do = torch.randn(B, TQ, HQ, D, generator=g).to(dtype)
    return q, k, v, bi, w, do, BS


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_plugin_weighted_entry_point_values_and_gradients(dtype, dev):
    """FSA_topk_sparse_attention_weighted_bthd: o, dq, dk, dv, dw against autograd through the oracle; chapter lists
    that differ between the KV heads of one token."""
    from memory_b200 import _lib as L
    from memory_b200.plugin import FSA_topk_sparse_attention_weighted_bthd as fn
    q, k, v, bi, w, do, BS = _plugin_problem(dev, dtype)
    qc, kc, vc, wc = (t.float().clone().requires_grad_(True) for t in (q, k, v, w))
    ref = O.weighted_chapter_attention(qc, kc, vc, bi, wc, BS)
    ref.backward(do.float())
    qg, kg, vg, wg = (t.to(dev).clone().requires_grad_(True) for t in (q, k, v, w))
    o = fn(q_bthd=qg, k_bthd=kg, v_bthd=vg, block_indices_bths=bi.to(dev), chapter_weights_bts=wg, block_size=BS,
           softmax_scale=None, assume_sorted_topk=False, disable_causal_mask=True)
    o.backward(do.to(dev))
    L.check_device_status(dev)
    ftol, btol = (FP32_FWD, FP32_BWD) if dtype == torch.float32 else (BF16_FWD, BF16_BWD)
    assert o.dtype == dtype and o.shape == q.shape
    assert_close_all_forms(o, ref, ftol, "o")
    assert_close_all_forms(qg.grad, qc.grad, btol, "dq")
    assert_close_all_forms(kg.grad, kc.grad, btol, "dk")
    assert_close_all_forms(vg.grad, vc.grad, btol, "dv")
    assert_close_all_forms(wg.grad, wc.grad, btol, "dw")
    with pytest.raises(ValueError):
        fn(qg, kg, vg, bi.to(dev), wg, BS, disable_causal_mask=False)
    with pytest.raises(ValueError):
        fn(qg, kg, vg, bi.to(dev), wg[:, :, :2], BS, disable_causal_mask=True)


TC_SHAPES = {
    "per_head_lists_multi_tile": dict(B=2, TQ=300, TK=512, HQ=4, H=2, S=3),
    "small_ragged": dict(B=1, TQ=70, TK=256, HQ=2, H=2, S=4),
    "gqa6_three_tiles_per_chapter": dict(B=1, TQ=520, TK=192, HQ=6, H=1, S=2),
    "two_sequences_one_kv_head": dict(B=2, TQ=100, TK=256, HQ=2, H=1, S=2),
}


@pytest.mark.parametrize("shape", list(TC_SHAPES))
def test_plugin_weighted_entry_point_tensor_core_path(shape, dev):
    """bf16, head_dim 64, 64-row chapters: the chapter-stationary tcgen05 kernels (inverted index, gathered query
    tiles, per-pair partial outputs summed in slot order).  Chapters hold fewer than, exactly and several times
    128 (token, slot) pairs."""
    from memory_b200 import _lib as L
    from memory_b200 import ops
    from memory_b200.plugin import FSA_topk_sparse_attention_weighted_bthd as fn
    q, k, v, bi, w, do, BS = _plugin_problem(dev, torch.bfloat16, BS=64, seed=11, **TC_SHAPES[shape])
    assert ops.token_mix_supported(q, k, BS, bi.shape[2])
    qc, kc, vc, wc = (t.float().clone().requires_grad_(True) for t in (q, k, v, w))
    ref = O.weighted_chapter_attention(qc, kc, vc, bi, wc, BS)
    ref.backward(do.float())
    qg, kg, vg, wg = (t.to(dev).clone().requires_grad_(True) for t in (q, k, v, w))
    seen = []
    ops.LAUNCH_HOOK = seen.append
    try:
        o = fn(q_bthd=qg, k_bthd=kg, v_bthd=vg, block_indices_bths=bi.to(dev), chapter_weights_bts=wg, block_size=BS,
               disable_causal_mask=True)
        o.backward(do.to(dev))
    finally:
        ops.LAUNCH_HOOK = None
    L.check_device_status(dev)
    assert any(n.startswith("token_mix_fwd") for n in seen) and any(n.startswith("token_mix_bwd") for n in seen)
    assert_close_all_forms(o, ref, BF16_FWD, "o")
    assert_close_all_forms(qg.grad, qc.grad, BF16_BWD, "dq")
    assert_close_all_forms(kg.grad, kc.grad, BF16_BWD, "dk")
    assert_close_all_forms(vg.grad, vc.grad, BF16_BWD, "dv")
    assert_close_all_forms(wg.grad, wc.grad, BF16_BWD, "dw")


def test_token_mix_shared_lists_base_scale_and_reproducibility(dev):
    """One chapter list per token for all heads (the module path): a base term, an output scale, a chapter that every
    token selects (several tiles), one nobody selects (its gradient rows stay zero), bit-identical repeats, and an
    out-of-range chapter id reported through the status word."""
    from memory_b200 import _lib as L
    from memory_b200 import ops
    g = torch.Generator().manual_seed(21)
    B, TQ, HQ, H, D, M_, S = 1, 333, 4, 2, 64, 6, 3
    q = torch.randn(B, TQ, HQ, D, generator=g).bfloat16()
    kv = torch.randn(B, M_ * 64, 2 * H * D, generator=g).bfloat16()            # K and V of a row share a projected row
    bi = torch.stack([torch.cat([torch.zeros(1, dtype=torch.long), 1 + torch.randperm(M_ - 2, generator=g)[:S - 1]])
                      for _ in range(B * TQ)]).view(B, TQ, 1, S).int()          # chapter 0 always, chapter 5 never
    w = torch.rand(B, TQ, S, generator=g) + 0.1
    base = torch.randn(B, TQ, HQ, D, generator=g).bfloat16()
    do = torch.randn(B, TQ, HQ, D, generator=g).bfloat16()
    rho = 2.5
    k4 = kv[..., :H * D].unflatten(-1, (H, D))
    v4 = kv[..., H * D:].unflatten(-1, (H, D))
    qc, kc, vc, wc = (t.float().clone().requires_grad_(True) for t in (q, k4, v4, w))
    ref = base.float() + rho * O.weighted_chapter_attention(qc, kc, vc, bi.expand(B, TQ, H, S), wc, 64)
    ref.backward(do.float())
    kvd = kv.to(dev)
    k4d, v4d = kvd[..., :H * D].unflatten(-1, (H, D)), kvd[..., H * D:].unflatten(-1, (H, D))
    scale = D ** -0.5

    def run():
        o, lse, ws = ops.token_mix_fwd(q.to(dev), k4d, v4d, bi.to(dev), w.to(dev), scale, base=base.to(dev),
                                       out_scale=rho)
        d_kv = torch.full_like(kvd, float("nan"))           # the call must write every row, zeros where nobody selected
        dk4, dv4 = d_kv[..., :H * D].unflatten(-1, (H, D)), d_kv[..., H * D:].unflatten(-1, (H, D))
        dq0 = torch.full_like(q, 0.5).to(dev)
        dq, dw = ops.token_mix_bwd(q.to(dev), k4d, v4d, bi.to(dev), w.to(dev), lse, do.to(dev), scale, rho, ws, dk4,
                                   dv4, d_q_base=dq0)
        return o, dq, dw, d_kv

    o, dq, dw, d_kv = run()
    L.check_device_status(dev)
    assert_close_all_forms(o, ref, BF16_FWD, "o")
    assert_close_all_forms(dq.float() - 0.5, qc.grad, BF16_BWD, "dq")
    assert_close_all_forms(dw, wc.grad, BF16_BWD, "dw")
    assert_close_all_forms(d_kv[..., :H * D].unflatten(-1, (H, D)), kc.grad, BF16_BWD, "dk")
    assert_close_all_forms(d_kv[..., H * D:].unflatten(-1, (H, D)), vc.grad, BF16_BWD, "dv")
    assert not d_kv[:, 5 * 64:].any(), "rows of a chapter nobody selected must stay zero"
    o2, dq2, dw2, d_kv2 = run()
    assert torch.equal(o, o2) and torch.equal(dq, dq2) and torch.equal(dw, dw2) and torch.equal(d_kv, d_kv2)
    bad = bi.clone()
    bad[0, 7, 0, 1] = M_
    ops.token_mix_fwd(q.to(dev), k4d, v4d, bad.to(dev), w.to(dev), scale)
    with pytest.raises(RuntimeError, match="out of range"):
        L.check_device_status(dev)


def test_plugin_joint_entry_point_and_backward_exports(dev):
    """FSA_topk_sparse_attention_bthd (one softmax over the selected chapters) and the stand-alone
    memory_cross_attn_backward / _preprocess_delta surfaces."""
    import memory_b200 as M
    from memory_b200.plugin import FSA_topk_sparse_attention_bthd as fn
    q, k, v, bi, _, do, BS = _plugin_problem(dev, torch.float32, seed=3)
    qc, kc, vc = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = O.sparse_chapter_attention(qc, kc, vc, bi, BS)
    ref.backward(do)
    qg, kg, vg = (t.to(dev).clone().requires_grad_(True) for t in (q, k, v))
    o = fn(qg, kg, vg, bi.to(dev), BS, disable_causal_mask=True)
    o.backward(do.to(dev))
    assert_close_all_forms(o, ref, FP32_FWD, "o")
    assert_close_all_forms(qg.grad, qc.grad, FP32_BWD, "dq")
    assert_close_all_forms(kg.grad, kc.grad, FP32_BWD, "dk")
    assert_close_all_forms(vg.grad, vc.grad, FP32_BWD, "dv")
    o2, lse = M.memory_cross_attn_forward(q.to(dev), k.to(dev), v.to(dev), bi.to(dev), BS)
    delta = M.memory_cross_attn_preprocess_delta(o2, do.to(dev))
    assert delta.shape == lse.shape and rel_err(delta, (ref.detach() * do).sum(-1)) < 1e-5
    dq, dk, dv = M.memory_cross_attn_backward(q.to(dev), k.to(dev), v.to(dev), o2, lse, do.to(dev), bi.to(dev), BS)
    assert_close_all_forms(dq, qc.grad, FP32_BWD, "dq")
    assert_close_all_forms(dk, kc.grad, FP32_BWD, "dk")
    assert_close_all_forms(dv, vc.grad, FP32_BWD, "dv")


@pytest.mark.skipif(not ref_install.available(), reason="reference not installed under baseline/_ref")
def test_reference_attention_module_runs_on_the_plugin_file(dev):
    """The reference's own MemoryCrossAttention, unmodified, with its file-path loader pointed at re-export files
    of this plugin (kernels-final/kernel_v4.py): on CUDA + bf16 + 64-row chapters it takes its fused weighted
    kernel path (memory_attention.py:598-617), which now runs these kernels.  Result against the oracle."""
    from memory_b200 import ops
    from memory_b200.plugin import install_plugin_files
    mt = ref_install.import_reference()
    trk = mt.token_routing_kernel
    kernels_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(trk.__file__))), "kernels-final")
    written = install_plugin_files(kernels_dir, versions=("v2", "v4"))
    assert len(written) == 2
    for cache in (trk._KERNEL_FN_CACHE, trk._WEIGHTED_KERNEL_FN_CACHE, trk._KERNEL_IMPORT_ERROR):
        cache.clear()
    assert trk.get_token_routing_weighted_kernel_fn("v4") is not None
    case = TOKEN_CASES["token_gqa_rms"]
    inp = {k: torch.from_numpy(v) for k, v in make_inputs(case).items()}
    from memory_transformer.memory_attention import MemoryCrossAttention
    attn = MemoryCrossAttention(case.hidden_dim, case.num_heads, num_kv_heads=case.num_kv_heads, wo_init_zero=False,
                                use_flash_attention=False)
    with torch.no_grad():
        attn.q_proj.weight.copy_(inp["wq"]); attn.k_proj.weight.copy_(inp["wk"])
        attn.v_proj.weight.copy_(inp["wv"]); attn.o_proj.weight.copy_(inp["wo"])
    attn = attn.to(dev).bfloat16().eval()
    s, t = case.num_shared_chapters, case.tokens_per_chapter
    idx, w = O.route_token_level(inp["h_router"], inp["router_w"], inp["router_b"], case.top_k, s)
    shared, routed = _split_bank(inp["bank"], case)
    state = {"shared_memory": shared.to(dev).bfloat16(), "routed_memory": routed.to(dev).bfloat16(),
             "token_chapter_indices": (idx - s).to(torch.int32).to(dev), "tokens_per_chapter": t,
             "routed_scale": float(case.routed_scaling_factor), "kernel_version": "v4",
             "chapter_weights": w.to(dev)}
    seen = []
    ops.LAUNCH_HOOK = seen.append
    try:
        with torch.no_grad():
            out, _ = attn(inp["h_router"].to(dev).bfloat16(), None, token_routing_state=state,
                          token_routing_kernel_version="v4")
    finally:
        ops.LAUNCH_HOOK = None
    assert "token_mix_fwd:bf16" in seen, sorted(set(seen))        # 64-row chapters, head_dim 64: tensor-core mixture
    ref = O.token_routed_attention(inp["h_router"], shared, routed, idx - s, w, t, case.routed_scaling_factor,
                                   inp["wq"], inp["wk"], inp["wv"], inp["wo"], case.num_heads, case.num_kv_heads)
    assert rel_err(out, ref) < 3e-2     # the reference's own bf16 projections and output rounding are in this path
