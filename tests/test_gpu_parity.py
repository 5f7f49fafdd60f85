"""GPU parity: the CUDA path (through the C ABI) against the reference's outputs stored as golden
fixtures and against the CPU oracle.  Bars: chapter indices bit-exact, fp32 within 1e-4 relative
(5e-4 for gradients, the reference harness's own fp32 bar), bf16 within 2e-2 relative."""
import os

import numpy as np
import pytest
import torch

from util_cases import (BF16_CASES, CASES, assert_close_all_forms, attn_reference, load_gold, make_inputs, rel_err,
                        run_layer_gpu, shape_of)
from oracle import moc_oracle as O

pytestmark = pytest.mark.gpu
FP32_FWD, FP32_BWD, BF16 = 1e-4, 5e-4, 2e-2


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _status_ok(dev):
    from memory_b200 import _lib as L
    L.check_device_status(dev)


@pytest.mark.parametrize("name", list(CASES))
def test_layer_fp32_matches_reference_golden(name, dev):
    case = CASES[name]
    gold = load_gold(name)
    out, losses, info, P = run_layer_gpu(case, torch.float32, dev)
    _status_ok(dev)
    assert np.array_equal(info["indices"].cpu().numpy(), gold["indices"])
    assert np.array_equal(info["combined_indices"].cpu().numpy(), gold["combined_indices"])
    assert rel_err(info["weights"], torch.from_numpy(gold["weights"])) < 1e-5
    assert rel_err(info["combined_weights"], torch.from_numpy(gold["combined_weights"])) < 1e-5
    for k in ("load_balance", "auxiliary", "z_loss", "entropy"):
        np.testing.assert_allclose(losses[k].item(), float(gold["loss_" + k]), rtol=1e-5, atol=1e-8)
    assert rel_err(out, torch.from_numpy(gold["out"])) < FP32_FWD
    pairs = [("d_h_router", "h_router"), ("d_router_w", "router_w"), ("d_router_b", "router_b"),
             ("d_wq", "wq"), ("d_wk", "wk"), ("d_wv", "wv"), ("d_wo", "wo")]
    if case.separate_router_input:
        pairs.append(("d_h_attn", "h_attn"))
    if case.pre_norm is not None:
        pairs.append(("d_pre_norm_w", "pre_norm_w"))
        if case.pre_norm != "rms":
            pairs.append(("d_pre_norm_b", "pre_norm_b"))
    for g, p in pairs:
        assert rel_err(P[p].grad, torch.from_numpy(gold[g])) < FP32_BWD, g
    T = case.tokens_per_chapter
    rows = (gold["bank_touched_chapters"][:, None] * T + np.arange(T)[None]).reshape(-1)
    bg = P["bank"].grad.cpu()
    assert rel_err(bg[rows], torch.from_numpy(gold["d_bank_touched"])) < FP32_BWD
    mask = torch.ones(bg.shape[0], dtype=torch.bool)
    mask[rows] = False
    assert not bg[mask].any(), "bank gradient must be zero outside the touched chapters"


@pytest.mark.parametrize("fused", [False, True, "in_place"], ids=["two_pass", "fused_gather", "fused_in_place"])
@pytest.mark.parametrize("name", list(BF16_CASES))
def test_layer_bf16_matches_reference_golden(name, fused, dev):
    """bf16 tensor-core path, with and without row normalisation of the gathered chapters (the paper's
    setting is ``rms``), against the fp32 reference and against the reference under bf16 autocast; both with the
    gathered rows materialised and with the fused gather-and-project route."""
    case = CASES[name]
    gold = load_gold(name)
    seen = []
    from memory_b200 import ops
    ops.LAUNCH_HOOK = seen.append
    try:
        out, losses, info, P = run_layer_gpu(case, torch.bfloat16, dev, fused=bool(fused), in_place=fused == "in_place")
    finally:
        ops.LAUNCH_HOOK = None
    # affine-free LayerNorm rows cannot be a row scale: that case keeps the two-pass route even when asked
    assert ("gather_rows_fwd:f32" in seen) == (not fused or case.norm_type == "layernorm"), sorted(set(seen))
    if fused == "in_place" and case.norm_type != "layernorm":
        assert not any(s_.startswith("gather_rows_fwd") for s_ in seen), sorted(set(seen))
    _status_ok(dev)
    assert np.array_equal(info["indices"].cpu().numpy(), gold["indices"])
    for prefix in ("", "bf16_"):
        assert_close_all_forms(out, torch.from_numpy(gold[prefix + "out"]), BF16, prefix + "out")
        pairs = [("d_h_router", "h_router"), ("d_wq", "wq"), ("d_wk", "wk"), ("d_wv", "wv"), ("d_wo", "wo")]
        if case.pre_norm is not None:
            pairs.append(("d_pre_norm_w", "pre_norm_w"))
        for g, p in pairs:
            assert_close_all_forms(P[p].grad, torch.from_numpy(gold[prefix + g]), BF16, prefix + g)
    for g, p in (("d_router_w", "router_w"), ("d_router_b", "router_b")):
        assert_close_all_forms(P[p].grad, torch.from_numpy(gold[g]), BF16, g)
    T = case.tokens_per_chapter
    rows = (gold["bank_touched_chapters"][:, None] * T + np.arange(T)[None]).reshape(-1)
    bg = P["bank"].grad.cpu()
    for prefix in ("", "bf16_"):
        assert_close_all_forms(bg[rows], torch.from_numpy(gold[prefix + "d_bank_touched"]), BF16, prefix + "d_bank")
    mask = torch.ones(bg.shape[0], dtype=torch.bool)
    mask[rows] = False
    assert not bg[mask].any(), "bank gradient must be zero outside the touched chapters"


def test_router_matches_oracle_with_all_loss_gradients(dev):
    import memory_b200 as M
    for name in ("cfg0", "two_shared", "no_shared", "k_exceeds"):
        case = CASES[name]
        inp = {k: torch.from_numpy(v) for k, v in make_inputs(case).items()}
        hr = inp["h_router"].clone().requires_grad_(True)
        wr = inp["router_w"].clone().requires_grad_(True)
        br = inp["router_b"].clone().requires_grad_(True)
        idx, w, losses, _ = O.router_forward(hr, wr, br, case.top_k, case.num_shared_chapters)
        cidx, cw = O.prepend_shared_chapters(idx, w, case.num_chapters, case.num_shared_chapters,
                                             case.routed_scaling_factor)
        g_w, g_cw = torch.randn_like(w), torch.randn_like(cw)
        coef = {"load_balance": 0.3, "auxiliary": 700.0, "z_loss": 0.2, "entropy": 0.1}
        (sum(coef[k] * losses[k] for k in coef) + (w * g_w).sum() + (cw * g_cw).sum()).backward()
        h = inp["h_router"].to(dev).requires_grad_(True)
        W = inp["router_w"].to(dev).requires_grad_(True)
        b = inp["router_b"].to(dev).requires_grad_(True)
        gi, gw, gci, gcw, gl = M.route(h, W, b, case.top_k, case.num_shared_chapters,
                                       case.routed_scaling_factor, True)
        (sum(coef[k] * gl[k] for k in coef) + (gw * g_w.to(dev)).sum() + (gcw * g_cw.to(dev)).sum()).backward()
        _status_ok(dev)
        assert torch.equal(gi.cpu(), idx) and torch.equal(gci.cpu().long(), cidx)
        assert rel_err(gw, w) < 1e-5 and rel_err(gcw, cw) < 1e-5
        assert rel_err(W.grad, wr.grad) < 1e-4 and rel_err(b.grad, br.grad) < 1e-4
        assert rel_err(h.grad, hr.grad) < 1e-4


def test_router_tie_break_prefers_lower_chapter_id(dev):
    """Identical router rows give identical probabilities: the selection must be the lowest ids."""
    import memory_b200 as M
    d, C, k = 64, 40, 6
    h = torch.randn(2, 16, d, device=dev)
    row = torch.randn(d)
    W = torch.zeros(C, d)
    W[5:] = row            # chapters 5..39 tie exactly; 1..4 are lower (zero logit vs typical +/-)
    W[1:5] = row * 3.0     # make 1..4 distinct from the tied block
    idx, w, _, _, _ = M.route(h, W.to(dev), torch.zeros(C, device=dev), k, 1, 2.5, False)
    oi, ow, _, _ = O.router_forward(h.cpu(), W, torch.zeros(C), k, 1, False)
    assert torch.equal(idx.cpu(), oi)
    for b in range(2):
        tied = [c for c in idx[b].tolist() if c >= 5]
        # whatever part of the tied block is selected, it is its lowest ids, in ascending order
        assert tied == list(range(5, 5 + len(tied)))


def test_router_bf16_hidden_states_use_fp32_arithmetic(dev):
    import memory_b200 as M
    case = CASES["cfg0"]
    inp = {k: torch.from_numpy(v) for k, v in make_inputs(case).items()}
    hb = inp["h_router"].bfloat16()
    idx, w, _, _ = O.router_forward(hb.float(), inp["router_w"], inp["router_b"], case.top_k, 1, False)
    gi, gw, _, _, _ = M.route(hb.to(dev), inp["router_w"].to(dev), inp["router_b"].to(dev), case.top_k, 1, 2.5, False)
    assert torch.equal(gi.cpu(), idx) and rel_err(gw, w) < 1e-5


def test_gather_bad_chapter_index_sets_status_not_fault(dev):
    """An out-of-range chapter id is reported through the status word; the rows read as zero."""
    import memory_b200 as M
    from memory_b200 import _lib as L
    bank = torch.randn(8 * 16, 32, device=dev)
    idx = torch.tensor([[0, 3, 99]], dtype=torch.int32, device=dev)
    rows = M.gather_chapters(bank, idx, None, 16)
    with pytest.raises(RuntimeError, match="chapter index"):
        L.check_device_status(dev)
    assert not rows[0, 32:].any()
    L.check_device_status(dev)      # cleared by the failed check


def test_duplicate_chapters_across_batch_accumulate(dev):
    """Every batch item selecting the same chapters: the bank gradient is the sum over items."""
    import memory_b200 as M
    T, d, C = 16, 64, 12
    bank = torch.randn(C * T, d, device=dev, requires_grad=True)
    idx = torch.tensor([[0, 4, 7]] * 5, dtype=torch.int32, device=dev)
    w = torch.rand(5, 3, device=dev, requires_grad=True)
    rows = M.gather_chapters(bank, idx, w, T)
    g = torch.randn_like(rows)
    (rows * g).sum().backward()
    ref_bank = bank.detach().cpu().clone().requires_grad_(True)
    ref_w = w.detach().cpu().clone().requires_grad_(True)
    mem = O.scale_memory(O.gather_chapters(ref_bank, idx.cpu().long(), T), ref_w, T)
    (mem * g.cpu()).sum().backward()
    assert rel_err(rows, mem) < 1e-6
    assert rel_err(bank.grad, ref_bank.grad) < 1e-5 and rel_err(w.grad, ref_w.grad) < 1e-5


def test_sparse_bank_grad_sink_equals_dense(dev):
    import memory_b200 as M
    case = CASES["cfg0"]
    _, _, _, P_dense = run_layer_gpu(case, torch.float32, dev)
    inp = {k: torch.from_numpy(v).to(dev) for k, v in make_inputs(case).items()}
    bank = inp["bank"].clone().requires_grad_(True)
    bank.moc_sparse_grad = M.SparseBankGrad()
    out, losses, _ = M.memory_layer(inp["h_router"], inp["h_router"], bank, inp["router_w"], inp["router_b"],
                                    inp["wq"].requires_grad_(True), inp["wk"], inp["wv"], inp["wo"],
                                    num_heads=case.num_heads, num_kv_heads=case.num_kv_heads,
                                    tokens_per_chapter=case.tokens_per_chapter, top_k=case.top_k,
                                    compute_dtype=torch.float32)
    (out * inp["d_out"]).sum().backward()
    assert bank.grad is None
    dense = bank.moc_sparse_grad.to_dense(bank)
    # the dense run also carries the router-loss terms, which do not reach the bank
    assert rel_err(dense, P_dense["bank"].grad) < 1e-5


@pytest.mark.parametrize("shape", [(300, 200, 136), (128, 128, 64), (257, 130, 72)])
@pytest.mark.parametrize("a_k,b_k", [(True, True), (True, False), (False, True), (False, False)])
def test_projection_kernels_all_operand_layouts(shape, a_k, b_k, dev):
    from memory_b200 import ops
    m, n, k = shape
    a = torch.randn((m, k) if a_k else (k, m), device=dev)
    b = torch.randn((n, k) if b_k else (k, n), device=dev)
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-5)):
        if dt == torch.bfloat16 and (m % 8 or n % 8):
            continue   # 16-byte row alignment of the MN-major operands
        aa, bb = a.to(dt), b.to(dt)
        ref = (aa.float() if a_k else aa.float().t()) @ (bb.float().t() if b_k else bb.float())
        c = ops.gemm(aa, bb, a_kmajor=a_k, b_kmajor=b_k, out_dtype=torch.float32)
        assert rel_err(c, ref) < tol
    _status_ok(dev)


def test_projection_split_k_accumulate_and_row_scale(dev):
    from memory_b200 import ops
    a = torch.randn(4096, 256, device=dev).bfloat16()
    b = torch.randn(4096, 192, device=dev).bfloat16()
    ref = a.float().t() @ b.float()
    c = ops.gemm(a, b, a_kmajor=False, b_kmajor=False, out_dtype=torch.float32, split_k=8)
    assert rel_err(c, ref) < 1e-5
    c2 = ops.gemm(a, b, a_kmajor=False, b_kmajor=False, out=c.clone(), accumulate=True)
    assert rel_err(c2, 2 * ref) < 1e-5
    x = torch.randn(512, 128, device=dev).bfloat16()
    w = torch.randn(256, 128, device=dev).bfloat16()
    sc = torch.rand(8, device=dev) + 0.5
    y = ops.gemm(x, w, out_dtype=torch.float32, row_scale=sc, scale_block_rows=64)
    assert rel_err(y, (x.float() @ w.float().t()) * sc.repeat_interleave(64).unsqueeze(1)) < 1e-5
    _status_ok(dev)


@pytest.mark.parametrize("T", [64, 16])
def test_fused_gather_projection_reads_chapters_from_bank(T, dev):
    """K/V projection with the chapter rows fetched by TMA through the gather list."""
    from memory_b200 import ops
    C, d = 40, 256
    bank = torch.randn(C * T, d, device=dev).bfloat16()
    idx = torch.randperm(C, device=dev)[:8].int()
    sc = torch.rand(8, device=dev) + 0.5
    w = torch.randn(384, d, device=dev).bfloat16()
    c = ops.gemm(bank, w, out_dtype=torch.float32, row_scale=sc, scale_block_rows=T, a_row_blocks=idx,
                 a_block_rows=T, m=8 * T)
    ref = (bank.view(C, T, d)[idx.long()].float() * sc.view(-1, 1, 1)).view(-1, d) @ w.float().t()
    assert rel_err(c, ref) < 1e-5
    _status_ok(dev)


@pytest.mark.parametrize("cfg", [(1, 128, 64, 1, 1), (2, 256, 320, 2, 2), (2, 128, 80, 4, 2), (1, 192, 4160, 2, 2),
                                 (2, 192, 320, 2, 2), (3, 64, 96, 4, 2), (2, 192, 80, 2, 1)])
def test_attention_bf16_tensor_core_kernels(cfg, dev):
    """The last three shapes have 128-query tiles that straddle a batch boundary (L % 128 == 64 with B > 1): the
    tile then holds rows of the next sequence, which the row masks must keep out of every result."""
    from memory_b200 import ops
    B, L, N, H, HK = cfg
    D = 64
    q = torch.randn(B, L, H * D, device=dev).bfloat16().float().requires_grad_(True)
    kv = torch.randn(B, N, 2 * HK * D, device=dev).bfloat16().float().requires_grad_(True)
    ref, lref = attn_reference(q, kv, H, HK, D)
    g = torch.randn_like(ref).bfloat16().float()
    ref.backward(g)
    o, lse = ops.attn_fwd(q.detach().bfloat16(), kv.detach().bfloat16(), H, HK, D ** -0.5)
    dq, dkv = ops.attn_bwd(q.detach().bfloat16(), kv.detach().bfloat16(), o, lse, g.bfloat16(), H, HK, D ** -0.5)
    _status_ok(dev)
    assert rel_err(o, ref) < BF16 and rel_err(lse, lref) < 1e-4
    assert rel_err(dq, q.grad) < BF16 and rel_err(dkv, kv.grad) < BF16


@pytest.mark.parametrize("cfg", [(2, 100, 80, 4, 4, 64), (2, 64, 96, 4, 2, 32), (1, 130, 70, 2, 1, 16)])
def test_attention_fp32_kernels(cfg, dev):
    from memory_b200 import ops
    B, L, N, H, HK, D = cfg
    q = torch.randn(B, L, H * D, device=dev, requires_grad=True)
    kv = torch.randn(B, N, 2 * HK * D, device=dev, requires_grad=True)
    ref, lref = attn_reference(q, kv, H, HK, D)
    g = torch.randn_like(ref)
    ref.backward(g)
    o, lse = ops.attn_fwd(q.detach(), kv.detach(), H, HK, D ** -0.5)
    dq, dkv = ops.attn_bwd(q.detach(), kv.detach(), o, lse, g, H, HK, D ** -0.5)
    assert rel_err(o, ref) < FP32_FWD and rel_err(lse, lref) < FP32_FWD
    assert rel_err(dq, q.grad) < FP32_BWD and rel_err(dkv, kv.grad) < FP32_BWD


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_memory_cross_attn_entry_point(dtype, dev):
    """Per-token chapter-sparse attention against the oracle's restatement of its contract."""
    import memory_b200 as M
    B, TQ, TK, HQ, H, D, S, BS = 2, 40, 128, 4, 2, 64, 3, 16
    q = torch.randn(B, TQ, HQ, D, device=dev).to(dtype).requires_grad_(True)
    k = torch.randn(B, TK, H, D, device=dev).to(dtype).requires_grad_(True)
    v = torch.randn(B, TK, H, D, device=dev).to(dtype).requires_grad_(True)
    bi = torch.stack([torch.randperm(TK // BS)[:S] for _ in range(B * TQ * H)]).view(B, TQ, H, S).int().to(dev)
    o = M.memory_cross_attn(q, k, v, bi, BS)
    ref = O.sparse_chapter_attention(q.detach().cpu().float(), k.detach().cpu().float(), v.detach().cpu().float(),
                                     bi.cpu(), BS)
    tol = FP32_FWD if dtype == torch.float32 else BF16
    assert rel_err(o, ref) < tol
    # sequence-level selection through the same entry point equals the dense joint softmax
    bi_seq = bi[:, :1].expand(-1, TQ, -1, -1).contiguous()
    o2 = M.memory_cross_attn(q, k, v, bi_seq, BS)
    ref2 = O.sparse_chapter_attention(q.detach().cpu().float(), k.detach().cpu().float(),
                                      v.detach().cpu().float(), bi_seq.cpu(), BS)
    assert rel_err(o2, ref2) < tol
    g = torch.randn_like(o)
    o.backward(g)
    assert q.grad.shape == q.shape and k.grad.dtype == dtype
    # gradient values against autograd through the oracle's restatement
    qc, kc, vc = (t.detach().cpu().float().requires_grad_(True) for t in (q, k, v))
    refg = O.sparse_chapter_attention(qc, kc, vc, bi.cpu(), BS)
    refg.backward(g.cpu().float())
    btol = FP32_BWD if dtype == torch.float32 else 3e-2      # the reference harness's bf16 backward bar
    assert_close_all_forms(q.grad, qc.grad, btol, "dq")
    assert_close_all_forms(k.grad, kc.grad, btol, "dk")
    assert_close_all_forms(v.grad, vc.grad, btol, "dv")
    with pytest.raises(ValueError):
        M.memory_cross_attn(q.cpu(), k, v, bi, BS)
    with pytest.raises(ValueError):
        M.memory_cross_attn(q, k, v, bi, BS, dkv_strategy="z")


def test_module_api_matches_reference_contract(dev):
    """Drop-in classes: constructor errors, parameter names, return shapes."""
    import memory_b200 as M
    with pytest.raises(ValueError):
        M.ChapterRouter(64, 8, top_k=9)
    with pytest.raises(ValueError):
        M.ChapteredMemoryBank(M.StandardMemoryBank(100, 8), 7)
    with pytest.raises(ValueError):
        M.MemoryCrossAttention(100, 3)
    router = M.ChapterRouter(64, 9, top_k=3).to(dev)
    bank = M.ChapteredMemoryBank(M.StandardMemoryBank(9 * 16, 64), 9).to(dev)
    attn = M.MemoryCrossAttention(64, 1, wo_init_zero=False, use_flash_attention=False).to(dev)
    keys = set(dict(router.named_parameters())) | set(dict(bank.named_parameters())) | set(dict(attn.named_parameters()))
    assert {"router.weight", "router.bias", "base_bank.memory", "q_proj.weight", "k_proj.weight",
            "v_proj.weight", "o_proj.weight"} <= keys
    h = torch.randn(2, 32, 64, device=dev)
    idx, w, losses = router(h, return_losses=True, exclude_prefix_chapters=1)
    assert idx.dtype == torch.int64 and idx.shape == (2, 3) and set(losses) == {"load_balance", "auxiliary", "z_loss", "entropy"}
    with pytest.raises(ValueError):
        router(h, exclude_prefix_chapters=10)
    mem, flat = bank.get_chapters_batched(idx)
    assert mem.shape == (2, 48, 64) and flat.shape == (2, 48)
    assert torch.equal(mem, bank.get_memory()[flat])
    out, none = attn(h, mem * 0.5)
    assert out.shape == h.shape and none is None
    with pytest.raises(ValueError):
        attn(h, None)
    # the strict boundary equals the oracle's cross_attention
    ref = O.cross_attention(h.cpu(), (mem * 0.5).detach().cpu(), attn.q_proj.weight.detach().cpu(),
                            attn.k_proj.weight.detach().cpu(), attn.v_proj.weight.detach().cpu(),
                            attn.o_proj.weight.detach().cpu(), 1, 1)
    assert rel_err(out, ref) < FP32_FWD
    out2, _ = attn(h, mem[0] * 0.5)     # (N, d) memory shared by the batch
    ref2 = O.cross_attention(h.cpu(), (mem[0] * 0.5).detach().cpu(), attn.q_proj.weight.detach().cpu(),
                             attn.k_proj.weight.detach().cpu(), attn.v_proj.weight.detach().cpu(),
                             attn.o_proj.weight.detach().cpu(), 1, 1)
    assert rel_err(out2, ref2) < FP32_FWD


@pytest.mark.parametrize("kind", ["rms", "layernorm"])
@pytest.mark.parametrize("rows,dim", [(8192, 1024), (37, 1536), (5, 64)])
def test_block_norm_matches_oracle(kind, rows, dim, dev):
    """moc_norm_fwd / moc_norm_bwd against the restated RMSNorm / LayerNorm, residual gradient included;
    row counts that do not fill a block and a width above one register chunk."""
    from memory_b200 import ops
    g = torch.Generator().manual_seed(rows + dim)
    x = torch.randn(rows, dim, generator=g) * 1.7 + 0.3
    w = 1.0 + 0.1 * torch.randn(dim, generator=g)
    b = 0.1 * torch.randn(dim, generator=g) if kind == "layernorm" else None
    dy = torch.randn(rows, dim, generator=g)
    res = torch.randn(rows, dim, generator=g)
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    br = b.clone().requires_grad_(True) if b is not None else None
    y_ref = O.block_norm(xr, wr, br, kind, 1e-6)
    (y_ref * dy).sum().backward()
    y, stats = ops.norm_fwd(x.to(dev), w.to(dev), None if b is None else b.to(dev), kind, 1e-6, torch.float32)
    y16, _ = ops.norm_fwd(x.to(dev), w.to(dev), None if b is None else b.to(dev), kind, 1e-6, torch.bfloat16)
    dx, dw, db = ops.norm_bwd(dy.to(dev), x.to(dev), w.to(dev), stats, res.to(dev), kind, b is not None)
    assert rel_err(y, y_ref) < 1e-5
    assert rel_err(y16, y_ref) < 1e-2
    assert rel_err(dx, xr.grad + res) < 1e-4
    assert rel_err(dw, wr.grad) < 1e-4
    if b is not None:
        assert rel_err(db, br.grad) < 1e-4
    else:
        assert db is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_projection_epilogue_adds_residual(dtype, dev):
    """C = A B^T + residual, single pass and split over K, ragged edges."""
    from memory_b200 import ops
    g = torch.Generator().manual_seed(7)
    m, n, k = 300, 200, 512
    a = torch.randn(m, k, generator=g).to(dev)
    b = (torch.randn(n, k, generator=g) * 0.05).to(dev)
    r = torch.randn(m, n, generator=g).to(dev)
    ref = a.to(dtype).float() @ b.to(dtype).float().T + r
    tol = 1e-5 if dtype == torch.float32 else 1e-3
    out = ops.gemm(a.to(dtype), b.to(dtype), out_dtype=torch.float32, residual=r)
    assert rel_err(out, ref) < tol
    if dtype == torch.bfloat16:
        out = ops.gemm(a.to(dtype), b.to(dtype), out_dtype=torch.float32, residual=r, split_k=4)
        assert rel_err(out, ref) < tol
    _status_ok(dev)


def test_memory_sub_block_module_matches_oracle(dev):
    """The module form: state-dict names of the reference block's memory step, fp32 parity with the oracle."""
    import memory_b200 as M
    torch.manual_seed(3)
    d, H, HK, n = 128, 4, 2, 96
    for use_rms in (True, False):
        blk = M.MemorySubBlock(d, H, num_kv_heads=HK, use_rms_norm=use_rms, wo_init_zero=False).to(dev)
        with torch.no_grad():
            blk.memory_layernorm.weight.add_(0.1 * torch.randn(d, device=dev))
        keys = set(blk.state_dict())
        assert {"memory_layernorm.weight", "memory_attn.q_proj.weight", "memory_attn.k_proj.weight",
                "memory_attn.v_proj.weight", "memory_attn.o_proj.weight"} <= keys
        h = torch.randn(2, 40, d, device=dev, requires_grad=True)
        mem = (torch.randn(2, n, d, device=dev) * 0.5).requires_grad_(True)
        out = blk(h, mem)
        out.square().sum().backward()
        sd = {k: v.detach().cpu() for k, v in blk.state_dict().items()}
        hc, mc = h.detach().cpu().requires_grad_(True), mem.detach().cpu().requires_grad_(True)
        ref = O.memory_sub_block(hc, mc, sd["memory_layernorm.weight"], sd.get("memory_layernorm.bias"),
                                 "rms" if use_rms else "layernorm", blk.norm_eps, sd["memory_attn.q_proj.weight"],
                                 sd["memory_attn.k_proj.weight"], sd["memory_attn.v_proj.weight"],
                                 sd["memory_attn.o_proj.weight"], H, HK)
        ref.square().sum().backward()
        assert rel_err(out, ref) < FP32_FWD
        assert rel_err(h.grad, hc.grad) < FP32_BWD
        assert rel_err(mem.grad, mc.grad) < FP32_BWD
    _status_ok(dev)


def test_two_stream_layer_equals_chained_nodes(dev):
    """The single two-stream autograd node and the three chained nodes run the same kernels: outputs, router
    losses and every gradient must agree to rounding of the split-K atomics."""
    import memory_b200 as M
    case = CASES["block_rms"]
    inp = {k: torch.from_numpy(v).to(dev) for k, v in make_inputs(case).items()}
    results = []
    for two_stream in (True, False):
        names = ("h_router", "bank", "router_w", "router_b", "wq", "wk", "wv", "wo", "pre_norm_w")
        P = {k: inp[k].clone().requires_grad_(True) for k in names}
        out, losses, info = M.memory_layer(
            P["h_router"], P["h_router"], P["bank"], P["router_w"], P["router_b"], P["wq"], P["wk"], P["wv"], P["wo"],
            num_heads=case.num_heads, num_kv_heads=case.num_kv_heads, tokens_per_chapter=case.tokens_per_chapter,
            top_k=case.top_k, num_shared_chapters=case.num_shared_chapters,
            routed_scaling_factor=case.routed_scaling_factor, compute_dtype=torch.bfloat16, pre_norm="rms",
            pre_norm_weight=P["pre_norm_w"], pre_norm_eps=case.pre_norm_eps, add_residual=True, two_stream=two_stream)
        ((out.float() * inp["d_out"]).sum() + 0.01 * losses["load_balance"] + 0.001 * losses["z_loss"]).backward()
        torch.cuda.synchronize()
        results.append((out.detach(), {k: P[k].grad for k in names}, info["indices"]))
    (o1, g1, i1), (o2, g2, i2) = results
    assert torch.equal(i1, i2)
    assert rel_err(o1, o2) < 1e-6
    for k in g1:
        assert rel_err(g1[k], g2[k]) < 2e-3, k
    _status_ok(dev)


@pytest.mark.parametrize("name,norm", [("head64_t64", None), ("gqa", None), ("gqa", "rms"), ("two_shared", "layernorm")])
def test_decode_over_projected_bank_cache_matches_oracle(name, norm, dev):
    """Generation mode: cached K/V rows of the whole bank, rolling routing window, one query token per sequence,
    against the oracle's gather-and-project layer on the same states (bf16 bar)."""
    import memory_b200 as M
    case = CASES[name]
    if case.hidden_dim // case.num_heads != 64:
        pytest.skip("the cached decode path is the bf16 head_dim-64 path")
    inp = {k: torch.from_numpy(v) for k, v in make_inputs(case).items()}
    shape = shape_of(case)
    shape.norm_type, shape.norm_eps = norm, 1e-5
    g = torch.Generator().manual_seed(11)
    cache = M.ProjectedBankCache(inp["bank"].to(dev), inp["wk"].to(dev), inp["wv"].to(dev), case.tokens_per_chapter,
                                 case.num_shared_chapters, norm, 1e-5, chapters_per_pass=7)
    dec = M.MemoryDecoder(cache, inp["router_w"].to(dev), inp["router_b"].to(dev), inp["wq"].to(dev),
                          inp["wo"].to(dev), num_heads=case.num_heads, num_kv_heads=case.num_kv_heads,
                          top_k=case.top_k, num_shared_chapters=case.num_shared_chapters,
                          routed_scaling_factor=case.routed_scaling_factor)
    window = M.RoutingWindow(window_size=24, strategy="hybrid")
    prompt = inp["h_router"]                                     # [B, L, d]
    states = window.prefill(prompt)
    assert states.shape[1] == prompt.shape[1] and window.cache.shape[1] == 24
    for step in range(3):
        h_t = torch.randn(case.batch, 1, case.hidden_dim, generator=g)
        states = window.step(h_t) if step else states           # first token routes on the whole prompt
        out, info = dec.step(h_t.to(dev), states.to(dev))
        ref = O.memory_layer(shape, states, h_t, inp["bank"], inp["router_w"], inp["router_b"], inp["wq"], inp["wk"],
                             inp["wv"], inp["wo"], return_losses=False)
        assert torch.equal(info["indices"].cpu(), ref["indices"])
        assert rel_err(out, ref["out"]) < BF16
    _status_ok(dev)


def test_rms_norm_module_matches_oracle(dev):
    """The stand-alone RMSNorm module (forward and autograd) against the restated reference norm."""
    import memory_b200 as M
    torch.manual_seed(5)
    d = 192
    norm = M.RMSNorm(d, eps=1e-6).to(dev)
    with torch.no_grad():
        norm.weight.add_(0.2 * torch.randn(d, device=dev))
    x = torch.randn(3, 17, d, device=dev, requires_grad=True)
    g = torch.randn(3, 17, d, device=dev)
    y = norm(x)
    (y * g).sum().backward()
    xc = x.detach().cpu().requires_grad_(True)
    wc = norm.weight.detach().cpu().requires_grad_(True)
    yr = O.rms_norm(xc, wc, 1e-6)
    (yr * g.cpu()).sum().backward()
    assert rel_err(y, yr) < 1e-5
    assert rel_err(x.grad, xc.grad) < 1e-4
    assert rel_err(norm.weight.grad, wc.grad) < 1e-4


def test_router_sequence_rolling_pooling_matches_reference_golden(dev):
    """ChapterRouter(routing_strategy="sequence-rolling") against the reference's own module (fixture) with all
    loss gradients; also the "token" strategy of forward(), which is the sequence rule up to rounding."""
    import memory_b200 as M
    from make_golden import ROLLING
    case = CASES[ROLLING["case"]]
    gold = load_gold("rolling")
    inp = {k: torch.from_numpy(v) for k, v in make_inputs(case).items()}
    router = M.ChapterRouter(case.hidden_dim, case.num_chapters, top_k=case.top_k,
                             routing_strategy="sequence-rolling").to(dev)
    with torch.no_grad():
        router.router.weight.copy_(inp["router_w"]); router.router.bias.copy_(inp["router_b"])
    h = inp["h_router"].to(dev).requires_grad_(True)
    idx, w, losses = router(h, return_losses=True, exclude_prefix_chapters=case.num_shared_chapters,
                            rolling_window_size=ROLLING["window"])
    (sum(c * losses[k] for k, c in ROLLING["coef"].items()) + (w * torch.from_numpy(gold["g_w"]).to(dev)).sum()).backward()
    _status_ok(dev)
    assert np.array_equal(idx.cpu().numpy(), gold["indices"])
    assert rel_err(w, torch.from_numpy(gold["weights"])) < 1e-5
    for k in ("load_balance", "auxiliary", "z_loss", "entropy"):
        np.testing.assert_allclose(losses[k].item(), float(gold["loss_" + k]), rtol=1e-5, atol=1e-8)
    assert rel_err(h.grad, torch.from_numpy(gold["d_h"])) < FP32_BWD
    assert rel_err(router.router.weight.grad, torch.from_numpy(gold["d_router_w"])) < FP32_BWD
    assert rel_err(router.router.bias.grad, torch.from_numpy(gold["d_router_b"])) < FP32_BWD
    with pytest.raises(ValueError):
        router(h, rolling_window_size=0)
    router.routing_strategy = "token"
    ti, tw, _ = router(h.detach(), return_losses=False, exclude_prefix_chapters=case.num_shared_chapters)
    oi, ow, _, _ = O.router_forward(inp["h_router"], inp["router_w"], inp["router_b"], case.top_k,
                                    case.num_shared_chapters, False)
    assert torch.equal(ti.cpu(), oi) and rel_err(tw, ow) < 1e-5
    router.routing_strategy = "nonsense"
    with pytest.raises(ValueError):
        router(h)


def test_bounded_device_wait_gives_up_and_reports(dev):
    """A wait that cannot be satisfied (3 arrivals expected, 2 made) runs out after its poll limit: the kernel
    returns, the status word reads MOC_DEV_TIMEOUT, later waits of the CTA return at once, and the context
    stays usable.  With all arrivals made the same kernel reports success."""
    from memory_b200 import _lib as L, ops
    L.check_device_status(dev)
    ok, again, abort = ops.wait_probe(dev, expected=3, arrivals=3, poll_limit=1 << 16)
    assert (ok, again, abort) == (1, 1, 0)
    L.check_device_status(dev)
    ok, again, abort = ops.wait_probe(dev, expected=3, arrivals=2, poll_limit=2000)
    assert (ok, again, abort) == (0, 0, 1)
    with pytest.raises(RuntimeError, match="timed out"):
        L.check_device_status(dev)
    L.check_device_status(dev)                       # cleared by the failed check
    x = torch.randn(256, 64, device=dev).bfloat16()  # the context is intact: a tensor-core kernel still runs
    y = ops.gemm(x, x, out_dtype=torch.float32)
    assert rel_err(y, x.float() @ x.float().t()) < 1e-5
    _status_ok(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bank_grad_union_sum_over_rank_lists(dtype, dev):
    """Consumer of the gradient exchange: rows of several ranks summed over the union of their chapter lists,
    lists only partly filled, chapters shared between ranks, sums in ascending (rank, slot) order."""
    from memory_b200 import ops
    W, n, T, d, C = 3, 7, 4, 24, 20
    g = torch.Generator().manual_seed(9)
    counts = torch.tensor([7, 4, 5], dtype=torch.int32)
    ids = torch.stack([torch.sort(torch.randperm(C, generator=g)[:n]).values for _ in range(W)]).int()
    rows = [torch.randn(n * T, d, generator=g).to(dtype) for _ in range(W)]
    dense = torch.zeros(C * T, d)
    for r in range(W):
        for s_ in range(int(counts[r])):
            c = int(ids[r, s_])
            dense[c * T:(c + 1) * T] += rows[r][s_ * T:(s_ + 1) * T].float()
    dense *= 0.5
    out = ops.bank_grad_merge([x.to(dev) for x in rows], ids.to(dev), counts.to(dev), T, C, scale=0.5)
    _status_ok(dev)
    nu = int(out["num_unique"].item())
    uniq = out["uniq"][:nu].cpu().long()
    want_ids = torch.unique(torch.cat([ids[r, :counts[r]] for r in range(W)])).long()
    assert torch.equal(uniq, want_ids)
    got = out["rows"][:nu * T].cpu().view(nu, T, d)
    ref = dense.view(C, T, d)[uniq]
    assert rel_err(got, ref) < 1e-6
    # the same buffers can be reused
    out2 = ops.bank_grad_merge([x.to(dev) for x in rows], ids.to(dev), counts.to(dev), T, C, scale=0.5, out=out)
    assert out2["rows"].data_ptr() == out["rows"].data_ptr()
    # bf16 mean rows: the same sums, rounded once
    out3 = ops.bank_grad_merge([x.to(dev) for x in rows], ids.to(dev), counts.to(dev), T, C, scale=0.5,
                               out_dtype=torch.bfloat16)
    assert out3["rows"].dtype == torch.bfloat16 and torch.equal(out3["uniq"][:nu].cpu().long(), want_ids)
    assert torch.equal(out3["rows"][:nu * T].cpu(), out["rows"][:nu * T].cpu().bfloat16())


def test_bank_grad_union_sum_eight_ranks_at_the_paper_chapter_count(dev):
    """Eight ranks x 520 chapter slots (8 sequences x 65 selections, ascending lists partly filled) over 4,097
    chapters: the union (about 2,500 chapters) and the sums against a dense scatter-add."""
    from memory_b200 import ops
    W, n, T, d, C = 8, 520, 8, 64, 4097
    g = torch.Generator().manual_seed(19)
    counts = torch.tensor([483, 470, 520, 455, 501, 478, 466, 490], dtype=torch.int32)
    ids = torch.zeros(W, n, dtype=torch.int32)
    rows = []
    dense = torch.zeros(C, T, d, device=dev)
    for r in range(W):
        mine = torch.sort(torch.cat([torch.zeros(1, dtype=torch.long),
                                     1 + torch.randperm(C - 1, generator=g)[:int(counts[r]) - 1]])).values
        ids[r, :int(counts[r])] = mine.int()
        x = torch.randn(n * T, d, generator=g).bfloat16()
        rows.append(x.to(dev))
        dense.index_add_(0, mine.to(dev), x.to(dev).float().view(n, T, d)[:int(counts[r])])
    dense *= 0.125
    out = ops.bank_grad_merge(rows, ids.to(dev), counts.to(dev), T, C, scale=0.125)
    _status_ok(dev)
    nu = int(out["num_unique"].item())
    uniq = out["uniq"][:nu].long()
    want_ids = torch.unique(torch.cat([ids[r, :int(counts[r])] for r in range(W)])).long().to(dev)
    assert torch.equal(uniq, want_ids) and 2000 < nu < 3200
    got = out["rows"][:nu * T].view(nu, T, d)
    assert rel_err(got, dense[uniq]) < 1e-6


def test_peer_flag_barrier_arrives_and_gives_up(dev):
    """The flag barrier of the gradient exchange on one GPU, one launch at a time (no kernel waits for another):
    with the peers' words already at the epoch the kernel stores its own arrival into their arrays and returns; with
    a peer that never arrives the bounded wait runs out, the status word says so and the kernel returns."""
    from memory_b200 import _lib as L, ops
    L.check_device_status(dev)
    world, rank = 3, 1
    flags = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(world)]
    flags[rank][0] = 5          # ranks 0 and 2 have arrived at epoch 5 (they write word `their rank` of my array)
    flags[rank][2] = 6          # ... rank 2 is already one exchange ahead
    ops.peer_barrier(flags, rank, 5, poll_limit=1000)
    L.check_device_status(dev)
    assert int(flags[0][rank]) == 5 and int(flags[2][rank]) == 5 and int(flags[rank][rank]) == 0
    ops.peer_barrier(flags, rank, 6, poll_limit=200)          # rank 0 never reaches epoch 6
    with pytest.raises(RuntimeError, match="timed out"):
        L.check_device_status(dev)
    assert int(flags[0][rank]) == 6                           # my own arrival was still published
    L.check_device_status(dev)


def test_fused_layer_bank_gradient_as_bf16_rows_only(dev):
    """A sink that wants the bank gradient in bf16 rows only (a data-parallel step: the mean gradient is formed from
    the ranks' bf16 rows): the entry holds exactly the bf16 rounding of the fp32 rows a plain sink receives."""
    import memory_b200 as M
    case = CASES["head64_t64_rms"]
    plain, lean = M.SparseBankGrad(), M.SparseBankGrad(torch.bfloat16, wire_only=True)
    run_layer_gpu(case, torch.bfloat16, dev, fused=True, sink=plain)
    run_layer_gpu(case, torch.bfloat16, dev, fused=True, sink=lean)
    _status_ok(dev)
    (u0, n0, r0, t0), (u1, n1, r1, t1) = plain.entries[0], lean.entries[0]
    assert r0.dtype == torch.float32 and r1.dtype == torch.bfloat16 and lean.wire[0] is r1
    nu = int(n0.item())
    assert int(n1.item()) == nu and torch.equal(u0[:nu], u1[:nu]) and t0 == t1
    assert torch.equal(r1[:nu * t0], r0[:nu * t0].bfloat16())


def test_bank_adamw_from_compact_gradient_matches_torch_adamw(dev):
    """SparseBankAdamW against torch.optim.AdamW fed the dense form of the same gradients, three steps with
    different touched chapters: parameter, both moments, the bf16 working copy, and the gradient norm."""
    import memory_b200 as M
    T, d, C = 8, 64, 40
    g = torch.Generator().manual_seed(21)
    p0 = torch.randn(C * T, d, generator=g) * 0.02
    ref_p = torch.nn.Parameter(p0.clone())
    ref = torch.optim.AdamW([ref_p], lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    p = p0.clone().to(dev)
    shadow = torch.empty(C * T, d, dtype=torch.bfloat16, device=dev)
    opt = M.SparseBankAdamW(p, T, lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01, shadow=shadow)
    for step in range(3):
        n = 12
        touched = torch.sort(torch.randperm(C, generator=g)[:7 + step]).values.int()
        nu = touched.numel()
        uniq = torch.zeros(n, dtype=torch.int32)
        uniq[:nu] = touched
        rows = torch.randn(n * T, d, generator=g)
        dense = torch.zeros(C * T, d)
        for u in range(nu):
            c = int(touched[u])
            dense[c * T:(c + 1) * T] = rows[u * T:(u + 1) * T]
        scale = 0.5
        ref_p.grad = dense * scale
        ref.step()
        sg = M.SparseBankGrad()
        sg.add(uniq.to(dev), torch.tensor([nu], dtype=torch.int32, device=dev), rows.to(dev), T)
        sg.scale = scale
        assert rel_err(opt.grad_sqnorm(sg), (dense * scale).pow(2).sum().reshape(1)) < 1e-5
        opt.step(sg)
        _status_ok(dev)
        st = ref.state[ref_p]
        assert rel_err(p, ref_p.detach()) < 1e-6
        assert rel_err(opt.exp_avg, st["exp_avg"]) < 1e-6 and rel_err(opt.exp_avg_sq, st["exp_avg_sq"]) < 1e-6
        assert torch.equal(shadow, p.bfloat16())
    assert int(opt.state_dict()["step"]) == 3


def test_backward_entered_first_on_a_fresh_autograd_thread():
    """out.backward(g) with nothing else in the graph: the first device call an autograd worker thread makes is then
    the tensor-map encoder of a projection (a driver-API call), which must find a context on that thread.  Run in a
    child process: the worker threads of this one have long made runtime calls."""
    import subprocess
    import sys
    code = (
        "import torch, memory_b200 as M\n"
        "from memory_b200 import functional as F, _lib as L\n"
        "dev = torch.device('cuda:0')\n"
        "x = torch.randn(256, 128, device=dev).bfloat16().requires_grad_(True)\n"
        "w = (torch.randn(64, 128, device=dev) * 0.1).bfloat16().requires_grad_(True)\n"
        "y = F.linear(x, w)\n"
        "g = torch.randn(256, 64, device=dev).bfloat16()\n"
        "y.backward(g)\n"
        "torch.cuda.synchronize(); L.check_device_status(dev)\n"
        "ref = g.float() @ w.float()\n"
        "assert (x.grad.float() - ref).abs().max() <= 2e-2 * ref.abs().max()\n"
        "print('ok')\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]
