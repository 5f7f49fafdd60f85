"""The CPU oracle must reproduce the reference's own outputs (fixtures made by
tests/golden/make_golden.py) before anything is compared against the oracle."""
import os

import numpy as np
import pytest
import torch

from cases import CASES, TOKEN_CASES, make_inputs
from oracle import moc_oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def shape_of(case):
    return O.LayerShape(case.hidden_dim, case.num_heads, case.num_kv_heads, case.num_chapters,
                        case.tokens_per_chapter, case.top_k, case.num_shared_chapters,
                        case.routed_scaling_factor, case.norm_type, case.norm_eps, case.pre_norm,
                        case.pre_norm_eps)


def run_oracle(case, autocast_bf16=False):
    inp = {k: torch.from_numpy(v) for k, v in make_inputs(case).items()}
    if not case.separate_router_input:
        inp["h_attn"] = inp["h_router"]
    d_out = inp.pop("d_out")
    return O.memory_layer_fwd_bwd(shape_of(case), inp, d_out, autocast_bf16=autocast_bf16)


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_reference_fp32(name):
    case = CASES[name]
    gold = np.load(os.path.join(GOLDEN, name + ".npz"))
    res = run_oracle(case)
    assert np.array_equal(res["indices"].numpy(), gold["indices"])
    assert np.array_equal(res["combined_indices"].numpy(), gold["combined_indices"])
    tol = dict(rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(res["weights"].numpy(), gold["weights"], **tol)
    np.testing.assert_allclose(res["combined_weights"].numpy(), gold["combined_weights"], **tol)
    np.testing.assert_allclose(res["out"].numpy(), gold["out"], rtol=1e-4, atol=1e-6)
    for k in ("load_balance", "auxiliary", "z_loss", "entropy"):
        np.testing.assert_allclose(res["losses"][k].numpy(), gold["loss_" + k], rtol=1e-5, atol=1e-7)
    for k in ("d_h_router", "d_router_w", "d_router_b", "d_wq", "d_wk", "d_wv", "d_wo"):
        np.testing.assert_allclose(res[k].numpy(), gold[k], rtol=1e-4, atol=2e-6, err_msg=k)
    if case.separate_router_input:
        np.testing.assert_allclose(res["d_h_attn"].numpy(), gold["d_h_attn"], rtol=1e-4, atol=2e-6)
    for k in ("d_pre_norm_w", "d_pre_norm_b"):
        if k in gold.files:
            np.testing.assert_allclose(res[k].numpy(), gold[k], rtol=1e-4, atol=2e-6, err_msg=k)
    touched = gold["bank_touched_chapters"]
    T = case.tokens_per_chapter
    rows = (touched[:, None] * T + np.arange(T)[None, :]).reshape(-1)
    g = res["d_bank"].numpy()
    np.testing.assert_allclose(g[rows], gold["d_bank_touched"], rtol=1e-4, atol=2e-6)
    mask = np.ones(g.shape[0], bool); mask[rows] = False
    assert not g[mask].any()


def test_oracle_matches_reference_bf16_autocast():
    case = CASES["head64_t64"]
    gold = np.load(os.path.join(GOLDEN, "head64_t64.npz"))
    res = run_oracle(case, autocast_bf16=True)
    # same library, same ops, same rounding points: equal up to reduction order
    np.testing.assert_allclose(res["out"].float().numpy(), gold["bf16_out"], rtol=2e-2, atol=2e-3)
    np.testing.assert_allclose(res["d_wq"].numpy(), gold["bf16_d_wq"], rtol=2e-2, atol=2e-3)


def test_oracle_rolling_pool_router_matches_reference():
    """routing_strategy "sequence-rolling" (router.py:100-105, 159-195)."""
    from make_golden import ROLLING
    case = CASES[ROLLING["case"]]
    gold = np.load(os.path.join(GOLDEN, "rolling.npz"))
    inp = {k: torch.from_numpy(v) for k, v in make_inputs(case).items()}
    h = inp["h_router"].clone().requires_grad_(True)
    W = inp["router_w"].clone().requires_grad_(True)
    b = inp["router_b"].clone().requires_grad_(True)
    idx, w, losses, _ = O.router_forward(h, W, b, case.top_k, case.num_shared_chapters, True,
                                         routing_strategy="sequence-rolling", rolling_window_size=ROLLING["window"])
    (sum(c * losses[k] for k, c in ROLLING["coef"].items()) + (w * torch.from_numpy(gold["g_w"])).sum()).backward()
    assert np.array_equal(idx.numpy(), gold["indices"])
    np.testing.assert_allclose(w.detach().numpy(), gold["weights"], rtol=1e-5, atol=1e-7)
    for k in ("load_balance", "auxiliary", "z_loss", "entropy"):
        np.testing.assert_allclose(losses[k].item(), gold["loss_" + k], rtol=1e-5, atol=1e-8)
    np.testing.assert_allclose(h.grad.numpy(), gold["d_h"], rtol=1e-4, atol=1e-8)
    np.testing.assert_allclose(W.grad.numpy(), gold["d_router_w"], rtol=1e-4, atol=1e-8)


@pytest.mark.parametrize("name", list(TOKEN_CASES))
def test_oracle_token_level_layer_matches_reference(name):
    """route_token_level + token_routing_state attention (model.py:544-606, memory_attention.py:480-716)."""
    case = TOKEN_CASES[name]
    gold = np.load(os.path.join(GOLDEN, name + ".npz"))
    inp = {k: torch.from_numpy(v) for k, v in make_inputs(case).items()}
    res = O.token_memory_layer_fwd_bwd(shape_of(case), inp, inp["d_out"])
    assert np.array_equal(res["indices"].numpy(), gold["indices"])
    np.testing.assert_allclose(res["weights"].numpy(), gold["weights"], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(res["out"].numpy(), gold["out"], rtol=1e-4, atol=1e-6)
    for k in ("load_balance", "auxiliary", "z_loss", "entropy"):
        np.testing.assert_allclose(res["losses"][k].numpy(), gold["loss_" + k], rtol=1e-5, atol=1e-7)
    for k in ("d_h_router", "d_router_w", "d_router_b", "d_wq", "d_wk", "d_wv", "d_wo", "d_bank"):
        np.testing.assert_allclose(res[k].numpy(), gold[k], rtol=1e-4, atol=2e-6, err_msg=k)


def test_rank_gaps_of_token_cases_are_wide():
    for name, case in TOKEN_CASES.items():
        inp = make_inputs(case)
        z = inp["h_router"].astype(np.float64) @ inp["router_w"].astype(np.float64).T + inp["router_b"]
        p = np.exp(z - z.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
        p = p[..., case.num_shared_chapters:]
        srt = -np.sort(-p, axis=-1)
        k = case.top_k
        rel = ((srt[..., :k] - srt[..., 1:k + 1]) / srt[..., :k]).min()
        assert rel > 64 * np.finfo(np.float32).eps, (name, rel)


def test_topk_order_is_value_desc_then_index_asc():
    p = torch.tensor([[0.5, 1.0, 1.0, 0.2, 1.0, 1.0, 0.1]])
    v, i = O.topk_lower_index_first(p, 3)
    assert i.tolist() == [[1, 2, 4]]
    assert v.tolist() == [[1.0, 1.0, 1.0]]


def test_rank_gaps_of_golden_cases_are_wide():
    """Index parity is only meaningful when the top-(k+1) probabilities are
    separated by far more than fp32 rounding noise of a differently ordered
    GEMV; recompute the logits in fp64 and check the gaps."""
    for name, case in CASES.items():
        inp = make_inputs(case)
        pooled = inp["h_router"].astype(np.float64).mean(axis=1)
        z = pooled @ inp["router_w"].astype(np.float64).T + inp["router_b"]
        p = np.exp(z - z.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
        p[:, :case.num_shared_chapters] = 0
        srt = -np.sort(-p, axis=-1)
        k = min(case.top_k, case.num_chapters - case.num_shared_chapters)
        gaps = srt[:, :k] - srt[:, 1:k + 1]
        rel = gaps / srt[:, :k]
        assert rel.min() > 64 * np.finfo(np.float32).eps, (name, rel.min())


def test_flop_accounting_paper_shape():
    s = O.LayerShape(768, 12, 12, 4097, 64, 64)
    f = O.layer_flops(8, 1024, s)
    assert abs(f - 2.0259e11) / 2.0259e11 < 1e-3
