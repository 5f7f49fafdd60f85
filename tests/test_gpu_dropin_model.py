"""The reference's own ``MemoryTransformer`` (memory_transformer/model.py), unmodified, run twice: with its stock
classes and with this package's ``ChapterRouter`` / ``ChapteredMemoryBank`` / ``MemoryCrossAttention`` bound in
their place (``memory_b200.dropin``).  Same state dict, same token ids, forward + backward under the trainer's bf16
autocast (training/trainer.py:100-103).

The stock comparator is the copy installed under ``baseline/_ref`` by ``oracle/install_reference.py``; without it
these tests skip.  The stock router is called outside autocast in fp32 -- the benchmark configuration asks for an
fp32 router, and under autocast the reference's router ``nn.Linear`` would run in bf16, where chapter ranks are
not comparable.
"""
import copy

import pytest
import torch

from oracle import install_reference as ref_install
from util_cases import assert_close_all_forms, rel_err

needs_ref = pytest.mark.skipif(not ref_install.available(), reason="reference not installed under baseline/_ref")
BF16 = 2e-2


def small_config(mt, norm_rows=True):
    cfg = mt.config.Config()
    m, mem = cfg.model, cfg.memory
    m.hidden_dim, m.num_heads, m.num_kv_heads, m.num_layers = 128, 2, 2, 2
    m.intermediate_dim, m.vocab_size, m.max_seq_len = 256, 512, 128
    m.use_flash_attention = False
    mem.num_memory_tokens, mem.use_chapters, mem.num_chapters, mem.top_k_chapters = 17 * 64, True, 17, 4
    mem.memory_layer_placement, mem.memory_layer_indices = "custom", [1]
    mem.num_shared_chapters, mem.routed_scaling_factor = 1, 2.5
    mem.normalize_shared_routed_before_mixing = norm_rows
    mem.shared_routed_norm_type, mem.shared_routed_norm_eps = "rms", 1e-5
    mem.use_load_balance_loss, mem.use_z_loss = True, True
    mem.wo_init_zero = False
    mem.memory_gradient_checkpointing = False
    return cfg


def build_models(mt, cfg):
    from memory_b200.dropin import use_b200_memory_layer
    torch.manual_seed(0)
    stock = mt.model.MemoryTransformer(copy.deepcopy(cfg))
    with torch.no_grad():
        for r in stock.routers.values():          # a sharper router: chapter ranks well separated
            r.router.weight.normal_(0, 1.0)
    with use_b200_memory_layer(mt):
        swapped = mt.model.MemoryTransformer(copy.deepcopy(cfg))
    missing = swapped.load_state_dict(stock.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    return stock, swapped


@needs_ref
def test_swapped_model_has_the_reference_state_dict_and_our_classes():
    import memory_b200 as M
    mt = ref_install.import_reference()
    stock, swapped = build_models(mt, small_config(mt))
    assert list(stock.state_dict()) == list(swapped.state_dict())
    assert isinstance(swapped.routers["1"], M.ChapterRouter)
    assert isinstance(swapped.memory_banks["0"], M.ChapteredMemoryBank)
    assert isinstance(swapped.layers[1].memory_attn, M.MemoryCrossAttention)
    assert type(stock.routers["1"]).__module__.startswith("memory_transformer")
    # the names are put back when the context ends
    assert mt.model.ChapterRouter is type(stock.routers["1"])
    assert mt.memory_block.MemoryCrossAttention is type(stock.layers[1].memory_attn)


def _fp32_router(router):
    """Calls the stock router outside autocast, on fp32 states."""
    inner = router.forward

    def forward(hidden_states, *a, **k):
        with torch.autocast("cuda", enabled=False):
            return inner(hidden_states.float(), *a, **k)
    router.forward = forward


@needs_ref
@pytest.mark.gpu
@pytest.mark.parametrize("norm_rows", [True, False], ids=["rows_rms", "rows_raw"])
def test_reference_model_with_swapped_classes_matches_stock_under_autocast(norm_rows):
    from memory_b200 import _lib as L, ops
    dev = torch.device("cuda:0")
    mt = ref_install.import_reference()
    stock, swapped = build_models(mt, small_config(mt, norm_rows))
    stock, swapped = stock.to(dev).train(), swapped.to(dev).train()
    for r in stock.routers.values():
        _fp32_router(r)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 512, (2, 128), generator=g).to(dev)

    def run(model):
        model.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = model(ids, labels=ids)
        out["loss"].backward()
        return out

    seen = []
    hook = lambda name: seen.append(name)      # noqa: E731
    ops.LAUNCH_HOOK = hook
    try:
        so = run(swapped)
    finally:
        ops.LAUNCH_HOOK = None
    L.check_device_status(dev)
    ro = run(stock)
    # the bf16 tensor-core kernels ran, the fp32 FMA fallbacks did not
    assert "attn_fwd:bf16" in seen and "attn_bwd:bf16" in seen and "gemm:bf16" in seen, sorted(set(seen))
    assert not any(s.endswith(":f32") and s.split(":")[0] in ("attn_fwd", "attn_bwd", "gemm") for s in seen), sorted(set(seen))

    assert rel_err(so["logits"], ro["logits"]) < BF16
    assert abs(so["loss"].item() - ro["loss"].item()) < 2e-2 * abs(ro["loss"].item())
    for ls, lr in zip(so["router_losses"], ro["router_losses"]):
        assert set(ls) == set(lr)
        for k in lr:
            assert abs(ls[k].item() - lr[k].item()) <= 1e-4 * abs(lr[k].item()) + 1e-7, k
    sg = dict(swapped.named_parameters())
    checked = 0
    for name, p in stock.named_parameters():
        if not any(t in name for t in ("memory_banks", "routers", "memory_attn", "memory_layernorm")):
            continue
        assert p.grad is not None and sg[name].grad is not None, name
        assert_close_all_forms(sg[name].grad, p.grad, 3e-2, name)     # the reference harness's bf16 backward bar
        checked += 1
    assert checked >= 7
    bank_g = sg["memory_banks.0.base_bank.memory"].grad
    ref_g = dict(stock.named_parameters())["memory_banks.0.base_bank.memory"].grad
    assert torch.equal(bank_g == 0, ref_g == 0) or rel_err(bank_g, ref_g) < 3e-2
