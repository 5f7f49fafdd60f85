"""Regenerate the parity fixtures from the reference implementation.

Usage (needs the reference checkout; run on CPU):

    python tests/golden/make_golden.py --reference /path/to/Memory

For every case in ``cases.py`` the reference's own objects are driven exactly as
its model does for sequence-level routing (model.py:624-692, then
memory_block.py:549-558): ``ChapterRouter`` -> ``_prepend_shared_chapters`` ->
``ChapteredMemoryBank.get_chapters_batched`` -> optional
``_normalize_shared_routed_memory_vectors`` -> weight multiply ->
``MemoryCrossAttention(use_flash_attention=False)``.  Cases with ``pre_norm`` wrap the attention as the
block does (memory_block.py:549-558): ``h + memory_attn(memory_layernorm(h), memory)`` with the reference's
``RMSNorm`` or ``torch.nn.LayerNorm``.  The loss is
``(out * d_out).sum() + 0.01 * load_balance + 0.001 * z_loss``.  Outputs and all
gradients are stored as ``<case>.npz`` next to this script.  The only import
shim is an empty ``omegaconf`` module (the reference imports it for YAML
loading, which this path never uses).
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from cases import BF16_CASES, CASES, TOKEN_CASES, make_inputs  # noqa: E402


def import_reference(path: str):
    if "omegaconf" not in sys.modules:
        stub = types.ModuleType("omegaconf")
        stub.OmegaConf = type("OmegaConf", (), {})
        stub.DictConfig = dict
        sys.modules["omegaconf"] = stub
    sys.path.insert(0, path)
    import memory_transformer  # noqa: F401
    from memory_transformer.memory_attention import MemoryCrossAttention
    from memory_transformer.memory_bank import ChapteredMemoryBank, StandardMemoryBank
    from memory_transformer.memory_block import RMSNorm
    from memory_transformer.model import MemoryTransformer
    from memory_transformer.router import ChapterRouter, compute_total_router_loss
    return dict(MemoryCrossAttention=MemoryCrossAttention, ChapteredMemoryBank=ChapteredMemoryBank,
                StandardMemoryBank=StandardMemoryBank, MemoryTransformer=MemoryTransformer,
                ChapterRouter=ChapterRouter, compute_total_router_loss=compute_total_router_loss,
                RMSNorm=RMSNorm)


def run_reference(ref, case, inputs, autocast_bf16=False):
    t = {k: torch.from_numpy(v.copy()) for k, v in inputs.items()}
    d = case.hidden_dim
    router = ref["ChapterRouter"](d, case.num_chapters, top_k=case.top_k, routing_strategy="sequence")
    base = ref["StandardMemoryBank"](case.num_chapters * case.tokens_per_chapter, d)
    bank = ref["ChapteredMemoryBank"](base, case.num_chapters)
    attn = ref["MemoryCrossAttention"](d, case.num_heads, num_kv_heads=case.num_kv_heads,
                                       wo_init_zero=False, use_flash_attention=False)
    with torch.no_grad():
        router.router.weight.copy_(t["router_w"]); router.router.bias.copy_(t["router_b"])
        base.memory.copy_(t["bank"])
        attn.q_proj.weight.copy_(t["wq"]); attn.k_proj.weight.copy_(t["wk"])
        attn.v_proj.weight.copy_(t["wv"]); attn.o_proj.weight.copy_(t["wo"])
    norm = None
    if case.pre_norm is not None:
        norm = (ref["RMSNorm"](d, eps=case.pre_norm_eps) if case.pre_norm == "rms"
                else torch.nn.LayerNorm(d, eps=case.pre_norm_eps))
        with torch.no_grad():
            norm.weight.copy_(t["pre_norm_w"])
            if case.pre_norm != "rms":
                norm.bias.copy_(t["pre_norm_b"])
    router.train(); attn.train()
    h_router = t["h_router"].clone().requires_grad_(True)
    h_attn = h_router if not case.separate_router_input else t["h_attn"].clone().requires_grad_(True)

    idx, w, losses = router(h_router, return_losses=True,
                            exclude_prefix_chapters=case.num_shared_chapters)
    MT = ref["MemoryTransformer"]
    cidx, cw = MT._prepend_shared_chapters(idx, w, num_chapters=case.num_chapters,
                                           num_shared_chapters=case.num_shared_chapters,
                                           routed_scaling_factor=case.routed_scaling_factor)
    memory, _ = bank.get_chapters_batched(cidx)
    if case.norm_type is not None:
        memory = MT._normalize_shared_routed_memory_vectors(
            memory, num_shared_chapters=case.num_shared_chapters,
            tokens_per_chapter=case.tokens_per_chapter, norm_type=case.norm_type, eps=case.norm_eps)
    wexp = cw.unsqueeze(-1).repeat(1, 1, case.tokens_per_chapter).reshape(memory.shape[0], -1, 1)
    memory = memory * wexp
    def memory_step():
        if norm is None:
            return attn(h_attn, memory)[0]
        residual = h_attn
        mem_output, _ = attn(norm(h_attn), memory)
        return residual + mem_output

    if autocast_bf16:
        with torch.autocast(device_type="cpu", dtype=torch.bfloat16):
            out = memory_step()
    else:
        out = memory_step()
    aux = ref["compute_total_router_loss"](losses, load_balance_coef=0.01, auxiliary_coef=0.0,
                                           z_loss_coef=0.001)
    loss = (out.float() * t["d_out"]).sum() + aux
    loss.backward()

    res = {
        "indices": idx.numpy(), "weights": w.detach().numpy(),
        "combined_indices": cidx.numpy(), "combined_weights": cw.detach().numpy(),
        "out": out.detach().float().numpy(), "loss": loss.detach().numpy(),
        "d_h_router": h_router.grad.numpy(),
        "d_router_w": router.router.weight.grad.numpy(), "d_router_b": router.router.bias.grad.numpy(),
        "d_wq": attn.q_proj.weight.grad.numpy(), "d_wk": attn.k_proj.weight.grad.numpy(),
        "d_wv": attn.v_proj.weight.grad.numpy(), "d_wo": attn.o_proj.weight.grad.numpy(),
    }
    for k, v in losses.items():
        res["loss_" + k] = v.detach().numpy()
    if norm is not None:
        res["d_pre_norm_w"] = norm.weight.grad.numpy()
        if case.pre_norm != "rms":
            res["d_pre_norm_b"] = norm.bias.grad.numpy()
    if case.separate_router_input:
        res["d_h_attn"] = h_attn.grad.numpy()
    # Bank gradient: dense in the reference; store the touched rows and check the rest is zero.
    g = base.memory.grad
    touched = torch.unique(cidx.reshape(-1))
    rows = (touched.unsqueeze(-1) * case.tokens_per_chapter
            + torch.arange(case.tokens_per_chapter)).reshape(-1)
    mask = torch.ones(g.shape[0], dtype=torch.bool); mask[rows] = False
    assert float(g[mask].abs().max() if mask.any() else 0.0) == 0.0
    res["bank_touched_chapters"] = touched.numpy()
    res["d_bank_touched"] = g[rows].numpy()
    return res


def run_reference_token(ref, case, inputs):
    """Token-level routing exactly as the reference's model wires it (model.py:544-606): ``route_token_level``,
    bank split into shared / routed rows (whole-bank normalisation when configured), the ``token_routing_state``
    payload, ``MemoryCrossAttention.forward(token_routing_state=...)`` (on CPU: its emulated per-chapter path,
    memory_attention.py:667-686, 856-898)."""
    t = {k: torch.from_numpy(v.copy()) for k, v in inputs.items()}
    d, T, S = case.hidden_dim, case.tokens_per_chapter, case.num_shared_chapters
    router = ref["ChapterRouter"](d, case.num_chapters, top_k=case.top_k, routing_strategy="token")
    base = ref["StandardMemoryBank"](case.num_chapters * T, d)
    bank = ref["ChapteredMemoryBank"](base, case.num_chapters)
    attn = ref["MemoryCrossAttention"](d, case.num_heads, num_kv_heads=case.num_kv_heads, wo_init_zero=False,
                                       use_flash_attention=False)
    with torch.no_grad():
        router.router.weight.copy_(t["router_w"]); router.router.bias.copy_(t["router_b"])
        base.memory.copy_(t["bank"])
        attn.q_proj.weight.copy_(t["wq"]); attn.k_proj.weight.copy_(t["wk"])
        attn.v_proj.weight.copy_(t["wv"]); attn.o_proj.weight.copy_(t["wo"])
    router.train(); attn.train()
    h = t["h_router"].clone().requires_grad_(True)
    idx, w, losses = router.route_token_level(hidden_states=h, return_losses=True, exclude_prefix_chapters=S)
    full = bank.get_memory()
    shared, routed = full[:S * T].contiguous(), full[S * T:].contiguous()
    if case.norm_type is not None:
        merged = ref["MemoryTransformer"]._normalize_shared_routed_memory_vectors(
            torch.cat([shared, routed], dim=0).unsqueeze(0), num_shared_chapters=S, tokens_per_chapter=T,
            norm_type=case.norm_type, eps=case.norm_eps).squeeze(0)
        shared, routed = merged[:S * T].contiguous(), merged[S * T:].contiguous()
    state = {"shared_memory": shared, "routed_memory": routed,
             "token_chapter_indices": (idx - S).to(torch.int32), "tokens_per_chapter": T,
             "routed_scale": float(case.routed_scaling_factor), "kernel_version": "v2", "chapter_weights": w}
    out, _ = attn(h, None, token_routing_state=state, token_routing_kernel_version="v2")
    aux = ref["compute_total_router_loss"](losses, load_balance_coef=0.01, auxiliary_coef=0.0, z_loss_coef=0.001)
    loss = (out.float() * t["d_out"]).sum() + aux
    loss.backward()
    res = {"indices": idx.numpy(), "weights": w.detach().numpy(), "out": out.detach().numpy(),
           "loss": loss.detach().numpy(), "d_h_router": h.grad.numpy(),
           "d_router_w": router.router.weight.grad.numpy(), "d_router_b": router.router.bias.grad.numpy(),
           "d_wq": attn.q_proj.weight.grad.numpy(), "d_wk": attn.k_proj.weight.grad.numpy(),
           "d_wv": attn.v_proj.weight.grad.numpy(), "d_wo": attn.o_proj.weight.grad.numpy(),
           "d_bank": base.memory.grad.numpy()}
    for k, v in losses.items():
        res["loss_" + k] = v.detach().numpy()
    return res


ROLLING = dict(case="rms_norm", window=8, coef={"load_balance": 0.3, "auxiliary": 700.0, "z_loss": 0.2, "entropy": 0.1})


def run_reference_rolling(ref):
    """``ChapterRouter`` with ``routing_strategy="sequence-rolling"`` (router.py:100-105, 159-195) on the inputs
    of one small case: selection, weights, losses and the gradients of a weighted sum of all of them."""
    case = CASES[ROLLING["case"]]
    t = {k: torch.from_numpy(v.copy()) for k, v in make_inputs(case).items()}
    router = ref["ChapterRouter"](case.hidden_dim, case.num_chapters, top_k=case.top_k,
                                  routing_strategy="sequence-rolling")
    with torch.no_grad():
        router.router.weight.copy_(t["router_w"]); router.router.bias.copy_(t["router_b"])
    router.train()
    h = t["h_router"].clone().requires_grad_(True)
    idx, w, losses = router(h, return_losses=True, exclude_prefix_chapters=case.num_shared_chapters,
                            rolling_window_size=ROLLING["window"])
    g_w = torch.from_numpy(np.random.Generator(np.random.PCG64(77)).standard_normal(tuple(w.shape), dtype=np.float32))
    (sum(c * losses[k] for k, c in ROLLING["coef"].items()) + (w * g_w).sum()).backward()
    res = {"indices": idx.numpy(), "weights": w.detach().numpy(), "g_w": g_w.numpy(), "d_h": h.grad.numpy(),
           "d_router_w": router.router.weight.grad.numpy(), "d_router_b": router.router.bias.grad.numpy()}
    for k, v in losses.items():
        res["loss_" + k] = v.detach().numpy()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    ref = import_reference(args.reference)
    torch.manual_seed(0)
    torch.set_num_threads(8)
    if not args.only or args.only == "rolling":
        np.savez_compressed(os.path.join(HERE, "rolling.npz"), **run_reference_rolling(ref))
        print("rolling", os.path.getsize(os.path.join(HERE, "rolling.npz")))
    for name, case in TOKEN_CASES.items():
        if args.only and name != args.only:
            continue
        res = run_reference_token(ref, case, make_inputs(case))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **res)
        print(name, "loss", float(res["loss"]), "size", os.path.getsize(os.path.join(HERE, name + ".npz")))
    for name, case in CASES.items():
        if args.only and name != args.only:
            continue
        inputs = make_inputs(case)
        res = run_reference(ref, case, inputs, autocast_bf16=False)
        if name in BF16_CASES:
            bf = run_reference(ref, case, inputs, autocast_bf16=True)
            for k in ("out", "d_h_router", "d_wq", "d_wk", "d_wv", "d_wo", "d_bank_touched", "d_pre_norm_w"):
                if k in bf:
                    res["bf16_" + k] = bf[k]
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **res)
        print(name, "indices", res["indices"].tolist(), "loss", float(res["loss"]),
              "size", os.path.getsize(os.path.join(HERE, name + ".npz")))


if __name__ == "__main__":
    main()
