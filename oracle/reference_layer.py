"""One sequence-level memory layer driven through the reference's own modules.

TEST INFRASTRUCTURE ONLY (comparator and timed baseline; nothing in ``memory_b200`` imports it).  The
modules come from the unmodified copy installed under ``baseline/_ref`` (``oracle/install_reference.py``)
and are called exactly as the reference's model calls them for sequence-level routing
(memory_transformer/model.py:624-692, then memory_attention.py:402-478):

    ChapterRouter -> MemoryTransformer._prepend_shared_chapters -> ChapteredMemoryBank.get_chapters_batched
    -> optional MemoryTransformer._normalize_shared_routed_memory_vectors -> weight multiply
    -> MemoryCrossAttention(use_flash_attention=False)

with the loss ``(out * d_out).sum() + 0.01 load_balance + 0.001 z_loss`` (the form of the reference's kernel
harness, kernels-final/benchmark_kernels_final.py:721-728, plus the router terms of model.py:776-806).
"""
from __future__ import annotations

import time
from typing import Dict, Optional

import torch

from . import install_reference


class ReferenceLayer:
    def __init__(self, cfg: Dict, params: Dict[str, torch.Tensor], device, norm_type: Optional[str] = None,
                 norm_eps: float = 1e-5):
        mt = install_reference.import_reference()
        from memory_transformer.memory_attention import MemoryCrossAttention
        from memory_transformer.memory_bank import ChapteredMemoryBank, StandardMemoryBank
        from memory_transformer.model import MemoryTransformer
        from memory_transformer.router import ChapterRouter, compute_total_router_loss
        self.mt = mt
        self.cfg = cfg
        self.norm_type, self.norm_eps = norm_type, norm_eps
        self.MT = MemoryTransformer
        self.total_loss = compute_total_router_loss
        d = cfg["hidden_dim"]
        self.router = ChapterRouter(d, cfg["num_chapters"], top_k=cfg["top_k"], routing_strategy="sequence")
        base = StandardMemoryBank(cfg["num_chapters"] * cfg["tokens_per_chapter"], d)
        self.bank = ChapteredMemoryBank(base, cfg["num_chapters"])
        self.attn = MemoryCrossAttention(d, cfg["num_heads"], num_kv_heads=cfg["num_kv_heads"], wo_init_zero=False,
                                         use_flash_attention=False)
        with torch.no_grad():
            self.router.router.weight.copy_(params["router_w"]); self.router.router.bias.copy_(params["router_b"])
            base.memory.copy_(params["bank"])
            self.attn.q_proj.weight.copy_(params["wq"]); self.attn.k_proj.weight.copy_(params["wk"])
            self.attn.v_proj.weight.copy_(params["wv"]); self.attn.o_proj.weight.copy_(params["wo"])
        for m in (self.router, self.bank, self.attn):
            m.to(device).train()
        self.device = torch.device(device)

    def parameters(self):
        for m in (self.router, self.bank, self.attn):
            yield from m.parameters()

    def step(self, h: torch.Tensor, d_out: torch.Tensor, autocast_dtype: Optional[torch.dtype] = None):
        """Forward + backward.  The router runs in fp32 outside autocast (the benchmark configuration's
        "fp32 router"); with ``autocast_dtype`` the attention part runs under autocast as in the trainer."""
        cfg = self.cfg
        for p in self.parameters():
            p.grad = None
        h = h.detach().requires_grad_(True)
        idx, w, losses = self.router(h.float(), return_losses=True, exclude_prefix_chapters=cfg["num_shared_chapters"])
        cidx, cw = self.MT._prepend_shared_chapters(idx, w, num_chapters=cfg["num_chapters"],
                                                    num_shared_chapters=cfg["num_shared_chapters"],
                                                    routed_scaling_factor=cfg["routed_scaling_factor"])
        t = cfg["tokens_per_chapter"]

        def attention_part():
            memory, _ = self.bank.get_chapters_batched(cidx)
            if self.norm_type is not None:
                memory = self.MT._normalize_shared_routed_memory_vectors(
                    memory, num_shared_chapters=cfg["num_shared_chapters"], tokens_per_chapter=t,
                    norm_type=self.norm_type, eps=self.norm_eps)
            wexp = cw.unsqueeze(-1).repeat(1, 1, t).reshape(memory.shape[0], -1, 1)
            return self.attn(h, memory * wexp)[0]

        if autocast_dtype is not None:
            with torch.autocast(device_type=self.device.type, dtype=autocast_dtype):
                out = attention_part()
        else:
            out = attention_part()
        aux = self.total_loss(losses, load_balance_coef=0.01, auxiliary_coef=0.0, z_loss_coef=0.001)
        loss = (out.float() * d_out.float()).sum() + aux
        loss.backward()
        return {"out": out.detach(), "indices": idx, "weights": w.detach(), "losses": {k: v.detach() for k, v in losses.items()},
                "d_h": h.grad}


def time_steps(layer: ReferenceLayer, h, d_out, steps: int, warmup: int, autocast_dtype=None):
    """Seconds per step (mean over ``steps``), wall clock with a device synchronise on both sides."""
    cuda = layer.device.type == "cuda"
    times = []
    for i in range(warmup + steps):
        if cuda:
            torch.cuda.synchronize(layer.device)
        t0 = time.perf_counter()
        layer.step(h, d_out, autocast_dtype)
        if cuda:
            torch.cuda.synchronize(layer.device)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return sum(times) / len(times)
