"""CPU-side checks: the library loads and exports every declared symbol, host-side validation,
and that nothing in the package routes through the oracle or a CPU fallback."""
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_builds_and_exports_every_declared_symbol():
    from memory_b200 import _lib as L
    from memory_b200.build import build
    build()
    handle = L.lib()
    header = open(os.path.join(ROOT, "include", "moc_b200.h")).read()
    declared = set(re.findall(r"\b(moc_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    for name in L.EXPORTED:
        assert name in declared, f"{name} bound in Python but not declared in the header"
    assert handle.moc_abi_version() == 2


def test_host_side_argument_validation_without_a_gpu():
    import ctypes as C
    from memory_b200 import _lib as L
    handle = L.lib()
    s = L.RouterShape(2, 8, 16, 4, 9, 0, 1.0, 0)      # top_k > num_chapters
    assert handle.moc_router_workspace_bytes(C.byref(s)) > 0
    rc = handle.moc_router_fwd(C.byref(s), *([None] * 13), None, 0, None, None)
    assert rc == -1 and b"top_k" in handle.moc_last_error()
    g = L.GemmDesc(1, 1, 0, 8, 8, 1, 1, 8, 8, 8, 0, 1, 1, 0, 0)
    assert handle.moc_gemm(C.byref(g), None, None, None, None, None, None, None) == -1


def test_operators_refuse_cpu_tensors():
    import memory_b200 as M
    h = torch.randn(2, 8, 16)
    with pytest.raises(ValueError, match="CUDA"):
        M.route(h, torch.randn(4, 16), torch.zeros(4), 2, 0, 1.0, True)
    with pytest.raises(ValueError, match="CUDA"):
        M.gather_chapters(torch.randn(32, 16), torch.zeros(2, 2, dtype=torch.int32), None, 8)


def test_module_constructors_validate_like_the_reference():
    import memory_b200 as M
    with pytest.raises(ValueError, match="num_chapters must be > 0"):
        M.ChapterRouter(8, 0)
    with pytest.raises(ValueError, match="top_k must be > 0"):
        M.ChapterRouter(8, 4, top_k=0)
    with pytest.raises(ValueError, match="must be <= num_chapters"):
        M.ChapterRouter(8, 4, top_k=5)
    with pytest.raises(ValueError, match="divisible"):
        M.ChapteredMemoryBank(M.StandardMemoryBank(10, 4), 3)
    with pytest.raises(ValueError, match="divisible by num_heads"):
        M.MemoryCrossAttention(10, 3)
    with pytest.raises(ValueError, match="divisible by num_kv_heads"):
        M.MemoryCrossAttention(16, 4, num_kv_heads=3)
    r = M.ChapterRouter(8, 4, top_k=2)
    assert r.router.weight.shape == (4, 8) and float(r.router.bias.abs().sum()) == 0.0
    a = M.MemoryCrossAttention(16, 4)
    assert float(a.o_proj.weight.abs().sum()) == 0.0      # zero-initialised output projection
    assert M.compute_total_router_loss({}).item() == 0.0


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "memory_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f"{f} mentions the oracle"


def test_rolling_pool_coefficients_reproduce_the_window_means():
    """sum_s c[s] h[s] must equal the mean over t of the rolling-window means (router.py:159-195)."""
    from memory_b200.ops import rolling_pool_coefficients
    from oracle import moc_oracle as O
    for seq, window in ((37, 8), (16, None), (5, 100), (128, 1), (64, 64)):
        h = torch.randn(3, seq, 16, dtype=torch.float64)
        c = rolling_pool_coefficients(seq, window).double()
        ref = O.router_pool_rolling(h.float(), window).double()
        assert float((ref - (h * c.view(1, -1, 1)).sum(1)).abs().max()) < 1e-5
        assert abs(float(c.sum()) - 1.0) < 1e-6
    with pytest.raises(ValueError):
        rolling_pool_coefficients(8, 0)


def test_token_mixture_dispatch_and_split_k_rules():
    """Host-side rules that need no device: which problems the tensor-core token mixture takes, and the K-splits of
    the weight-gradient projections."""
    import torch
    from memory_b200 import functional as F, ops
    q = torch.empty(1, 8, 4, 64, dtype=torch.bfloat16)
    k = torch.empty(1, 256, 2, 64, dtype=torch.bfloat16)
    assert ops.token_mix_supported(q, k, 64, 1) and ops.token_mix_supported(q, k, 64, 2)
    assert not ops.token_mix_supported(q, k, 64, 4)                       # lists per query head are not taken
    assert not ops.token_mix_supported(q, k, 32, 1)                       # 64-row chapters only
    assert not ops.token_mix_supported(q.float(), k.float(), 64, 1)       # bf16 only
    assert not ops.token_mix_supported(q, k[:, :200], 64, 1)              # whole chapters only
    assert not ops.token_mix_supported(q[..., :32], k[..., :32], 64, 1)   # head_dim 64 only
    assert F._weight_grad_splits(torch.float32, 1 << 20, 768, 768) == 1
    assert F._weight_grad_splits(torch.bfloat16, 8192, 768, 768) == 8      # 18 tiles -> 148 // 18
    assert F._weight_grad_splits(torch.bfloat16, 262144, 1536, 768) == 4   # 36 tiles
    assert F._weight_grad_splits(torch.bfloat16, 256, 768, 768) == 1       # too few rows to split
