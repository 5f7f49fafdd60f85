"""The allocation-free attention backward (moc_attn_bwd_static) against the regular entry point.

Some hosts of this library may not allocate device memory at the moment they need the backward pass
(frozen memory pools in serving processes, callbacks where cudaMalloc is forbidden).  For them the
scratch the backward needs is a fixed array inside the library.  This file is collected last on
purpose: if it fails under ``-x`` every other test has already run.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(dev, dtype, B=2, L=128, N=192, H=2, HK=2, D=64, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, L, H * D, generator=g).to(dev).to(dtype)
    kv = torch.randn(B, N, 2 * HK * D, generator=g).to(dev).to(dtype)
    d_o = torch.randn(B, L, H * D, generator=g).to(dev).to(dtype)
    return q, kv, d_o, H, HK, D


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_backward_matches_regular_entry_point_twice(dtype):
    from memory_b200 import _lib as L, ops
    dev = torch.device("cuda:0")
    for call in range(2):                      # two calls in a row share the built-in scratch
        q, kv, d_o, H, HK, D = _problem(dev, dtype, seed=call)
        o, lse = ops.attn_fwd(q, kv, H, HK, D ** -0.5)
        dq_ref, dkv_ref = ops.attn_bwd(q, kv, o, lse, d_o, H, HK, D ** -0.5)
        out = (torch.empty_like(q), torch.empty_like(kv))
        torch.cuda.synchronize()
        # the caching allocator's running count of allocation requests only ever grows
        before = torch.cuda.memory_stats(dev)["allocation.all.allocated"]
        dq, dkv = ops.attn_bwd_static(q, kv, o, lse, d_o, H, HK, D ** -0.5, out=out)
        torch.cuda.synchronize()
        after = torch.cuda.memory_stats(dev)["allocation.all.allocated"]
        assert after == before, "the allocation-free path allocated through torch"
        L.check_device_status(dev)
        # same kernels, same order of operations: the bars of the parity tests are met with room to spare
        tol = 2e-2 if dtype == torch.bfloat16 else 5e-4
        for a, b in ((dq, dq_ref), (dkv, dkv_ref)):
            err = float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-30))
            assert err < tol, (call, err)
        assert torch.equal(dq, dq_ref) and torch.equal(dkv, dkv_ref)


def test_static_scratch_backward_rejects_oversized_problems():
    from memory_b200 import _lib as L
    lib = L.lib()
    header = open(__import__("os").path.join(__import__("os").path.dirname(__import__("os").path.dirname(
        __import__("os").path.abspath(__file__))), "include", "moc_b200.h")).read()
    assert "#define MOC_ATTN_BWD_STATIC_MAX_FLOATS 1048576" in header and L.ATTN_BWD_STATIC_MAX_FLOATS == 1048576
    dev = torch.device("cuda:0")
    dummy = torch.zeros(16, device=dev)
    s = L.AttnShape(64, 8192, 64, 16, 16, 64, 0.125, L.MOC_BF16)     # 6*B*H*L = 50M floats
    p = dummy.data_ptr()
    rc = lib.moc_attn_bwd_static(C.byref(s), p, p, p, p, p, p, p, L.status_word(dev).data_ptr(), None)
    assert rc == -1 and b"built-in scratch" in lib.moc_last_error()
