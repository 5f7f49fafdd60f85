"""Stand-alone launcher of the hot kernels at the paper shape, for CUDA-event timing and for profilers.

    python -m memory_b200.kernel_bench --batch 8 --iters 5 [--only attn_fwd,attn_bwd_dq,...]

Prints one line per kernel: mean milliseconds per launch and executed TFLOP/s (or GB/s for the
bandwidth-bound ones).  Inputs are synthetic; no bank is allocated, so the footprint stays at a few
hundred MB and a profiler capture of a single launch ends quickly.
"""
from __future__ import annotations

import argparse

import torch

from . import _lib as L
from . import ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--chapters", type=int, default=65, help="selected chapters per sequence (shared included)")
    ap.add_argument("--tokens-per-chapter", type=int, default=64)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    b, l, h, dh = args.batch, args.seq, args.heads, 64
    d = h * dh
    n_sel = args.chapters * args.tokens_per_chapter
    only = set(x for x in args.only.split(",") if x)
    torch.manual_seed(0)
    q = torch.randn(b, l, d, device=dev).bfloat16()
    kv = (torch.randn(b, n_sel, 2 * d, device=dev) * 0.3).bfloat16()
    g = torch.randn(b, l, d, device=dev).bfloat16()
    mem = (torch.randn(b * n_sel, d, device=dev) * 0.02).bfloat16()
    wkv = (torch.randn(2 * d, d, device=dev) * 0.02).bfloat16()
    wq = (torch.randn(d, d, device=dev) * 0.02).bfloat16()
    o, lse = ops.attn_fwd(q, kv, h, h, dh ** -0.5)
    bufs = (torch.empty_like(q), torch.empty_like(kv), torch.empty(6, b, h, l, dtype=torch.float32, device=dev))
    ops.attn_bwd(q, kv, o, lse, g, h, h, dh ** -0.5, parts=1, buffers=bufs)
    unit = 2.0 * b * l * n_sel * d
    kv2 = kv.view(b * n_sel, 2 * d)
    cases = {
        "attn_fwd": (lambda: ops.attn_fwd(q, kv, h, h, dh ** -0.5), 2 * unit),
        "attn_bwd_dq": (lambda: ops.attn_bwd(q, kv, o, lse, g, h, h, dh ** -0.5, parts=2, buffers=bufs), 3 * unit),
        "attn_bwd_dkv": (lambda: ops.attn_bwd(q, kv, o, lse, g, h, h, dh ** -0.5, parts=4, buffers=bufs), 4 * unit),
        "kv_proj": (lambda: ops.gemm(mem, wkv), 2.0 * b * n_sel * d * 2 * d),
        "q_proj": (lambda: ops.gemm(q.view(b * l, d), wq), 2.0 * b * l * d * d),
        "d_mem": (lambda: ops.gemm(kv2, wkv, b_kmajor=False), 2.0 * b * n_sel * d * 2 * d),
        "d_wkv": (lambda: ops.gemm(kv2, mem, a_kmajor=False, b_kmajor=False, out_dtype=torch.float32, split_k=16),
                  2.0 * b * n_sel * d * 2 * d),
    }
    for name, (fn, flops) in cases.items():
        if only and name not in only:
            continue
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        evs = []
        for _ in range(args.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(c) for a, c in evs) / len(evs)
        print(f"{name:14s} {ms:8.4f} ms  {flops / ms / 1e9:8.1f} TFLOP/s executed")
    if "decode_attn" in only:
        # generation step at the benchmark's decode shape: 64 sequences, one token each, 65 chapters of the cached
        # 262,208-row K/V bank per sequence; bandwidth-bound, so the figure is bytes of cache rows per second
        bd, c_total, t = 64, 4097, args.tokens_per_chapter
        kv_bank = (torch.randn(c_total * t, 2 * d, device=dev) * 0.3).bfloat16()
        qd = torch.randn(bd, 1, d, device=dev).bfloat16()
        cidx = torch.stack([torch.cat([torch.zeros(1, dtype=torch.long), 1 + torch.randperm(c_total - 1)[:args.chapters - 1]])
                            for _ in range(bd)]).to(torch.int32).to(dev)
        cw = torch.rand(bd, args.chapters, device=dev) + 0.5
        fn = lambda: ops.decode_attn(qd, kv_bank, cidx, cw, h, h, t, dh ** -0.5)
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        evs = []
        for _ in range(args.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(c) for a, c in evs) / len(evs)
        gbytes = bd * args.chapters * t * 2 * d * 2 / 1e9
        print(f"{'decode_attn':14s} {ms:8.4f} ms  {gbytes / ms * 1e3:8.1f} GB/s of cached rows ({gbytes:.2f} GB per step)")
    L.check_device_status(dev)


if __name__ == "__main__":
    main()
