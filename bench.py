#!/usr/bin/env python
"""Benchmark of the Mixture-of-Chapters memory cross-attention layer (forward + backward).

    python bench.py --gpus N --steps K --warmup W          # CUDA path (this repository)
    python bench.py --impl reference --steps K --warmup W  # CPU restatement of the reference, host cores

One "step" is one forward+backward pass of one memory layer over one batch of synthetic hidden states
at the paper shape (B=8 per GPU, L=1024, d=768, 12x64 heads, 4,097 chapters of 64 rows, top-64 routed
plus one shared chapter, routed scale 2.5, bf16 activations, fp32 router), including router losses,
projection / router gradients and the gradient of the touched bank rows.  Rank 0 prints one JSON line.

Other modes: ``--kernels`` (the hot kernels alone), ``--token-level`` (the token-level routing variant).  Switches for
experiments, read from the environment and off by default: MOC_BENCH_SLOTS=n (sets of captured step buffers at N > 1),
MOC_BENCH_TWO_SLOTS=1 (two sets at N = 1), MOC_BENCH_NO_REDUCER=1 (N > 1 as independent replicas, no exchange),
MOC_BENCH_FLAT_PRIORITY=1 (compute graph on a default-priority stream), MOC_BENCH_DEBUG=1 (status word after each
set-up phase), MOC_DQ_ON_SIDE_STREAM=0 (dQ kernel back on the main stream).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PAPER = dict(batch=8, seq=1024, hidden_dim=768, num_heads=12, num_kv_heads=12, num_chapters=4097,
             tokens_per_chapter=64, top_k=64, num_shared_chapters=1, routed_scaling_factor=2.5)
METRIC = "memory-xattn fwd+bwd tokens/sec/GPU at L=1024,k=64; % of bf16 TC roofline"
N_INPUT_SETS = 4       # distinct hidden-state batches rotated between steps
# dram__bytes_read.sum + dram__bytes_write.sum per launch at this shape, from the ncu captures summarised under
# profiles/ (bytes); kernels without a capture report null
DOMINANT_KERNEL_DRAM_BYTES = {"attn_bwd_dkv": 193.2e6, "attn_bwd_dq": 136.2e6, "attn_fwd": 123.0e6}


def layer_flops(cfg) -> float:
    """Matmul FLOPs of one forward pass with the reference's accounting (scripts/estimate_flops.py:
    353-357, 385-417); fwd+bwd = 3x this (estimate_flops.py:805)."""
    b, l, d = cfg["batch"], cfg["seq"], cfg["hidden_dim"]
    dkv = cfg["num_kv_heads"] * (d // cfg["num_heads"])
    n_sel = (cfg["top_k"] + cfg["num_shared_chapters"]) * cfg["tokens_per_chapter"]
    return (2.0 * b * l * d * d * 2 + 2.0 * b * n_sel * d * dkv * 2 + 4.0 * b * l * n_sel * d
            + 2.0 * b * d * cfg["num_chapters"])


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tflops=float(p["bf16_tflops"]), tflops_sustained=float(p["bf16_tflops_sustained"]),
                    hbm_gbs=float(p["hbm_gbs"]), source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = os.path.join("/tmp", f"moc_clocks_{os.getpid()}.csv")

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "20"], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.remove(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_params(cfg, device, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    d = cfg["hidden_dim"]
    dkv = cfg["num_kv_heads"] * (d // cfg["num_heads"])
    rows = cfg["num_chapters"] * cfg["tokens_per_chapter"]

    def normal(shape, std):
        return (torch.randn(shape, generator=g) * std).to(device)

    return dict(bank=normal((rows, d), 0.02), router_w=normal((cfg["num_chapters"], d), 0.02),
                router_b=torch.zeros(cfg["num_chapters"], device=device), wq=normal((d, d), 0.02),
                wk=normal((dkv, d), 0.02), wv=normal((dkv, d), 0.02), wo=normal((d, d), 0.02))


def make_hidden(cfg, n_sets, seed, dtype):
    g = torch.Generator(device="cpu").manual_seed(seed)
    shape = (cfg["batch"], cfg["seq"], cfg["hidden_dim"])
    return [torch.randn(shape, generator=g).to(dtype) for _ in range(n_sets)], \
           [torch.randn(shape, generator=g).to(dtype) for _ in range(n_sets)]


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's own modules (installed copy under baseline/_ref) on the host cores; the oracle's
# restatement of them when that copy is absent
# ----------------------------------------------------------------------------------------------
def host_threads() -> int:
    """Threads the CPU arm uses: every core this process may run on (torchrun exports OMP_NUM_THREADS=1, which
    would otherwise pin the arm to one core)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, n)


def cpu_reference_step_time(cfg, sample_batch, steps, warmup, threads=None):
    """Seconds per fwd+bwd step of the layer on the host, (kind, cores).  kind = "reference": the reference's own
    router / bank / attention modules; "port": oracle/moc_oracle.py."""
    threads = threads or host_threads()
    torch.set_num_threads(threads)
    small = dict(cfg, batch=sample_batch)
    params = make_params(small, "cpu")
    hs, gs = make_hidden(small, 1, 1234, torch.float32)
    from oracle import install_reference
    if install_reference.available():
        from oracle.reference_layer import ReferenceLayer, time_steps
        layer = ReferenceLayer(small, params, "cpu")
        return time_steps(layer, hs[0], gs[0], steps, warmup), "reference", torch.get_num_threads()
    from oracle import moc_oracle as O
    shape = O.LayerShape(cfg["hidden_dim"], cfg["num_heads"], cfg["num_kv_heads"], cfg["num_chapters"],
                         cfg["tokens_per_chapter"], cfg["top_k"], cfg["num_shared_chapters"],
                         cfg["routed_scaling_factor"])
    tensors = dict(params, h_router=hs[0])
    tensors["h_attn"] = tensors["h_router"]
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.memory_layer_fwd_bwd(shape, tensors, gs[0], 0.01, 0.001, autocast_bf16=False)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    return sum(times) / len(times), "port", torch.get_num_threads()


def cpu_sample_text(cfg, sample_b, kind, steps, warmup):
    what = ("the reference's own ChapterRouter / ChapteredMemoryBank / MemoryCrossAttention modules (eager, fp32)"
            if kind == "reference" else "fp32 eager restatement of the reference (oracle port)")
    return (f"{sample_b} of {cfg['batch']} sequences per step (same L, bank, top-k), {what}, "
            f"{warmup} warm-up + {steps} timed steps")


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = dict(PAPER)
    sample_b = args.cpu_sample_batch
    warm = 1
    step_s, kind, cores = cpu_reference_step_time(cfg, sample_b, args.steps, warm)
    tokens = sample_b * cfg["seq"]
    value = tokens / step_s
    sample = cpu_sample_text(cfg, sample_b, kind, args.steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, max(1, args.gpus)),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, n_gpus):
    return {"workload": "paper-shape single memory layer fwd+bwd (bf16 activations, fp32 router; the configuration the headline metric is quoted on)",
            "batch_per_gpu": cfg["batch"], "global_batch": cfg["batch"] * n_gpus, "seq_len": cfg["seq"],
            "hidden_dim": cfg["hidden_dim"], "heads": f"{cfg['num_heads']}x{cfg['hidden_dim'] // cfg['num_heads']}",
            "bank_rows": cfg["num_chapters"] * cfg["tokens_per_chapter"], "chapters": cfg["num_chapters"],
            "tokens_per_chapter": cfg["tokens_per_chapter"], "top_k": cfg["top_k"],
            "shared_chapters": cfg["num_shared_chapters"], "routed_scale": cfg["routed_scaling_factor"],
            "row_norm": "off", "gather": "fused into the K/V projection (TMA gather list over a bf16 copy of the bank)",
            "parallelism": f"dp{n_gpus} (batch sharded, bank replicated)",
            "l2_policy": f"inputs larger than L2: {N_INPUT_SETS} rotating hidden-state batches, "
                         "per-step working set > 400 MB against a 126 MB L2",
            "launch": "one CUDA graph replay per step (forward + backward captured once)"}


# ----------------------------------------------------------------------------------------------
# CUDA arm
# ----------------------------------------------------------------------------------------------
class LayerRunner:
    """One memory layer with its parameters; ``step`` = forward + backward (+ gradient reduction)."""

    def __init__(self, cfg, device, world=1, group=None, use_graph=True, exchange="nccl", wire="bf16", merge=True,
                 fused_gather=True, merged="fp32", sync="collective"):
        import memory_b200 as M
        from memory_b200.graph import GraphedStep
        self.M = M
        self.cfg = cfg
        self.device = device
        self.world = world
        p = make_params(cfg, device)
        self.params = {k: v.requires_grad_(True) for k, v in p.items()}
        # bf16 working copy of the bank: what the fused gather-and-project kernel reads (in training it is refreshed
        # by the optimizer step's own pass over the bank)
        from memory_b200 import ops as _ops
        self.bank_shadow = _ops.cast(self.params["bank"].detach(), torch.bfloat16) if fused_gather else None
        self.g_losses = torch.tensor([0.01, 0.0, 0.001, 0.0], device=device)   # load_balance, auxiliary, z, entropy
        self.reducer = None
        # sets of captured step buffers: step i waits for the exchange (and union-sum) of step i - n_slots.  From four
        # GPUs on those two together outlast a step, so a third set pays (eight GPUs: 1.50 ms per step against 1.56)
        n_slots = max(2, int(os.environ.get("MOC_BENCH_SLOTS", "3" if world >= 4 else "2"))) if use_graph else 1
        if world > 1 and not os.environ.get("MOC_BENCH_NO_REDUCER"):      # (debug: independent replicas, no exchange)
            from memory_b200.distributed import GradReducer
            self.wire_dtype = torch.bfloat16 if wire == "bf16" else torch.float32
            self.reducer = GradReducer(cfg["num_chapters"], cfg["tokens_per_chapter"], cfg["hidden_dim"], device,
                                       group=group, exchange=exchange, wire_dtype=self.wire_dtype, merge=merge,
                                       record_timings=True,
                                       merge_dtype=torch.bfloat16 if merged == "bf16" else torch.float32,
                                       sync=sync, parities=max(2, n_slots))
        # With a reduction the step is captured twice and the two graphs are replayed alternately: the
        # gradients of step i stay untouched in their graph's buffers while step i+1 runs in the other graph, so
        # the exchange reads them in place (no staging copy on the compute stream).
        self.slots = n_slots if ((world > 1 or os.environ.get("MOC_BENCH_TWO_SLOTS")) and use_graph) else 1
        # with a bf16 wire the mean gradient comes out of the union-sum over every rank's bf16 rows, this rank's
        # included: the backward then writes no fp32 rows at all
        self.sinks = [M.SparseBankGrad(self.wire_dtype if self.reducer is not None else None,
                                       wire_only=self.reducer is not None and merge and fused_gather)
                      for _ in range(self.slots)]
        if os.environ.get("MOC_BENCH_DEBUG"):
            torch.cuda.synchronize()
            from memory_b200 import _lib as _L
            print(f"[dbg] before capture: status = {int(_L.status_word(device).item())}", file=sys.stderr)
        self.sink = self.sinks[0]
        self.params["bank"].moc_sparse_grad = self.sink
        self.pending = [None] * self.slots
        self.step_index = 0
        self.prev_snap = None
        self.graphs, self.dense_by_slot = [], []
        self.graphed = None
        if use_graph:
            shape = (cfg["batch"], cfg["seq"], cfg["hidden_dim"])
            h0 = torch.zeros(shape, dtype=torch.bfloat16, device=device).requires_grad_(True)
            g0 = torch.zeros(shape, dtype=torch.bfloat16, device=device)
            h0.data.normal_()
            for s in range(self.slots):
                self.graphs.append(GraphedStep(lambda h, d, s=s: self._fwd_bwd(h, d, s), [h0, g0],
                                               high_priority=world > 1 and not os.environ.get("MOC_BENCH_FLAT_PRIORITY")))
                self.dense_by_slot.append([self.params[k].grad for k in self.DENSE_KEYS])
                if os.environ.get("MOC_BENCH_DEBUG"):
                    torch.cuda.synchronize()
                    from memory_b200 import _lib as _L
                    print(f"[dbg] after capture of slot {s}: status = {int(_L.status_word(device).item())}", file=sys.stderr)
            self.graphed = self.graphs[0]

    DENSE_KEYS = ("router_w", "router_b", "wq", "wk", "wv", "wo")

    def _fwd_bwd(self, h, d_out, slot=0):
        P, cfg = self.params, self.cfg
        for v in P.values():
            v.grad = None
        sink = self.sinks[slot]
        sink.clear()
        P["bank"].moc_sparse_grad = sink
        h.grad = None
        out, losses, _ = self.M.memory_layer(
            h, h, P["bank"], P["router_w"], P["router_b"], P["wq"], P["wk"], P["wv"], P["wo"],
            num_heads=cfg["num_heads"], num_kv_heads=cfg["num_kv_heads"],
            tokens_per_chapter=cfg["tokens_per_chapter"], top_k=cfg["top_k"],
            num_shared_chapters=cfg["num_shared_chapters"], routed_scaling_factor=cfg["routed_scaling_factor"],
            compute_dtype=torch.bfloat16, bank_shadow=self.bank_shadow)
        # d(loss)/d(out) = d_out, loss = <out, d_out> + 0.01 load_balance + 0.001 z_loss: seed the backward
        # directly instead of materialising the inner product on the device
        torch.autograd.backward([out, losses.vector], [d_out, self.g_losses])
        return losses.vector

    def step(self, h, d_out, eager=False):
        slot = self.step_index % self.slots
        self.step_index += 1
        if self.reducer is not None and self.pending[slot] is not None:
            # the exchange that still reads this slot's gradient buffers (started two steps ago) must be over, and
            # with it the union-sum that turned the ranks' rows into the mean gradient an optimizer step applies
            self.pending[slot].wait()
            self.pending[slot].release()
            self.pending[slot] = None
        if self.graphs and not eager:
            loss = self.graphs[slot](h, d_out)
            dense = self.dense_by_slot[slot]
        else:
            loss = self._fwd_bwd(h, d_out, slot)
            dense = [self.params[k].grad for k in self.DENSE_KEYS]
        if self.reducer is not None:
            if self.slots >= 2 and not eager:
                # zero-copy: the exchange of step i runs on the reducer's stream under the compute of step i+1
                snap = self.reducer.snapshot(dense, self.sinks[slot], copy=False)
                self.pending[slot] = self.reducer.reduce_snapshot_async(snap)
            else:
                # one set of buffers: stage a copy on the compute stream, exchange it one step later
                snap = self.reducer.snapshot(dense, self.sinks[slot])
                if self.prev_snap is not None:
                    if self.pending[0] is not None:
                        self.pending[0].wait()
                        self.pending[0].release()
                    self.pending[0] = self.reducer.reduce_snapshot_async(self.prev_snap)
                self.prev_snap = snap
        return loss

    def finish(self):
        """Exchange what is still staged and wait (on the stream) for everything in flight."""
        if self.reducer is None:
            return
        for i, p in enumerate(self.pending):
            if p is not None:
                p.wait()
                p.release()
                self.pending[i] = None
        if self.prev_snap is not None:
            last = self.reducer.reduce_snapshot_async(self.prev_snap)
            last.wait()
            last.release()
            self.prev_snap = None

    def verify_exchange(self, h, d_out):
        """Two consecutive steps (both receive-buffer parities): the exchanged + merged bank gradient and the dense
        bucket against plain NCCL all-reduces of each rank's own gradients divided by the world size."""
        import torch.distributed as dist
        P = self.params
        worst = {"bank": 0.0, "dense": 0.0}
        from memory_b200 import _lib as L
        dbg = os.environ.get("MOC_BENCH_DEBUG")
        for step in range(2):
            slot = step % self.slots
            if self.graphs:
                self.graphs[slot](h, d_out)
                dense = self.dense_by_slot[slot]
                if dbg:
                    torch.cuda.synchronize()
                    print(f"[dbg] verify step {step}: status after replay = {int(L.status_word(self.device).item())}", file=sys.stderr)
            else:
                self._fwd_bwd(h, d_out, slot)
                dense = [P[k].grad for k in self.DENSE_KEYS]
            copy = not (self.slots >= 2)
            snap = self.reducer.snapshot(dense, self.sinks[slot], copy=copy)
            pend = self.reducer.reduce_snapshot_async(snap)
            pend.wait()
            dense_red, bank_red = pend.result()
            got = bank_red.to_dense(P["bank"])
            want = self.sinks[slot].to_dense(P["bank"])
            dist.all_reduce(want)
            want /= self.world
            worst["bank"] = max(worst["bank"], float((got - want).abs().max() / (want.abs().max() + 1e-30)))
            del got, want
            for g_red, g_loc in zip(dense_red, dense):
                ref = g_loc.detach().float().clone()
                dist.all_reduce(ref)
                ref /= self.world
                worst["dense"] = max(worst["dense"], float((g_red - ref).abs().max() / (ref.abs().max() + 1e-30)))
            pend.release()
            torch.cuda.synchronize()
        self.reducer.timings.clear()
        return worst

    def launches_per_step(self):
        """Kernels of this library one step launches (counted on an eager pass into a scratch sink, so the sinks
        that hold the captured steps' gradient buffers are left alone)."""
        from memory_b200 import ops
        shape = (self.cfg["batch"], self.cfg["seq"], self.cfg["hidden_dim"])
        h = torch.randn(shape, device=self.device).bfloat16().requires_grad_(True)
        g = torch.randn(shape, device=self.device).bfloat16()
        n0 = ops.LAUNCHES
        saved_sinks, saved_grads = self.sinks, {k: v.grad for k, v in self.params.items()}
        self.sinks = [self.M.SparseBankGrad(s.wire_dtype, wire_only=s.wire_only) for s in saved_sinks]
        try:
            self._fwd_bwd(h, g)
            torch.cuda.synchronize()
        finally:
            self.sinks = saved_sinks
            for k, v in self.params.items():
                v.grad = saved_grads[k]
            self.params["bank"].moc_sparse_grad = self.sinks[0]
        return ops.LAUNCHES - n0


def time_dominant_kernels(cfg, device, iters=10):
    """The three attention kernels timed alone (CUDA events on the launching stream), inputs > L2:
    Q/KV/dO/O for B=8 are ~150 MB and are rotated over two copies."""
    from memory_b200 import ops
    b, l, d = cfg["batch"], cfg["seq"], cfg["hidden_dim"]
    h, hk = cfg["num_heads"], cfg["num_kv_heads"]
    dh = d // h
    n_sel = (cfg["top_k"] + cfg["num_shared_chapters"]) * cfg["tokens_per_chapter"]
    sets = []
    for s in range(2):
        q = (torch.randn(b, l, d, device=device) * 1.0).bfloat16()
        kv = (torch.randn(b, n_sel, 2 * hk * dh, device=device) * 0.3).bfloat16()
        g = torch.randn(b, l, d, device=device).bfloat16()
        o, lse = ops.attn_fwd(q, kv, h, hk, dh ** -0.5)
        sets.append((q, kv, g, o, lse))
    bufs = (torch.empty_like(sets[0][0]), torch.empty_like(sets[0][1]),
            torch.empty(6, b, h, l, dtype=torch.float32, device=device))
    res = {}

    def timeit(fn):
        for i in range(3):
            fn(sets[i % 2])
        torch.cuda.synchronize()
        evs = []
        for i in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(sets[i % 2]); e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs) / iters

    res["attn_fwd"] = timeit(lambda s: ops.attn_fwd(s[0], s[1], h, hk, dh ** -0.5))
    for s in sets:
        ops.attn_bwd(s[0], s[1], s[3], s[4], s[2], h, hk, dh ** -0.5, parts=1, buffers=bufs)
    res["attn_bwd_dq"] = timeit(lambda s: ops.attn_bwd(s[0], s[1], s[3], s[4], s[2], h, hk, dh ** -0.5, parts=2, buffers=bufs))
    res["attn_bwd_dkv"] = timeit(lambda s: ops.attn_bwd(s[0], s[1], s[3], s[4], s[2], h, hk, dh ** -0.5, parts=4, buffers=bufs))
    return res


def run_kernels_mode(args):
    """``--kernels``: the hot kernels alone at the paper shape (no bank, a few hundred MB), CUDA-event timed; the
    small footprint is what a profiler capture of one launch needs.  Prints one JSON object (not the benchmark
    line).  ``--only a,b`` restricts the list; ``--iters`` sets the launches per kernel."""
    from memory_b200 import _lib as L, ops
    from memory_b200.build import build
    build()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    cfg = dict(PAPER, batch=args.kernels_batch)
    b, l, d, h = cfg["batch"], cfg["seq"], cfg["hidden_dim"], cfg["num_heads"]
    dh = d // h
    n_sel = (cfg["top_k"] + cfg["num_shared_chapters"]) * cfg["tokens_per_chapter"]
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
    proj = 2.0 * b * n_sel * d * 2 * d
    cases = {      # name -> (launch, executed FLOPs, algorithmic FLOPs)
        "attn_fwd": (lambda: ops.attn_fwd(q, kv, h, h, dh ** -0.5), 2 * unit, 2 * unit),
        "attn_bwd_dq": (lambda: ops.attn_bwd(q, kv, o, lse, g, h, h, dh ** -0.5, parts=2, buffers=bufs), 3 * unit, 2 * unit),
        "attn_bwd_dkv": (lambda: ops.attn_bwd(q, kv, o, lse, g, h, h, dh ** -0.5, parts=4, buffers=bufs), 4 * unit, 2 * unit),
        "kv_proj": (lambda: ops.gemm(mem, wkv), proj, proj),
        "q_proj": (lambda: ops.gemm(q.view(b * l, d), wq), 2.0 * b * l * d * d, 2.0 * b * l * d * d),
        "d_mem": (lambda: ops.gemm(kv2, wkv, b_kmajor=False), proj, proj),
        "d_wkv": (lambda: ops.gemm(kv2, mem, a_kmajor=False, b_kmajor=False, out_dtype=torch.float32, split_k=16),
                  proj, proj),
    }
    res = {}
    for name, (fn, executed, algorithmic) in cases.items():
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
        res[name] = {"ms": round(ms, 4), "tflops_executed": round(executed / ms / 1e9, 1),
                     "tflops_algorithmic": round(algorithmic / ms / 1e9, 1)}
    L.check_device_status(dev)
    print(json.dumps({"kernels": res, "batch": b, "shape": "L 1024, 12 x 64 heads, 4160 keys per sequence, bf16"}))


TOKEN_LEVEL = dict(batch=4, seq=2048, hidden_dim=768, num_heads=12, num_kv_heads=12, num_chapters=4097,
                   tokens_per_chapter=64, top_k=16, num_shared_chapters=1, routed_scaling_factor=2.5)


def run_token_mode(args):
    """``--token-level``: the token-level routing variant of the layer (every token selects its own top-16 of 4,096
    routed chapters plus the shared one; B 4, L 2048, d 768, 12 x 64 heads, bf16 activations, fp32 router and bank)
    through the module API -- ``ChapterRouter.route_token_level`` + ``MemoryCrossAttention(token_routing_state=...)``,
    forward and backward.  CUDA-event timed; prints one JSON object (a measurement of that variant, not the
    benchmark line): step time, tokens/s, per-operator device time, and the HBM roofline of the two mixture
    kernels.  ``--token-batch`` shrinks the batch (a profiler capture wants a small footprint)."""
    import memory_b200 as M
    from memory_b200 import _lib as L, ops
    from memory_b200.build import build
    build()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    cfg = dict(TOKEN_LEVEL, batch=args.token_batch)
    b, l, d, h = cfg["batch"], cfg["seq"], cfg["hidden_dim"], cfg["num_heads"]
    c, t, k, s = cfg["num_chapters"], cfg["tokens_per_chapter"], cfg["top_k"], cfg["num_shared_chapters"]
    torch.manual_seed(0)
    bank_shared = (torch.randn(s * t, d, device=dev) * 0.02).requires_grad_(True)
    bank_routed = (torch.randn((c - s) * t, d, device=dev) * 0.02).requires_grad_(True)
    router = M.ChapterRouter(d, c, top_k=k, routing_strategy="token").to(dev)
    attn = M.MemoryCrossAttention(d, h, wo_init_zero=False, compute_dtype=torch.bfloat16).to(dev)
    params = [bank_shared, bank_routed] + list(router.parameters()) + list(attn.parameters())
    hs = [torch.randn(b, l, d, device=dev).bfloat16().requires_grad_(True) for _ in range(2)]
    gs = [torch.randn(b, l, d, device=dev).bfloat16() for _ in range(2)]

    def step(i):
        for p_ in params:
            p_.grad = None
        hs[i % 2].grad = None
        idx, w, losses = router.route_token_level(hs[i % 2], return_losses=True, exclude_prefix_chapters=s)
        state = {"shared_memory": bank_shared, "routed_memory": bank_routed,
                 "token_chapter_indices": (idx - s).to(torch.int32), "tokens_per_chapter": t,
                 "routed_scale": cfg["routed_scaling_factor"], "chapter_weights": w}
        out, _ = attn(hs[i % 2], None, token_routing_state=state)
        torch.autograd.backward([out, losses["load_balance"]], [gs[i % 2], torch.full_like(losses["load_balance"], 0.01)])

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    L.check_device_status(dev)
    steps = min(args.steps, 20)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    ops.TIMER = {}
    step(0)
    torch.cuda.synchronize()
    table = {n: round(sum(a.elapsed_time(z) for a, z in v), 4) for n, v in ops.TIMER.items()}
    ops.TIMER = None
    L.check_device_status(dev)
    peaks = measured_peaks()
    pairs = b * l * k
    kv_bytes = (c - s) * t * 2 * d * 2            # the projected routed bank, bf16 K and V rows
    act = b * l * d * 2
    # compulsory traffic: forward reads every K/V tile once (each chapter is selected), Q once, writes the output;
    # backward reads K/V, Q, dO and writes dK/dV of every selected chapter and dQ
    alg = {"token_mix_fwd": kv_bytes + 2 * act + pairs * 8, "token_mix_bwd": 2 * kv_bytes + 3 * act + pairs * 12}
    roof = {}
    for n, by in alg.items():
        if n in table:
            gbs = by / (table[n] * 1e-3) / 1e9
            roof[n] = {"bound": "hbm", "algorithmic_bytes": by, "ms": table[n], "achieved": round(gbs, 1),
                       "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
                       "peak_source": peaks["source"],
                       "what": "index build + chapter-stationary tcgen05 kernel + slot sum" if n.endswith("fwd")
                               else "chapter-stationary tcgen05 kernel + slot sum of the dQ partials"}
    print(json.dumps({"workload": "token-level routing variant of the memory layer, forward + backward", "config": cfg,
                      "ms_per_step": round(ms, 4), "tokens_per_s": round(b * l / (ms * 1e-3), 1), "steps": steps,
                      "dtype": "bf16", "data": "synthetic", "pairs_per_step": pairs,
                      "operator_ms": dict(sorted(table.items(), key=lambda kv: -kv[1])),
                      "roofline": roof, "max_memory_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2)}))


def verify_against_oracle(runner, cfg, h, device):
    """One-shot check, outside every timed region, of the very tensors the timed steps use: the CUDA layer's
    forward on ``h`` against the CPU oracle's (fp32, eager).  The benchmark draws its router weight from N(0, 0.02),
    so neighbouring chapter ranks can sit within fp32 rounding of each other; the selection is therefore held to
    an fp64 recomputation (exact top-k, in order, up to ties below 16 fp32 ulps) and the output is compared on the
    sequences whose selected chapter sets equal the oracle's."""
    from oracle import moc_oracle as O
    P = runner.params
    with torch.no_grad():
        out, losses, info = runner.M.memory_layer(
            h, h, P["bank"], P["router_w"], P["router_b"], P["wq"], P["wk"], P["wv"], P["wo"],
            num_heads=cfg["num_heads"], num_kv_heads=cfg["num_kv_heads"],
            tokens_per_chapter=cfg["tokens_per_chapter"], top_k=cfg["top_k"],
            num_shared_chapters=cfg["num_shared_chapters"], routed_scaling_factor=cfg["routed_scaling_factor"],
            compute_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    cpu = {k: v.detach().float().cpu() for k, v in P.items()}
    hc = h.detach().float().cpu()
    shape = O.LayerShape(cfg["hidden_dim"], cfg["num_heads"], cfg["num_kv_heads"], cfg["num_chapters"],
                         cfg["tokens_per_chapter"], cfg["top_k"], cfg["num_shared_chapters"],
                         cfg["routed_scaling_factor"])
    with torch.no_grad():
        ref = O.memory_layer(shape, hc, hc, cpu["bank"], cpu["router_w"], cpu["router_b"], cpu["wq"], cpu["wk"],
                             cpu["wv"], cpu["wo"], return_losses=True)
    s_ = cfg["num_shared_chapters"]
    z = hc.double().mean(1) @ cpu["router_w"].double().t() + cpu["router_b"].double()
    p = torch.softmax(z, -1)
    p[:, :s_] = 0
    gi = info["indices"].cpu()
    tau = 16 * 1.1920929e-07
    sel = torch.gather(p, 1, gi)
    ordered = bool((sel[:, :-1] >= sel[:, 1:] * (1 - tau)).all())
    rest = p.clone()
    rest.scatter_(1, gi, 0.0)
    topk = bool((rest.max(-1).values <= sel[:, -1] * (1 + tau)).all())
    same_pos = gi == ref["indices"]
    same_set = torch.tensor([set(a.tolist()) == set(b.tolist()) for a, b in zip(gi, ref["indices"])])
    o, r = out.float().cpu()[same_set], ref["out"][same_set]
    out_err = float((o - r).abs().max() / (r.abs().max() + 1e-30)) if o.numel() else None
    out_bad = int(((o - r).abs() > 2e-2 + 2e-2 * r.abs()).sum()) if o.numel() else None
    loss_err = max(abs(losses[k].item() - ref["losses"][k].item()) / (abs(ref["losses"][k].item()) + 1e-30)
                   for k in ("load_balance", "z_loss"))
    ok = ordered and topk and (out_err is None or out_err < 2e-2) and loss_err < 1e-4 and not out_bad
    return {"ok": bool(ok), "indices_exact_topk_vs_fp64_up_to_16ulp_ties": ordered and topk,
            "index_positions_equal_to_fp32_oracle": f"{int(same_pos.sum())}/{same_pos.numel()}",
            "sequences_with_oracle_chapter_set": f"{int(same_set.sum())}/{same_set.numel()}",
            "out_max_rel_err": out_err, "out_elementwise_violations_2e-2": out_bad,
            "router_loss_rel_err": loss_err}


def run_cuda_arm(args):
    # libraries (NCCL) may print to stdout; the contract is ONE JSON line there, so stdout is pointed at
    # stderr for the run and the line is written to the saved descriptor at the end
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the operators have no CPU path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    from memory_b200 import _lib as L
    from memory_b200.build import build
    if local_rank == 0:
        build()              # one process per node compiles; the others wait and then load the finished library
    if world > 1:
        dist.barrier()
    L.lib()

    cfg = dict(PAPER)
    runner = LayerRunner(cfg, device, world, use_graph=not args.no_graph, exchange=args.exchange, wire=args.wire,
                         merge=not args.no_merge, fused_gather=not args.two_pass_gather, merged=args.merged, sync=args.sync)
    hs_cpu, gs_cpu = make_hidden(cfg, N_INPUT_SETS, 1234 + rank, torch.bfloat16)
    hs = [t.to(device).requires_grad_(True) for t in hs_cpu]
    gs = [t.to(device) for t in gs_cpu]
    tokens_per_step = cfg["batch"] * cfg["seq"] * world

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if os.environ.get("MOC_BENCH_DEBUG"):
        torch.cuda.synchronize()
        print(f"[dbg] after runner init: status = {int(L.status_word(device).item())}", file=sys.stderr)
    if runner.reducer is not None:
        # peer mappings and streams exist before anything is timed
        runner.reducer.prepare(runner.sinks[0], [runner.params[k].grad for k in runner.DENSE_KEYS])
    if os.environ.get("MOC_BENCH_DEBUG"):
        torch.cuda.synchronize()
        print(f"[dbg] after prepare: status = {int(L.status_word(device).item())}", file=sys.stderr)
    # ---- headline: inputs resident in HBM ----
    exchange_check = None
    if world > 1 and not args.no_exchange_check and runner.reducer is not None:
        exchange_check = runner.verify_exchange(hs[0], gs[0])
        barrier()
        L.check_device_status(device)
    for i in range(args.warmup):
        runner.step(hs[i % N_INPUT_SETS], gs[i % N_INPUT_SETS])
    barrier()
    if runner.reducer is not None:
        runner.finish()
        torch.cuda.synchronize()
        runner.reducer.timings.clear()
    L.check_device_status(device)
    # host time to issue one step (eight steps from an idle device, nothing blocks): a step cannot be shorter
    torch.cuda.synchronize()
    t_issue = time.perf_counter()
    for i in range(8):
        runner.step(hs[i % N_INPUT_SETS], gs[i % N_INPUT_SETS])
    host_issue_ms = (time.perf_counter() - t_issue) / 8 * 1e3
    if runner.reducer is not None:
        runner.finish()
    torch.cuda.synchronize()
    if runner.reducer is not None:
        runner.reducer.timings.clear()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    per_step_launches = runner.launches_per_step()
    # the timed block of exactly --steps steps is repeated; the reported time is the median block (max over
    # ranks per block), the spread goes into the line
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    block_ms = []
    for _ in range(args.blocks):
        barrier()
        e0.record()
        for i in range(args.steps):
            runner.step(hs[i % N_INPUT_SETS], gs[i % N_INPUT_SETS])
        runner.finish()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        block_ms.append(ms / args.steps)
    launches = per_step_launches * args.steps
    L.check_device_status(device)
    exchange_ms = None
    if runner.reducer is not None and runner.reducer.timings:
        tm = runner.reducer.timings
        exchange_ms = {"exchange": sum(a.elapsed_time(b) for a, b, _ in tm) / len(tm),
                       "union_sum": sum(b.elapsed_time(c) for _, b, c in tm) / len(tm), "samples": len(tm)}
        runner.reducer.timings = []
        runner.reducer.record_timings = False
    ms_per_step = statistics.median(block_ms)
    value = tokens_per_step / (ms_per_step * 1e-3)

    # ---- end to end: hidden states come from pinned host memory every step, loss read back ----
    pinned = [t.pin_memory() for t in hs_cpu]
    copy_stream = torch.cuda.Stream(device)
    stage = [torch.empty_like(hs[0]).requires_grad_(True) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    loss_host = torch.empty(4, dtype=torch.float32).pin_memory()

    def prefetch(i):
        slot = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            with torch.no_grad():
                stage[slot].copy_(pinned[i % N_INPUT_SETS], non_blocking=True)
            ready[slot].record(copy_stream)

    def e2e_loop(n):
        cur = torch.cuda.current_stream(device)
        for s in range(2):
            consumed[s].record(cur)
        prefetch(0)
        for i in range(n):
            if i + 1 < n:
                prefetch(i + 1)
            cur.wait_event(ready[i % 2])
            loss = runner.step(stage[i % 2], gs[i % N_INPUT_SETS])
            consumed[i % 2].record(cur)
            loss_host.copy_(loss.detach(), non_blocking=True)
        runner.finish()
        torch.cuda.synchronize()

    e2e_loop(max(3, args.warmup))
    e2e_blocks = []
    for _ in range(args.blocks):
        barrier()
        e0.record()
        e2e_loop(args.steps)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        e2e_blocks.append(ms / args.steps)
    clocks = sampler.stop() if sampler else None
    e2e_ms_per_step = statistics.median(e2e_blocks)
    e2e_value = tokens_per_step / (e2e_ms_per_step * 1e-3)
    h2d = hs[0].numel() * hs[0].element_size()

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- rank 0 only: per-kernel timing, roofline, CPU baseline ----
    peaks = measured_peaks()
    f_fwd = layer_flops(cfg)
    f_step = 3.0 * f_fwd
    kern = time_dominant_kernels(cfg, device)
    b, l, d = cfg["batch"], cfg["seq"], cfg["hidden_dim"]
    n_sel = (cfg["top_k"] + cfg["num_shared_chapters"]) * cfg["tokens_per_chapter"]
    attn_unit = 2.0 * b * l * n_sel * d          # one [L x n_sel x D] GEMM over all heads and batch items
    # algorithmic share of each attention kernel: fwd = QK^T + PV; bwd (2x fwd) = dP, dQ | dK, dV
    alg = {"attn_fwd": 2 * attn_unit, "attn_bwd_dq": 2 * attn_unit, "attn_bwd_dkv": 2 * attn_unit}
    executed = {"attn_fwd": 2 * attn_unit, "attn_bwd_dq": 3 * attn_unit, "attn_bwd_dkv": 4 * attn_unit}
    dom = max(kern, key=kern.get)
    achieved = alg[dom] / (kern[dom] * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["tflops"], "traffic": DOMINANT_KERNEL_DRAM_BYTES.get(dom), "peak_source": peaks["source"] + " (burst, kernel timed alone)",
                "executed_tflops": executed[dom] / (kern[dom] * 1e-3) / 1e12,
                "kernel_ms": {k: round(v, 4) for k, v in kern.items()},
                "layer": {"algorithmic_flops_per_step": f_step, "achieved": f_step / (ms_per_step * 1e-3) / 1e12,
                          "peak": peaks["tflops_sustained"], "frac": f_step / (ms_per_step * 1e-3) / 1e12 / peaks["tflops_sustained"],
                          "peak_source": peaks["source"] + " (sustained, whole step)"}}

    verify = None
    if args.verify or (world == 1 and not args.no_verify):
        verify = verify_against_oracle(runner, cfg, hs[0], device)
        L.check_device_status(device)

    # the reference's own eager modules on this GPU (fp32 router, attention under bf16 autocast): the comparison a
    # user of the reference on the same hardware would make; informational, never part of `value`
    gpu_eager = None
    if world == 1 and not args.no_cpu_baseline:
        from oracle import install_reference
        if install_reference.available():
            from oracle.reference_layer import ReferenceLayer, time_steps
            try:
                layer = ReferenceLayer(cfg, {k: v.detach() for k, v in runner.params.items()}, device)
                sec = time_steps(layer, hs[0].detach(), gs[0], 5, 2, autocast_dtype=torch.bfloat16)
                gpu_eager = {"value": cfg["batch"] * cfg["seq"] / sec, "unit": "tokens/s", "ms_per_step": sec * 1e3,
                             "what": "reference modules (ChapterRouter, ChapteredMemoryBank, MemoryCrossAttention, "
                                     "eager torch) on the same GPU, bf16 autocast, fp32 router, full batch"}
                del layer
                torch.cuda.empty_cache()
            except Exception as exc:          # a comparator must never take the measurement down
                gpu_eager = {"unavailable": repr(exc)[:200]}

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        step_s, kind, cores = cpu_reference_step_time(cfg, args.cpu_sample_batch, 2, 1)
        cpu_baseline = {"value": args.cpu_sample_batch * cfg["seq"] / step_s, "unit": "tokens/s", "cores": cores,
                        "kind": kind, "sample": cpu_sample_text(cfg, args.cpu_sample_batch, kind, 2, 1)}

    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(cfg, world),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": 16 * world, "ms_per_step": e2e_ms_per_step,
                "ms_per_step_min_max": [min(e2e_blocks), max(e2e_blocks)]},
        "timed_blocks": {"blocks": args.blocks, "steps_per_block": args.steps, "statistic": "median",
                         "ms_per_step_min_max": [min(block_ms), max(block_ms)]},
        "gpu_launches": launches, "host_issue_ms_per_step": round(host_issue_ms, 4), "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "reference_eager_same_gpu": gpu_eager, "verify": verify,
        "pct_of_bf16_tc_roofline": 100.0 * roofline["layer"]["frac"],
    }
    if args.two_pass_gather:
        line["config"]["gather"] = "two-pass: gathered rows materialised, then the K/V projection"
    if world > 1 and runner.reducer is None:
        line["config"]["gradient_exchange"] = "none (debug: independent replicas)"
    elif world > 1:
        line["config"]["gradient_exchange"] = (
            ("dense bucket: one NCCL all-reduce; " if args.sync == "collective" or runner.reducer._peer is None
             or not runner.reducer._peer.n_dense else
             "dense bucket: pushed by copy engine and summed locally, a flag barrier over peer memory synchronises; ") +
            "bank rows: sparse, " + args.wire + " on the wire, " +
            ("copy-engine pushes into symmetric-memory receive buffers" if runner.reducer.exchange == "peer"
             and runner.reducer._peer is not None else "three fixed-size NCCL all-gathers") +
            ", then a union-sum kernel (fp32 accumulation, " + args.merged + " result) that leaves the mean gradient rows an optimizer step "
            "applies; all of it one step behind the compute on a second stream, inside the timed region")
        line["config"]["exchange_ms_per_step_rank0"] = exchange_ms
        line["exchange_check"] = exchange_check
        if exchange_check is not None:
            line["exchange_check"] = dict(exchange_check, reference=(
                "plain NCCL all-reduces of every rank's own gradients / N; the bank rows a rank contributes are "
                + ("its bf16 rows (the only ones the backward writes in this mode), so the figure shows the exchange "
                   "and the union-sum, not the 2^-9 rounding of the wire" if runner.sinks[0].wire_only
                   else "its fp32 rows")))
    sys.stdout.flush()
    os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--cpu-sample-batch", type=int, default=8,
                    help="sequences per CPU step (8 = the whole per-GPU batch of the workload)")
    ap.add_argument("--blocks", type=int, default=5, help="how many times the timed block of --steps steps is repeated")
    ap.add_argument("--verify", action="store_true", help="check the timed tensors against the CPU oracle first (default at N = 1)")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="issue every kernel from Python instead of a CUDA graph")
    ap.add_argument("--exchange", default="peer", choices=["nccl", "peer"],
                    help="N > 1: how the sparse bank-gradient rows travel (NCCL all-gathers, or copy-engine pushes "
                         "into symmetric-memory receive buffers; falls back to NCCL when those cannot be set up)")
    ap.add_argument("--wire", default="bf16", choices=["bf16", "fp32"],
                    help="N > 1: dtype of the bank-gradient rows between ranks (sums are formed in fp32 at the receiver; "
                         "the reference's DDP sends fp32)")
    ap.add_argument("--sync", default="collective", choices=["collective", "flags"],
                    help="N > 1, peer exchange: 'collective' = the dense bucket's NCCL all-reduce also synchronises the "
                         "exchange; 'flags' = the dense bucket is pushed like the rows and a flag barrier over peer "
                         "memory synchronises (no NCCL kernel in the steady state)")
    ap.add_argument("--merged", default="fp32", choices=["fp32", "bf16"],
                    help="N > 1: dtype of the mean gradient rows the union-sum leaves (sums are formed in fp32)")
    ap.add_argument("--two-pass-gather", action="store_true",
                    help="materialise the gathered rows before the K/V projection instead of reading the chapters "
                         "through the projection kernel's TMA gather list")
    ap.add_argument("--no-exchange-check", action="store_true", help="N > 1: skip the numerical check of the exchange")
    ap.add_argument("--no-merge", action="store_true", help="N > 1: leave the ranks' rows unsummed (exchange only)")
    ap.add_argument("--kernels", action="store_true", help="time the hot kernels alone (small footprint) and exit")
    ap.add_argument("--only", default="", help="--kernels: comma-separated kernel names")
    ap.add_argument("--iters", type=int, default=5, help="--kernels: launches per kernel")
    ap.add_argument("--kernels-batch", type=int, default=8)
    ap.add_argument("--token-level", action="store_true",
                    help="measure the token-level routing variant (top-16 chapters per token) and exit")
    ap.add_argument("--token-batch", type=int, default=4, help="--token-level: sequences of 2,048 tokens")
    args = ap.parse_args()
    if args.kernels:
        run_kernels_mode(args)
        return
    if args.token_level:
        run_token_mode(args)
        return
    if args.warmup < 3 and args.impl == "cuda":
        args.warmup = 3
    if args.impl == "reference":
        if args.steps > 3:
            args.steps = 3          # each CPU step is seconds long; keep the arm within minutes
        run_reference_arm(args)
    else:
        run_cuda_arm(args)


if __name__ == "__main__":
    main()
