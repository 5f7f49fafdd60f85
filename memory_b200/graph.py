"""CUDA-graph capture of a whole forward+backward step of the memory layer.

One step launches ~60 short kernels; issued one by one from Python the host becomes the limit
(each ctypes call, tensor-map encode and output allocation costs tens of microseconds).  Shapes are
static during training, so the step is captured once and replayed.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedStep:
    """``fn(*inputs)`` captured into a CUDA graph.

    ``fn`` must be free of host synchronisation and must produce its results (including any
    ``.grad`` it leaves on parameters) with the same shapes every call.  Calling the object copies
    the new inputs into the captured input buffers, replays the graph and returns the captured
    outputs -- the same tensor objects every time, valid until the next call.
    """

    def __init__(self, fn: Callable, inputs: Sequence[torch.Tensor], warmup: int = 3, high_priority: bool = False):
        """``high_priority``: capture on a high-priority stream.  Kernel nodes keep the priority of the stream they
        were captured on, so a replayed step is scheduled ahead of work on ordinary streams -- a gradient exchange
        running beside the next step then fills the gaps instead of taking SM slots from it."""
        self.fn = fn
        self.static_inputs = []
        for t in inputs:
            s = t.detach().clone()
            s.requires_grad_(t.requires_grad)
            self.static_inputs.append(s)
        device = self.static_inputs[0].device
        # warm-up runs on a side stream, capture on the capture stream: the AccumulateGrad nodes of the
        # parameters are created under different streams by design
        if hasattr(torch.autograd.graph, "set_warn_on_accumulate_grad_stream_mismatch"):
            torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                fn(*self.static_inputs)
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        self.graph = torch.cuda.CUDAGraph()
        capture_stream = torch.cuda.Stream(device, priority=-1) if high_priority else None
        with torch.cuda.graph(self.graph, stream=capture_stream):
            self.outputs = fn(*self.static_inputs)

    def load(self, *inputs: torch.Tensor) -> None:
        """Copy new values into the captured input buffers (asynchronous on the current stream)."""
        with torch.no_grad():
            for s, t in zip(self.static_inputs, inputs):
                s.copy_(t, non_blocking=True)

    def replay(self):
        self.graph.replay()
        return self.outputs

    def __call__(self, *inputs: torch.Tensor):
        self.load(*inputs)
        return self.replay()
