"""CUDA-graph replay of a fixed-shape step (the decode loops): one graph launch instead of hundreds of kernel launches.

The step function must be free of host reads and host-dependent shapes: positions live in device tensors, stores are
updated in place.  State that a step advances non-idempotently (position counters, recurrent states) is listed by the
caller; it is saved before the warm-up runs and the capture, and restored afterwards, so capturing costs no step."""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch


class GraphedStep:
    def __init__(self, fn: Callable[..., torch.Tensor], example_inputs: Sequence[torch.Tensor],
                 advancing_state: Sequence[torch.Tensor] = (), warmup: int = 2):
        self.fn = fn
        self.static_in = [t.clone() for t in example_inputs]
        saved = [t.clone() for t in advancing_state]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):                       # allocates workspaces, builds fused weights, loads modules
                fn(*self.static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..ops import _common as opc
        self.graph = torch.cuda.CUDAGraph()
        before = opc.LAUNCH_COUNT[0]
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_out = fn(*self.static_in)
        # launches of this library's kernels recorded into the graph: every replay runs them again
        self.kernel_launches_per_replay = opc.LAUNCH_COUNT[0] - before
        for t, s in zip(advancing_state, saved):
            t.copy_(s)
        self.replays = 0

    def __call__(self, *inputs: torch.Tensor):
        for dst, src in zip(self.static_in, inputs):
            dst.copy_(src)
        self.graph.replay()
        self.replays += 1
        from ..ops import _common as opc
        opc.LAUNCH_COUNT[0] += self.kernel_launches_per_replay
        return self.static_out
