"""Whole-step CUDA graphs for launch-bound training loops.

A small network's training step is a few hundred kernels of a few microseconds each, and the host (Python, the dispatcher,
autograd) cannot issue them as fast as the GPU retires them. `capture(step)` runs `step()` a few times, records one more
run into a CUDA graph and returns a callable that replays it: one launch per step.

What makes this work on this backend: every kernel of the library and every bridged ATen kernel is launched on PyTorch's
current CUDA stream; the caching allocator hands out the same addresses for the same allocation sequence, and after the
warm-up runs it serves a step entirely from its cache (no cudaMalloc inside the capture); the fused optimizers keep their
parameter tables on the device between steps.

Rules for the captured step (the usual CUDA-graph rules):
  * static shapes and static input tensors: refill them in place (`x.copy_(batch)`) before each replay;
  * no host synchronisation inside (`.item()`, printing a device tensor); read results from the tensors the step returned;
  * the graph re-uses the addresses its temporaries had during capture; they sit in the free lists of the side stream
    the capture ran on, which eager work on the default stream does not draw from. Do not call `empty_cache()` while a
    captured step is in use.
"""

import torch

from omarchy_mac_torch_b200 import capi
from omarchy_mac_torch_b200.native import core


class StepGraph:
    def __init__(self, step, warmup=3):
        capi.lib()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        # Autograd's worker threads do not inherit the forward's stream for this device type, so for the warm-up and the
        # capture every thread's work is routed to the side stream explicitly.
        core.set_stream_override(side.cuda_stream, True)
        try:
            with torch.cuda.stream(side):  # warm up off the default stream, as torch.cuda.graph asks
                for _ in range(max(1, warmup)):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            before = capi.lib().omt_launch_count()
            # capture on the stream the warm-up ran on: the allocator keeps free blocks per stream, so the recorded run finds
            # every size it needs in that stream's cache (no cudaMalloc inside the capture), and eager work on other streams
            # never takes those blocks between replays
            # relaxed mode: a size the warm-up did not leave in the cache may still be cudaMalloc'ed inside the capture
            with torch.cuda.graph(self.graph, stream=side, capture_error_mode="relaxed"):
                self.result = step()
        finally:
            core.set_stream_override(0, False)
        #: kernels of this library recorded in the graph (each replay launches them again)
        self.kernels = int(capi.lib().omt_launch_count() - before)

    def __call__(self):
        self.graph.replay()
        return self.result


def capture(step, warmup=3):
    """Record `step()` (after `warmup` eager runs) and return a callable that replays it and returns the tensors the
    recorded run returned."""
    return StepGraph(step, warmup)
