"""CUDA-graph replay of a fixed-shape forward pass.

A forward pass of this library is some ninety small launches; at batch 1 the host cannot enqueue them as fast as the GPU
retires them. `CapturedForward` records the launches once into a CUDA graph and replays it: the pass then costs one graph
launch on the host. During the capture the library's allocator runs in arena mode (`ttb_arena_begin`): every temporary and the
outputs get fixed addresses inside one reserved buffer, so the graph can be replayed as is. The shapes (and, for variable-length
batches, the lengths) are frozen into the graph: use one CapturedForward per shape. Every CapturedForward owns the buffer
its graph runs over (several may be alive and replayed in any order); `close()` or garbage collection releases it.

    fwd = CapturedForward(lambda ids: model(ids), example_ids)      # example_ids: a CUDA tensor, becomes the static input
    seq, pooled = fwd(new_ids)                                      # copies new_ids in, replays, returns the static outputs

The returned tensors are the graph's own output buffers: they are overwritten by the next call.
"""
from typing import Callable

import torch

from ._cxx import cxx

__all__ = ["CapturedForward"]


class CapturedForward:
    def __init__(self, fn: Callable, *static_inputs: torch.Tensor, warmup: int = 3):
        if not static_inputs or not all(isinstance(t, torch.Tensor) and t.is_cuda for t in static_inputs):
            raise ValueError("CapturedForward needs CUDA tensors as static inputs")
        self.device = static_inputs[0].device.index if static_inputs[0].device.index is not None else torch.cuda.current_device()
        self.inputs = static_inputs
        self.fn = fn
        # eager warm-up on a side stream (first-use work such as weight re-layout and cached length tables happens here),
        # measuring how much one pass allocates
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                before = cxx.bytes_allocated_total(self.device)
                fn(*static_inputs)
                per_pass = cxx.bytes_allocated_total(self.device) - before
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self.arena_bytes = int(per_pass * 1.1) + (4 << 20)  # 256-byte alignment of every block + slack
        self.graph = torch.cuda.CUDAGraph()
        cxx.arena_begin(self.device, self.arena_bytes)
        try:
            with torch.cuda.graph(self.graph):
                self.outputs = fn(*static_inputs)
        finally:
            self.arena_used, self._arena = cxx.arena_end(self.device)
            # the capture ran on a side stream: point the library back at the caller's stream
            cxx.set_stream(self.device, torch.cuda.current_stream(self.device).cuda_stream)

    def close(self):
        """Drops the graph and releases its buffer (the returned output tensors become invalid)."""
        arena, self._arena = getattr(self, "_arena", 0), 0
        if arena:
            self.graph = None
            self.outputs = None
            cxx.arena_release(self.device, arena)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __call__(self, *inputs: torch.Tensor):
        for dst, src in zip(self.inputs, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        if self.graph is None:
            raise RuntimeError("this CapturedForward has been closed")
        self.graph.replay()
        return self.outputs
