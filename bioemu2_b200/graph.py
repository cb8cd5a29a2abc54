"""One CUDA-graph replay per forward for a trunk that is called again and again with tensors of one shape.

A 48-block trunk is ~1,200 kernel launches; issued one by one from Python they cost a few milliseconds of host time
per forward that a serving loop does not need to pay.  ``trunk.graphed(s, z, mask)`` captures the block loop once on
static device buffers; calling the result copies the new inputs into those buffers (from pinned host memory or from
the device, asynchronously on the current stream), replays the graph and hands back the static output buffers, which
stay valid until the next call.  The kernels, their order and their results are those of the eager ``forward``.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import _lib


class GraphedTrunk:
    def __init__(self, trunk, s: Tensor, z: Tensor, mask: Tensor, warmup: int = 2) -> None:
        from .pairformer import PairformerModule

        if trunk.training:
            raise RuntimeError("bioemu2_b200 modules are inference-only: call .eval()")
        dev = next(trunk.parameters()).device
        if dev.type != "cuda":
            raise ValueError("the trunk must be on a CUDA device before it is captured")
        self.trunk = trunk
        self.composite = isinstance(trunk, PairformerModule)  # token mask [B, N]; the PairMixer trunk takes a pair mask
        want = (z.shape[0], z.shape[1]) if self.composite else tuple(z.shape[:3])
        if tuple(mask.shape) != want:
            raise ValueError(f"mask shape {tuple(mask.shape)}, expected {want}")
        self.s_in = torch.empty(s.shape, dtype=s.dtype, device=dev)
        self.z_in = torch.empty(z.shape, dtype=z.dtype, device=dev)
        self.mask_in = torch.empty(mask.shape, dtype=torch.bool, device=dev)
        self.s_out, self.z_out = torch.empty_like(self.s_in), torch.empty_like(self.z_in)
        self.s_in.copy_(s)
        self.z_in.copy_(z)
        self.mask_in.copy_(mask)
        with torch.no_grad():
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):  # warm-up outside the capture: weight packing, shared-memory attributes
                for _ in range(max(warmup, 1)):
                    self._run()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._run()
        _lib.raise_if_device_wait()

    def _run(self) -> None:
        self.s_out.copy_(self.s_in)
        self.z_out.copy_(self.z_in)
        if self.composite:
            pm = (self.mask_in[:, :, None] & self.mask_in[:, None, :]).to(torch.uint8)
            self.trunk.forward_(self.s_out, self.z_out, self.mask_in, pm)
        else:
            pm = self.mask_in.to(torch.uint8)
            for layer in self.trunk.layers:
                layer.forward_(self.z_out, pm)

    def __call__(self, s: Tensor, z: Tensor, mask: Tensor | None = None) -> tuple[Tensor, Tensor]:
        """Same shapes and dtypes as at capture; ``mask=None`` keeps the captured mask.  Returns ``(s, z)`` in static
        buffers that the next call overwrites."""
        if s.shape != self.s_in.shape or z.shape != self.z_in.shape or s.dtype != self.s_in.dtype or z.dtype != self.z_in.dtype:
            raise ValueError("a captured trunk takes the shapes and dtypes it was captured with")
        self.s_in.copy_(s, non_blocking=True)
        self.z_in.copy_(z, non_blocking=True)
        if mask is not None:
            if mask.shape != self.mask_in.shape:
                raise ValueError("a captured trunk takes the mask shape it was captured with")
            self.mask_in.copy_(mask, non_blocking=True)
        self.graph.replay()
        _lib.raise_if_device_wait()
        return self.s_out, self.z_out
