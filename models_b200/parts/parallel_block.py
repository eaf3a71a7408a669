"""A layer with ONE norm whose rows feed the mixer and the feed-forward side by side:
h = norm(x); x += mixer(h) + feed_forward(h).

Both sublayers are split parts (parts/split.py), so the layer is two matrix products with the parts' own
kernels between them: every first matrix of the layer, stacked, times h; then each part turns its columns
of that result into its columns of the last product's input; then the last matrices, side by side, times
that input, added into the float32 residual stream in the product's epilogue.  The sum over the sublayers
is thus part of the product's float32 accumulation.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, RunContext
from .linear import add_linear, linear, stack_columns, stack_rows
from .registry import build_part, register_part


class ParallelBlock(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.norm = build_part("norm", spec.norm, runtime)
        self.mixer_norm = self.norm  # the norm that reads the stream when this layer begins
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime) if spec.feed_forward is not None else None
        self.parts = [self.norm, self.mixer] + ([self.feed_forward] if self.feed_forward is not None else [])
        for part in self.parts[1:]:
            if not all(hasattr(part, name) for name in ("input_matrix", "output_matrix", "inner")):
                raise ValueError(f"{type(part).__name__} is no split part: a parallel block cannot run it")

    def parameters(self):
        return [p for part in self.parts for p in part.parameters()]

    def load(self, tensors):
        for part in self.parts:
            part.load(tensors)
        sublayers = self.parts[1:]
        first = [part.input_matrix() for part in sublayers]
        last = [part.output_matrix() for part in sublayers]
        if len({m.dtype for m in first + last}) > 1:
            first, last = [m.float() for m in first], [m.float() for m in last]
        self.w_in, self.in_starts = stack_rows(first)
        self.w_out, self.mid_starts, self.mid_padded = stack_columns(last)
        self.in_widths = [m.shape[0] for m in first]
        self.mid_widths = [m.shape[1] for m in last]

    def forward(self, x: torch.Tensor, pending, batch, run: RunContext):
        if pending is not None:
            ops.residual_add(x, pending)
        dtype = self.runtime.compute_dtype
        h = self.norm.forward(x)
        proj = linear(h, self.w_in, dtype)
        make = torch.zeros if self.mid_padded else torch.empty
        mid = make((x.shape[0], self.w_out.shape[1]), dtype=dtype, device=x.device)
        for part, a, n, c, m in zip(self.parts[1:], self.in_starts, self.in_widths, self.mid_starts, self.mid_widths):
            part.inner(proj[:, a:a + n], mid[:, c:c + m], batch, run, 1.0)
        add_linear(x, mid, self.w_out)
        return None


register_part("block", "parallel", ParallelBlock)
