"""Two mixers side by side on the same rows: left_scale * left(xn) + right_scale * right(xn).

Both must be split parts (parts/split.py): their first matrices are stacked into one product and their last
matrices put side by side into another, with each mixer's scale applied (in float32) to what it hands to
the last product.  At most one of the two may ask for keys and values, and at most one for per-sequence
state: a run of the schedule owns one of each.
"""

from __future__ import annotations

import torch

from .base import Mixer, RunContext
from .linear import stack_columns, stack_rows
from .registry import build_part, register_part
from .split import SplitPart


class SideBySideMixer(SplitPart, Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.left = build_part("mixer", spec.left, runtime)
        self.right = build_part("mixer", spec.right, runtime)
        for side in (self.left, self.right):
            if not all(hasattr(side, name) for name in ("input_matrix", "output_matrix", "inner")):
                raise ValueError(f"{type(side).__name__} is no split part: it cannot stand beside another mixer")
        if self.left.kv_request() is not None and self.right.kv_request() is not None:
            raise ValueError("both mixers ask for keys and values; a run owns one cache")
        if self.left.state_request() is not None and self.right.state_request() is not None:
            raise ValueError("both mixers ask for per-sequence state; a run owns one state")

    def parameters(self):
        return self.left.parameters() + self.right.parameters()

    def load(self, tensors):
        self.left.load(tensors)
        self.right.load(tensors)
        first = [self.left.input_matrix(), self.right.input_matrix()]
        last = [self.left.output_matrix(), self.right.output_matrix()]
        if first[0].dtype != first[1].dtype or last[0].dtype != last[1].dtype:
            first, last = [m.float() for m in first], [m.float() for m in last]
        self.w_in, self.in_starts = stack_rows(first)
        self.w_out, self.mid_starts, self.mid_padded = stack_columns(last)
        self.in_widths = [m.shape[0] for m in first]
        self.mid_widths = [m.shape[1] for m in last]

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_out

    def kv_request(self):
        return self.left.kv_request() or self.right.kv_request()

    def state_request(self):
        return self.left.state_request() or self.right.state_request()

    def decode_class(self, sequences: int, max_kv_len: int):
        return tuple(side.decode_class(sequences, max_kv_len) if hasattr(side, "decode_class") else 0
                     for side in (self.left, self.right))

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        if self.mid_padded:
            mid.zero_()  # columns that meet the last matrix's zero padding must be finite
        for side, a, n, c, m, s in zip((self.left, self.right), self.in_starts, self.in_widths, self.mid_starts, self.mid_widths,
                                       (self.spec.left_scale, self.spec.right_scale)):
            side.inner(proj[:, a:a + n], mid[:, c:c + m], batch, run, scale * s)


register_part("mixer", "side_by_side", SideBySideMixer)
