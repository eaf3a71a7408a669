"""Parts that are a first product, something in between, and a last product.

Many mixers and feed-forwards have this shape: some matrices read the normalised rows, something that is
not a matrix product happens to the results, and one matrix maps back to the model's width.  A part that
says so -- `input_matrix()` ([n_in, width], its first matrices stacked), `output_matrix()` ([width, n_mid])
and `inner(proj, mid, batch, run, scale)` (from its columns of the first product to `scale` times its
columns of the last product's input; both are column slices of wider tensors) -- can be put beside others
by a block that runs ONE first product and ONE last product for all of them (parts/parallel_block.py).
Alone, such a part runs through `forward` below.
"""

from __future__ import annotations

import torch

from .linear import linear


class SplitPart:
    """Mixin: `forward` for a part that offers input_matrix / output_matrix / inner."""

    def forward(self, xn: torch.Tensor, batch=None, run=None) -> torch.Tensor:
        dtype = self.runtime.compute_dtype
        w_out = self.output_matrix()
        proj = linear(xn, self.input_matrix(), dtype)
        mid = torch.empty((xn.shape[0], w_out.shape[1]), dtype=dtype, device=xn.device)
        self.inner(proj, mid, batch, run, 1.0)
        return linear(mid, w_out, dtype)
