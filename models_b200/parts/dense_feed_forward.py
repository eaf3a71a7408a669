"""Dense feed-forward without a gate: down(act(up(xn))); the activation is the spec's, a name of the
activation table (`ops.ACTIVATIONS`; "relu2" is the square of relu).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part
from .registry import register_part
from .split import SplitPart


class DenseFeedForward(SplitPart, Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"feed-forward activation {spec.activation!r} is not built "
                             f"(known: {', '.join(sorted(ops.ACTIVATIONS))})")

    def parameters(self):
        s, n = self.spec, self.spec.weights
        return [ParamRequest(n["up"], (s.intermediate_size, s.hidden_size)),
                ParamRequest(n["down"], (s.hidden_size, s.intermediate_size))]

    def load(self, tensors):
        n, rt = self.spec.weights, self.runtime
        self.w_up = rt.matrix(tensors[n["up"]])
        self.w_down = rt.matrix(tensors[n["down"]])

    def input_matrix(self):
        return self.w_up

    def output_matrix(self):
        return self.w_down

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch=None, run=None, scale: float = 1.0) -> None:
        ops.activate(proj, mid, self.spec.activation, scale)

    def forward(self, xn: torch.Tensor, batch=None, run=None) -> torch.Tensor:
        return SplitPart.forward(self, xn)


register_part("feed_forward", "dense", DenseFeedForward)
