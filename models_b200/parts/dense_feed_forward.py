"""Dense feed-forward without a gate: down(act(up(xn))); the activation is the spec's, a name of the
activation table (`ops.ACTIVATIONS`; "relu2" is the square of relu), or "xielu": a_pos z^2 + z/2 above zero and
a_neg (exp(z) - 1 - z) + z/2 below, with a_pos = softplus(p), a_neg = 1/2 + softplus(q) of the layer's two shape numbers
(a tensor of two, `weights["act"]`; the two constants are worked out once, on the host, when the tensor is loaded).
"""

from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part
from .registry import register_part
from .split import SplitPart


SHAPED_ACTIVATIONS = ("xielu",)  # activations with learned shape numbers


def _softplus(z: float) -> float:
    return max(z, 0.0) + math.log1p(math.exp(-abs(z)))


class DenseFeedForward(SplitPart, Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.activation not in ops.ACTIVATIONS and spec.activation not in SHAPED_ACTIVATIONS:
            raise ValueError(f"feed-forward activation {spec.activation!r} is not built "
                             f"(known: {', '.join(sorted(ops.ACTIVATIONS) + list(SHAPED_ACTIVATIONS))})")
        self.shaped = spec.activation in SHAPED_ACTIVATIONS

    def parameters(self):
        s, n = self.spec, self.spec.weights
        out = [ParamRequest(n["up"], (s.intermediate_size, s.hidden_size)),
               ParamRequest(n["down"], (s.hidden_size, s.intermediate_size))]
        if self.shaped:
            out.append(ParamRequest(n["act"], (2,), "bias"))
        return out

    def load(self, tensors):
        n, rt = self.spec.weights, self.runtime
        self.w_up = rt.matrix(tensors[n["up"]])
        self.w_down = rt.matrix(tensors[n["down"]])
        if self.shaped:
            p, q = (float(v) for v in tensors[n["act"]].detach().to("cpu", torch.float64).tolist())
            self.a_pos, self.a_neg = _softplus(p), 0.5 + _softplus(q)

    def input_matrix(self):
        return self.w_up

    def output_matrix(self):
        return self.w_down

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch=None, run=None, scale: float = 1.0) -> None:
        if self.shaped:
            ops.xielu(proj, mid, self.a_pos, self.a_neg, scale)
        else:
            ops.activate(proj, mid, self.spec.activation, scale)

    def forward(self, xn: torch.Tensor, batch=None, run=None) -> torch.Tensor:
        return SplitPart.forward(self, xn)


register_part("feed_forward", "dense", DenseFeedForward)
