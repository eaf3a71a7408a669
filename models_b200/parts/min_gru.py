"""minGRU: a gated recurrence whose gates read the current token only.

z = sigmoid(Wz.xn + bz); u = Wx.xn + bx; candidate c = u + 1/2 where u >= 0 and sigmoid(u) elsewhere;
S_t = (1 - z) S_(t-1) + z c, element by element; result Wo.(S_t * silu(Wg.xn)).  The state S is float32,
one vector per sequence in the engine's state area (zero when a sequence starts), and everything between
the first products and the last one is float32 arithmetic in both modes.
"""

from __future__ import annotations

import torch

from ..cache.state import StateRequest
from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Mixer, RunContext
from .linear import stack_rows
from .registry import register_part
from .split import SplitPart


class MinGruMixer(SplitPart, Mixer):
    def parameters(self):
        s, n = self.spec, self.spec.weights
        return [
            ParamRequest(n["z"], (s.state_size, s.hidden_size)),
            ParamRequest(n["z_bias"], (s.state_size,), "bias"),
            ParamRequest(n["x"], (s.state_size, s.hidden_size)),
            ParamRequest(n["x_bias"], (s.state_size,), "bias"),
            ParamRequest(n["gate"], (s.state_size, s.hidden_size)),
            ParamRequest(n["o"], (s.hidden_size, s.state_size)),
        ]

    def load(self, tensors):
        n, rt = self.spec.weights, self.runtime
        first = [rt.matrix(tensors[n[r]]) for r in ("z", "x", "gate")]
        if len({m.dtype for m in first}) > 1:
            first = [m.float() for m in first]
        self.w_in, self.starts = stack_rows(first)
        self.w_o = rt.matrix(tensors[n["o"]])
        self.z_bias = rt.vector(tensors[n["z_bias"]])
        self.x_bias = rt.vector(tensors[n["x_bias"]])

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_o

    def state_request(self):
        return StateRequest((self.spec.state_size,), torch.float32)

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        if run.state is None:
            raise RuntimeError("the minGRU mixer needs its per-sequence state; its run has none")
        width, at = self.spec.state_size, self.starts
        zin, xin, gin = (proj[:, a:a + width] for a in at)
        ops.mingru_scan(zin, xin, gin, self.z_bias, self.x_bias, run.state, batch.slots, batch.cu_q, batch.max_q_len, mid, scale)


register_part("mixer", "mingru", MinGruMixer)
