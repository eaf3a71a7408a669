"""Retention: linear attention with a fixed decay per head, no softmax and no denominator.

q = Wq.xn, k = Wk.xn (heads of `head_dim`), v = Wv.xn (heads of `value_dim`); q and k are rotated over the first
coordinates of every head (the spec's `position`), k is then multiplied by `key_scale`; per head
S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t; every head's o_t is divided by its root mean square, the heads
side by side are multiplied by silu(Wg.xn), then Wo.  The state S is float32 [heads, head_dim, value_dim] per sequence in
the engine's state area (zero when a sequence starts); the mixer keeps no keys or values.  Everything between the first
products and the last one is float32 arithmetic in both modes.
"""

from __future__ import annotations

import torch

from ..cache.state import StateRequest
from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Mixer, RunContext
from .linear import stack_rows
from .registry import build_part, register_part
from .split import SplitPart


class RetentionMixer(SplitPart, Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if len(spec.decay) != spec.num_heads:
            raise ValueError(f"{len(spec.decay)} decays for {spec.num_heads} heads")
        self.qk_width = spec.num_heads * spec.head_dim
        self.v_width = spec.num_heads * spec.value_dim
        self.position = None
        if spec.position is not None:
            if spec.position.rotary_dim > spec.head_dim:
                raise ValueError(f"rotary_dim {spec.position.rotary_dim} exceeds head_dim {spec.head_dim}")
            if spec.position.pairing != "half":
                raise ValueError("this mixer rotates split-half pairs only")
            key = ("position", spec.position, runtime.max_positions)
            if key not in runtime.shared:
                runtime.shared[key] = build_part("position", spec.position, runtime)
            self.position = runtime.shared[key]
        self.decay = torch.tensor(list(spec.decay), dtype=torch.float32, device=runtime.device)

    def parameters(self):
        s, n = self.spec, self.spec.weights
        return [ParamRequest(n["q"], (self.qk_width, s.hidden_size)), ParamRequest(n["k"], (self.qk_width, s.hidden_size)),
                ParamRequest(n["v"], (self.v_width, s.hidden_size)), ParamRequest(n["gate"], (self.v_width, s.hidden_size)),
                ParamRequest(n["o"], (s.hidden_size, self.v_width))]

    def load(self, tensors):
        n, rt = self.spec.weights, self.runtime
        first = [rt.matrix(tensors[n[r]]) for r in ("q", "k", "v", "gate")]
        if len({m.dtype for m in first}) > 1:
            first = [m.float() for m in first]
        self.w_in, self.starts = stack_rows(first)
        self.w_o = rt.matrix(tensors[n["o"]])

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_o

    def state_request(self):
        s = self.spec
        return StateRequest((s.num_heads, s.head_dim, s.value_dim), torch.float32)

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        s, pos = self.spec, self.position
        if run.state is None:
            raise RuntimeError("the retention mixer needs its per-sequence state; its run has none")
        at = self.starts
        q = proj[:, at[0]:at[0] + self.qk_width]
        k = proj[:, at[1]:at[1] + self.qk_width]
        v = proj[:, at[2]:at[2] + self.v_width]
        g = proj[:, at[3]:at[3] + self.v_width]
        ops.retention_scan(q, k, v, g, batch.positions, pos.cos if pos else None, pos.sin if pos else None,
                           pos.rotary_dim if pos else 0, self.decay, s.key_scale, s.eps, run.state, batch.slots, batch.cu_q,
                           s.num_heads, s.head_dim, s.value_dim, mid, scale, batch.max_q_len)


register_part("mixer", "retention", RetentionMixer)
