"""Grouped-query attention whose softmax weights are mixed across heads before they meet the values.

q = Wq.xn, k = Wk.xn, v = Wv.xn; rotation of the first `rotary_dim` coordinates of every query and key
head; keys and values stored at the token's position (value heads have a size of their own); per head
w_g = softmax(scale * q_g.K) over the visible positions -- j <= i with i - j < window, or j among the first
`keep_first` positions of the sequence; w'_h = sum_g talk[h, g] w_g; head h applies w'_h to the values of
its key/value head h / (heads / kv_heads), and the result is multiplied by sigmoid(gate_h . xn) when the
spec says `gated`; then Wo.  Scores, weights and their mixing are float32 in both modes.
"""

from __future__ import annotations

import torch

from ..cache.kv_cache import KvRequest
from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Mixer, RunContext
from .linear import stack_rows
from .registry import build_part, register_part
from .split import SplitPart


class TalkingAttentionMixer(SplitPart, Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are no multiple of {spec.num_kv_heads} kv heads")
        if spec.window is not None and spec.window <= 0:
            raise ValueError(f"attention window must be positive, got {spec.window}")
        if spec.keep_first < 0:
            raise ValueError(f"keep_first must not be negative, got {spec.keep_first}")
        self.q_width = spec.num_heads * spec.head_dim
        self.k_width = spec.num_kv_heads * spec.head_dim
        self.v_width = spec.num_kv_heads * spec.value_dim
        self.mid_width = spec.num_heads * spec.value_dim
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

    def parameters(self):
        s, n = self.spec, self.spec.weights
        out = [
            ParamRequest(n["q"], (self.q_width, s.hidden_size)),
            ParamRequest(n["k"], (self.k_width, s.hidden_size)),
            ParamRequest(n["v"], (self.v_width, s.hidden_size)),
            ParamRequest(n["talk"], (s.num_heads, s.num_heads)),
            ParamRequest(n["o"], (s.hidden_size, self.mid_width)),
        ]
        if s.gated:
            out.append(ParamRequest(n["gate"], (s.num_heads, s.hidden_size)))
        return out

    def load(self, tensors):
        n, rt = self.spec.weights, self.runtime
        first = [rt.matrix(tensors[n[r]]) for r in (("q", "k", "v", "gate") if self.spec.gated else ("q", "k", "v"))]
        if len({m.dtype for m in first}) > 1:
            first = [m.float() for m in first]
        self.w_in, self.starts = stack_rows(first)
        self.w_o = rt.matrix(tensors[n["o"]])
        self.talk = rt.vector(tensors[n["talk"]])

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_o

    def kv_request(self):
        s = self.spec
        return KvRequest(s.num_kv_heads, s.head_dim, s.window, s.value_dim, s.keep_first if s.window is not None else 0)

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        s, pos = self.spec, self.position
        if run.k_pool is None:
            raise RuntimeError("the attention mixer needs cache pools; its run has none")
        if not run.writes_cache:
            raise RuntimeError("this mixer writes the cache it reads; a run that reads another run's cache is not built for it")
        group = batch.groups[run.group]
        at = self.starts
        q = proj[:, at[0]:at[0] + self.q_width]
        k = proj[:, at[1]:at[1] + self.k_width]
        v = proj[:, at[2]:at[2] + self.v_width]
        gate = proj[:, at[3]:at[3] + s.num_heads] if s.gated else None
        ops.rotate_store(q, k, v, batch.positions, pos.cos if pos else None, pos.sin if pos else None, run.k_pool, run.v_pool,
                         group.slot_mapping, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, pos.rotary_dim if pos else 0)
        ops.talking_attention(q, mid, run.k_pool, run.v_pool, group.block_table, batch.cu_q, batch.kv_lens, batch.max_q_len,
                              s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, s.window, s.keep_first, s.scale,
                              self.talk, gate, scale)


register_part("mixer", "talking_attention", TalkingAttentionMixer)
