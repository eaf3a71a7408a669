"""Grouped-query attention with sigmoid weights instead of a softmax.

q = Wq.xn, k = Wk.xn, v = Wv.xn (keys of `head_dim`, values of `value_dim`); with `qk_norm` every query and key head
passes an RMS norm whose gain the heads share; the query at position p is multiplied by
1 + coef * ln(floor((p + 1) / every) + 1); key j <= i gets the weight
sigmoid(scale * q_i.k_j - slope_h * (i - j) + bias_h), slope_h = 2^(-slope_exponent (h + 1) / heads), and the weights are
not normalised over the keys; head h reads the keys and values of head h / (heads / kv_heads); the heads side by side are
multiplied element by element by sigmoid(Wg.xn) when the spec says `gated`; then Wo.  No rotation: positions enter
through the temperature and the distance term only.  Norms, temperature, scores and weights are float32 in both modes.
"""

from __future__ import annotations

import torch

from ..cache.kv_cache import KvRequest
from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Mixer, RunContext
from .linear import stack_rows
from .registry import register_part
from .split import SplitPart


class SigmoidAttentionMixer(SplitPart, Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are no multiple of {spec.num_kv_heads} kv heads")
        if spec.temperature_coef != 0.0 and spec.temperature_every < 1:
            raise ValueError(f"the query temperature's period must be at least 1, got {spec.temperature_every}")
        self.q_width = spec.num_heads * spec.head_dim
        self.k_width = spec.num_kv_heads * spec.head_dim
        self.v_width = spec.num_kv_heads * spec.value_dim
        self.mid_width = spec.num_heads * spec.value_dim

    def _first(self):
        return ("q", "k", "v", "gate") if self.spec.gated else ("q", "k", "v")

    def parameters(self):
        s, n = self.spec, self.spec.weights
        widths = {"q": self.q_width, "k": self.k_width, "v": self.v_width, "gate": self.mid_width}
        out = [ParamRequest(n[r], (widths[r], s.hidden_size)) for r in self._first()]
        out.append(ParamRequest(n["o"], (s.hidden_size, self.mid_width)))
        if s.qk_norm:
            out += [ParamRequest(n["q_norm"], (s.head_dim,), "gain"), ParamRequest(n["k_norm"], (s.head_dim,), "gain")]
        if s.head_bias:
            out.append(ParamRequest(n["head_bias"], (s.num_heads,), "bias"))
        return out

    def load(self, tensors):
        s, n, rt = self.spec, self.spec.weights, self.runtime
        first = [rt.matrix(tensors[n[r]]) for r in self._first()]
        if len({m.dtype for m in first}) > 1:
            first = [m.float() for m in first]
        self.w_in, self.starts = stack_rows(first)
        self.w_o = rt.matrix(tensors[n["o"]])
        self.q_gain = rt.vector(tensors[n["q_norm"]]) if s.qk_norm else None
        self.k_gain = rt.vector(tensors[n["k_norm"]]) if s.qk_norm else None
        self.head_bias = rt.vector(tensors[n["head_bias"]]) if s.head_bias else None

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_o

    def kv_request(self):
        s = self.spec
        return KvRequest(s.num_kv_heads, s.head_dim, None, s.value_dim)

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        s = self.spec
        if run.k_pool is None:
            raise RuntimeError("the attention mixer needs cache pools; its run has none")
        if not run.writes_cache:
            raise RuntimeError("this mixer writes the cache it reads; a run that reads another run's cache is not built for it")
        if scale != 1.0:
            raise ValueError("this mixer's result cannot be scaled on its way out")
        group = batch.groups[run.group]
        at = self.starts
        q = proj[:, at[0]:at[0] + self.q_width]
        k = proj[:, at[1]:at[1] + self.k_width]
        v = proj[:, at[2]:at[2] + self.v_width]
        gate = proj[:, at[3]:at[3] + self.mid_width] if s.gated else None
        ops.norm_store(q, k, v, batch.positions, self.q_gain, self.k_gain, s.eps, s.temperature_coef, s.temperature_every,
                       run.k_pool, run.v_pool, group.slot_mapping, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim)
        ops.gated_attention(q, mid, run.k_pool, run.v_pool, group.block_table, batch.cu_q, batch.kv_lens, batch.max_q_len,
                            s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, "sigmoid", s.scale, s.slope_exponent,
                            self.head_bias, gate, "element" if s.gated else None)


register_part("mixer", "sigmoid_attention", SigmoidAttentionMixer)
