"""Softmax attention whose keys and values are expanded from one low-rank row per position.

q = Wq.xn (heads of `head_dim`); c = rmsnorm(Wd.xn) with a gain, `latent_dim` numbers: the only thing the cache keeps
(one "key head" of latent_dim, no values).  Head h has k_j = Uk_h.c_j and v_j = Uv_h.c_j, so its score
scale * q_i.k_j equals scale * (Uk_h^T q_i).c_j and its result sum_j w_j v_j equals Uv_h.(sum_j w_j c_j): the query is taken
into the latent space once per token and head, the attention runs over the cached rows themselves (all heads read the same
rows, as key and as value), and the result is taken out of the latent space once per token and head.  No key or value is
ever expanded.  With `gated`, head h's result is multiplied by sigmoid((Wg.xn)_h); then Wo.  No positions enter.  The
norm, the scores and the softmax are float32 in both modes.
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


class LatentAttentionMixer(SplitPart, Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.q_width = spec.num_heads * spec.head_dim
        self.mid_width = spec.num_heads * spec.value_dim

    def _first(self):
        return ("q", "down", "gate") if self.spec.gated else ("q", "down")

    def parameters(self):
        s, n = self.spec, self.spec.weights
        widths = {"q": self.q_width, "down": s.latent_dim, "gate": s.num_heads}
        out = [ParamRequest(n[r], (widths[r], s.hidden_size)) for r in self._first()]
        out += [ParamRequest(n["down_norm"], (s.latent_dim,), "gain"),
                ParamRequest(n["up_k"], (self.q_width, s.latent_dim)),
                ParamRequest(n["up_v"], (self.mid_width, s.latent_dim)),
                ParamRequest(n["o"], (s.hidden_size, self.mid_width))]
        return out

    def load(self, tensors):
        s, n, rt = self.spec, self.spec.weights, self.runtime
        first = [rt.matrix(tensors[n[r]]) for r in self._first()]
        if len({m.dtype for m in first}) > 1:
            first = [m.float() for m in first]
        self.w_in, self.starts = stack_rows(first)
        self.w_o = rt.matrix(tensors[n["o"]])
        self.latent_gain = rt.vector(tensors[n["down_norm"]])
        dtype = rt.compute_dtype
        # per head: [latent_dim, head_dim] takes a query into the latent space, [value_dim, latent_dim] a result out of it
        self.into_latent = rt.matrix(tensors[n["up_k"]]).to(dtype).view(s.num_heads, s.head_dim, s.latent_dim).transpose(1, 2).contiguous()
        self.out_of_latent = rt.matrix(tensors[n["up_v"]]).to(dtype).view(s.num_heads, s.value_dim, s.latent_dim).contiguous()

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_o

    def kv_request(self):
        return KvRequest(1, self.spec.latent_dim, None, 0)  # one row per position, read as key and as value

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        s = self.spec
        if run.k_pool is None:
            raise RuntimeError("the latent attention mixer needs a cache pool; its run has none")
        if not run.writes_cache:
            raise RuntimeError("this mixer writes the cache it reads; a run that reads another run's cache is not built for it")
        if scale != 1.0:
            raise ValueError("this mixer's result cannot be scaled on its way out")
        group = batch.groups[run.group]
        at = self.starts
        q = proj[:, at[0]:at[0] + self.q_width]
        down = proj[:, at[1]:at[1] + s.latent_dim]
        gate = proj[:, at[2]:at[2] + s.num_heads] if s.gated else None
        ops.norm_store(None, down, None, batch.positions, None, self.latent_gain, s.eps, 0.0, 1, run.k_pool, None,
                       group.slot_mapping, 0, 1, s.latent_dim, 0)
        rows = proj.shape[0]
        q_latent = torch.empty((rows, s.num_heads * s.latent_dim), dtype=proj.dtype, device=proj.device)
        ops.head_linear(q, self.into_latent, q_latent, s.num_heads)
        mixed = torch.empty_like(q_latent)
        ops.gated_attention(q_latent, mixed, run.k_pool, None, group.block_table, batch.cu_q, batch.kv_lens, batch.max_q_len,
                            s.num_heads, 1, s.latent_dim, s.latent_dim, "softmax", s.scale)
        ops.head_linear(mixed, self.out_of_latent, mid, s.num_heads, gate)


register_part("mixer", "latent_attention", LatentAttentionMixer)
