"""A pre-norm layer whose sublayer results pass a gate on their way into the residual stream:

    h = mixer_norm(x);         x += sigmoid(Gm.h + bm) * mixer(h)
    h = feed_forward_norm(x);  x += sigmoid(Gf.h + bf) * feed_forward(h)      (if the layer has a feed-forward)

Both sublayers are split parts (parts/split.py): a first product, something in between, a last product.  A gate reads the
same rows as its sublayer's first matrices, so its matrix is stacked under them and one product serves both; the last
product's float32 result, the gate's columns of the first product and the bias then meet in one kernel that adds into the
float32 stream.  A sublayer is thus a norm, two matrix products, its own
kernels between them, and one element-wise kernel; with few rows (decode) the norm rides in the first product and the
gated add in the last one's epilogue.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part, RunContext, as_delta
from .linear import linear, stack_rows
from .registry import build_part, register_part


class GatedResidualBlock(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = build_part("norm", spec.feed_forward_norm, runtime)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime)
        self.parts = [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]
        for part in (self.mixer, self.feed_forward):
            if part is not None and not all(hasattr(part, name) for name in ("input_matrix", "output_matrix", "inner")):
                raise ValueError(f"{type(part).__name__} is no split part: a gated-residual block cannot run it")
        self.width = spec.mixer_norm.size

    def _gates(self):
        gates = [("mixer_gate", "mixer_gate_bias")]
        if self.feed_forward is not None:
            gates.append(("feed_forward_gate", "feed_forward_gate_bias"))
        return gates

    def parameters(self):
        out = [p for part in self.parts for p in part.parameters()]
        n = self.spec.weights
        for matrix, bias in self._gates():
            out += [ParamRequest(n[matrix], (self.width, self.width)), ParamRequest(n[bias], (self.width,), "bias")]
        return out

    def load(self, tensors):
        for part in self.parts:
            part.load(tensors)
        n, rt = self.spec.weights, self.runtime
        self.stacked = []  # per sublayer: (first matrices with the gate's under them, the gate's first row, bias)
        for part, (matrix, bias) in zip((self.mixer, self.feed_forward), self._gates()):
            first = [part.input_matrix(), rt.matrix(tensors[n[matrix]])]
            if first[0].dtype != first[1].dtype:
                first = [m.float() for m in first]
            w_in, starts = stack_rows(first)
            self.stacked.append((w_in, starts[1], rt.vector(tensors[n[bias]])))

    def _sublayer(self, x, norm, part, stacked, batch, run):
        w_in, gate_at, bias = stacked
        dtype = self.runtime.compute_dtype
        rows = x.shape[0]
        if (self.runtime.mode == "bfloat16" and getattr(norm, "foldable", False) and w_in.dtype == torch.bfloat16
                and ops.skinny_pays(w_in, rows, with_norm=True)):
            # few rows (decode): the norm rides in the first product, which normalises the float32 rows it reads
            proj = ops.skinny_gemm(w_in, ops.EPI_BF16, xf=x, gain=norm.weight, eps=norm.spec.eps)
        else:
            proj = linear(norm.forward(x, None), w_in, dtype)
        w_out = part.output_matrix()
        mid = torch.empty((rows, w_out.shape[1]), dtype=dtype, device=x.device)
        part.inner(proj[:, :part.input_matrix().shape[0]], mid, batch, run, 1.0)  # (rows of padding lie before the gate's)
        gate = proj[:, gate_at:gate_at + self.width]
        if (self.runtime.mode == "bfloat16" and w_out.dtype == torch.bfloat16 and proj.dtype == torch.bfloat16
                and ops.skinny_pays(w_out, rows) and mid.stride(0) % 8 == 0 and mid.data_ptr() % 16 == 0):
            ops.skinny_gemm_gated_residual(w_out, mid, x, gate, bias)  # few rows: gate and add ride in the last product
            return
        delta = linear(mid, w_out, torch.float32)
        ops.gated_residual_add(x, gate, bias, delta)

    def forward(self, x: torch.Tensor, pending, batch, run: RunContext):
        if as_delta(pending) is not None:
            ops.residual_add(x, as_delta(pending))
        self._sublayer(x, self.mixer_norm, self.mixer, self.stacked[0], batch, run)
        if self.feed_forward is not None:
            self._sublayer(x, self.feed_forward_norm, self.feed_forward, self.stacked[1], batch, run)
        return None


register_part("block", "prenorm_gated", GatedResidualBlock)
