"""Matrix products y = x . W^T for row-major W [out, in] (integrallis/models,
backend-java/.../ops/TensorOps.java:61-63), chosen by the weight's storage.

bfloat16 weights: with up to 8 activation rows (decode) this package's own weight-streaming kernel
(csrc/skinny_gemm.cu; it takes up to 32 rows but pays off up to 8); with 9 to 128 rows its tcgen05 kernel
with the weights as the 128-row operand and K split over a thread-block cluster
(csrc/wide_gemm_tcgen05.cu); with more rows (prefill) its tcgen05 kernel csrc/gemm_tcgen05.cu.  What is
left -- a matrix whose sizes are no multiples of 8, which TMA cannot address -- falls to a library product
(bfloat16 inputs, float accumulation), the place where the reference too calls a library (its matmul is
VectorUtil.batchDotProduct of an external artifact).
float32 weights: this package's own true-32-bit kernel, in both modes -- a matrix stored in 32-bit is
multiplied in 32-bit.
"""

from __future__ import annotations

import torch

from ..kernels import ops


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    if not x.is_cuda:
        raise ops.KernelError("models_b200 runs on a CUDA device only; there is no CPU path")
    if weight.dtype == torch.float32:
        a = x if x.dtype == torch.float32 else x.float()
        out = ops.gemm_f32(a, weight)
        return out if out_dtype == torch.float32 else out.to(out_dtype)
    if weight.dtype != torch.bfloat16:
        raise ops.KernelError(f"matrices are bfloat16 or float32, got {weight.dtype}")
    a = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    if ops.skinny_pays(weight, a.shape[0]) and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 \
            and out_dtype in (torch.bfloat16, torch.float32):
        # decode: few rows, the weights stream once through this package's own kernel
        return ops.skinny_gemm(weight, ops.EPI_F32 if out_dtype == torch.float32 else ops.EPI_BF16, x=a)
    if (ops.gemm_tcgen05_takes(weight, rows=a.shape[0]) and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
            and out_dtype in (torch.bfloat16, torch.float32)):
        # many rows: this package's tcgen05 kernels (wide decode form up to 128 rows, prefill form above)
        return ops.tensor_core_gemm(a, weight, ops.EPI_F32 if out_dtype == torch.float32 else ops.EPI_BF16)
    if out_dtype == torch.float32:
        return torch.mm(a, weight.t(), out_dtype=torch.float32)
    return torch.mm(a, weight.t())


def add_linear(x: torch.Tensor, a: torch.Tensor, weight: torch.Tensor) -> None:
    """x += a . weight^T for the float32 residual stream x [rows, out] and weight [out, in].  Where one of
    this package's bfloat16 products takes the sizes, the addition rides in its epilogue (the product's sums
    stay float32 all the way into the stream); otherwise the product's float32 result is added by a kernel."""
    if not x.is_cuda:
        raise ops.KernelError("models_b200 runs on a CUDA device only; there is no CPU path")
    rows = a.shape[0]
    if weight.dtype == torch.bfloat16 and a.dtype == torch.bfloat16 and a.stride(1) == 1 and a.stride(0) % 8 == 0 \
            and a.data_ptr() % 16 == 0:
        if ops.skinny_pays(weight, rows):
            ops.skinny_gemm(weight, ops.EPI_RESIDUAL, x=a, out=x)
            return
        if ops.gemm_tcgen05_takes(weight, ops.EPI_RESIDUAL, rows):
            ops.tensor_core_gemm(a, weight, ops.EPI_RESIDUAL, out=x)
            return
    ops.residual_add(x, linear(a, weight, torch.float32))


def stack_rows(matrices, multiple: int = 8):
    """Matrices [n_i, k] stacked into one [sum of padded n_i, k], each padded with zero rows to a multiple of
    `multiple` so that every part starts on a 16-byte boundary of a product's result row; returns the matrix
    and each part's first row."""
    parts, starts, at = [], [], 0
    for m in matrices:
        starts.append(at)
        parts.append(m)
        pad = -m.shape[0] % multiple
        if pad:
            parts.append(torch.zeros((pad, m.shape[1]), dtype=m.dtype, device=m.device))
        at += m.shape[0] + pad
    return torch.cat(parts, dim=0).contiguous(), starts


def stack_columns(matrices, multiple: int = 8):
    """Matrices [n, k_i] put side by side into one [n, sum of padded k_i], each padded with zero columns to a
    multiple of `multiple`; returns the matrix, each part's first column, and whether any column is padding
    (the activations that meet padding columns must then be finite, zeros for instance)."""
    parts, starts, at, padded = [], [], 0, False
    for m in matrices:
        starts.append(at)
        parts.append(m)
        pad = -m.shape[1] % multiple
        if pad:
            parts.append(torch.zeros((m.shape[0], pad), dtype=m.dtype, device=m.device))
            padded = True
        at += m.shape[1] + pad
    return torch.cat(parts, dim=1).contiguous(), starts, padded
