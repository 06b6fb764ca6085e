"""Dense bf16 linear map y = x W^T on the tcgen05 GEMM kernel, with autograd.
Used for the transcoder skip connection (sparsify/sparse_coder.py:221-222) in
the bf16 / mixed precisions; the fp32 precision keeps an fp32 matmul."""

from __future__ import annotations

import torch
from torch import Tensor

from . import ops


class LinearNT(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, W: Tensor) -> Tensor:
        """x [N, K], W [M, K] -> x W^T [N, M] (fp32 result, bf16 operands)."""
        xb = x.detach().to(torch.bfloat16).contiguous()
        wb = W.detach().to(torch.bfloat16).contiguous()
        ctx.save_for_backward(xb, wb)
        ctx.dtypes = (x.dtype, W.dtype)
        return ops.gemm_nt(xb, wb, out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, g: Tensor):
        xb, wb = ctx.saved_tensors
        gb = g.detach().to(torch.bfloat16).contiguous()
        gx = gW = None
        if ctx.needs_input_grad[0]:
            # g [N, M] W [M, K] = g (W^T)^T
            gx = ops.gemm_nt(gb, ops.transpose_bf16(wb), out_dtype=torch.float32).to(ctx.dtypes[0])
        if ctx.needs_input_grad[1]:
            # g^T [M, N] x [N, K] = g^T (x^T)^T
            gW = ops.gemm_nt(ops.transpose_bf16(gb), ops.transpose_bf16(xb), out_dtype=torch.float32).to(ctx.dtypes[1])
        return gx, gW


def linear_nt(x: Tensor, W: Tensor) -> Tensor:
    return LinearNT.apply(x, W)
