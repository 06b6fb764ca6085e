"""Sparse decoder op with the surface of sparsify/xformers.py:188-217:
``xformers_embedding_bag(indices, weight, per_sample_weights)`` =
sum_j per_sample_weights[n, j] * weight[indices[n, j]], differentiable in
`weight` and `per_sample_weights`.

Backward follows sparsify/xformers.py:139-185: a latent-major CSR of the index
matrix, then one pass per latent that writes every row of the weight gradient
(zeros for unused latents); the gradient of the per-sample weights is a
gathered dot product.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import ops


class EmbeddingBag(torch.autograd.Function):
    @staticmethod
    def forward(ctx, indices: Tensor, weight: Tensor, per_sample_weights: Tensor,
                weight_lp: Tensor | None = None):
        """weight_lp: optional bf16 copy of `weight` to gather from instead."""
        ctx.save_for_backward(indices, weight, per_sample_weights)
        ctx.weight_lp = weight_lp
        src = weight_lp if weight_lp is not None else weight
        out = ops.embedding_bag_fwd(indices, per_sample_weights, src)
        return out if weight_lp is not None else out.to(weight.dtype)

    @staticmethod
    def backward(ctx, gradient):
        indices, weight, psw = ctx.saved_tensors
        M, D = weight.shape
        k = indices.shape[1]
        g = gradient.detach().to(torch.float32).contiguous()
        weight_g = psw_g = None
        if ctx.needs_input_grad[2]:
            src = ctx.weight_lp if ctx.weight_lp is not None else weight
            psw_g = ops.embedding_bag_bwd_acts(indices, g, src).to(psw.dtype)
        if ctx.needs_input_grad[1]:
            row_ptr, entries = ops.csr_build(indices, M)
            res = ops.rows_accumulate(row_ptr, entries, k, M, D, psw, g)
            weight_g = res["gradA"].to(weight.dtype)
        return None, weight_g, psw_g, None


def xformers_embedding_bag(indices: Tensor, weight: Tensor, per_sample_weights: Tensor,
                           weight_lp: Tensor | None = None) -> Tensor:
    return EmbeddingBag.apply(indices, weight, per_sample_weights, weight_lp)
