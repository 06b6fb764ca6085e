"""Encoder op with the reference's surface (sparsify/fused_encoder.py:7-103):
``fused_encoder(input, weight, bias, k, activation) -> EncoderOutput`` and the
``FusedEncoder`` autograd function with its sparse backward.

Forward = relu(x W^T + b) followed by top-k (or groupmax). bf16 operands (or an
active CUDA bf16 autocast, which is how the reference's SparseCoder.forward
runs) take the tcgen05 kernel that keeps the [N, M] pre-activations on chip;
fp32 operands take the exact fp32 FMA kernel. Backward mirrors
sparsify/fused_encoder.py:52-87: grad-x is a k-row gather of W, grad-W / grad-b
are per-latent row accumulates over the selected latents only, and the gradient
arriving at ``pre_acts`` is dropped exactly as the reference drops it.
"""

from __future__ import annotations

from typing import Literal, NamedTuple

import torch
from torch import Tensor

from . import ops


class EncoderOutput(NamedTuple):
    top_acts: Tensor
    """Activations of the top-k latents."""

    top_indices: Tensor
    """Indices of the top-k features."""

    pre_acts: Tensor
    """Activations before the top-k selection."""


def _autocast_bf16(t: Tensor) -> bool:
    return (
        t.is_cuda
        and torch.is_autocast_enabled("cuda")
        and torch.get_autocast_dtype("cuda") == torch.bfloat16
    )


class FusedEncoder(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, bias, k: int, activation: Literal["groupmax", "topk"],
                need_pre_acts: bool = True, weight_bf16: Tensor | None = None, wide_k: int = 0):
        """
        input:  (N, D)   weight: (M, D)   bias: (M,)
        need_pre_acts: materialise the dense (N, M) pre-activations (the
            reference always does); False returns an empty placeholder.
        weight_bf16: optional up-to-date bf16 copy of `weight` for the
            tensor-core path (saves the per-call cast).
        wide_k: when > k, also return the top-`wide_k` set (values, indices;
            no gradient, as the reference drops the gradient of `pre_acts`), of
            which the top-k is the leading part. Multi-TopK uses it in place of
            a second selection over dense pre-activations.
        """
        if activation not in ("topk", "groupmax"):
            raise ValueError(f"Unknown activation: {activation}")
        N, D = input.shape
        M = weight.shape[0]
        low_precision = (
            weight_bf16 is not None
            or (input.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16)
            or _autocast_bf16(input)
        )
        x_c = input.detach().contiguous()
        preacts = None
        wide = None
        k_sel = max(k, wide_k)
        if activation == "topk" and low_precision and not need_pre_acts and ops.tc_encode_supported(D, M, k_sel):
            xb = x_c if x_c.dtype == torch.bfloat16 else ops.prep_input(x_c, None, torch.bfloat16)
            if weight_bf16 is None:
                w_c = weight.detach().contiguous()
                weight_bf16 = w_c if w_c.dtype == torch.bfloat16 else ops.cast_bf16(w_c)
            values, indices = ops.encode_topk_tc(xb, weight_bf16, bias, k_sel)
            if k_sel > k:  # descending order: the top-k is the leading part
                wide = (values, indices)
                values, indices = values[:, :k].contiguous(), indices[:, :k].contiguous()
            x_saved = xb
        elif (activation == "groupmax" and low_precision and not need_pre_acts
              and ops.tc_groupmax_supported(D, M, k)):
            xb = x_c if x_c.dtype == torch.bfloat16 else ops.prep_input(x_c, None, torch.bfloat16)
            if weight_bf16 is None:
                w_c = weight.detach().contiguous()
                weight_bf16 = w_c if w_c.dtype == torch.bfloat16 else ops.cast_bf16(w_c)
            values, indices = ops.encode_groupmax_tc(xb, weight_bf16, bias, k)
            x_saved = xb
        else:
            if low_precision:
                # same operand rounding as the tensor-core path, fp32 accumulation
                xb = x_c if x_c.dtype == torch.bfloat16 else ops.prep_input(x_c, None, torch.bfloat16)
                wb = weight_bf16 if weight_bf16 is not None else (
                    weight.detach().contiguous() if weight.dtype == torch.bfloat16
                    else ops.cast_bf16(weight.detach().contiguous()))
                if D % 8 == 0:
                    # tensor-core GEMM with bias + ReLU in the epilogue, fp32 result
                    preacts = ops.gemm_nt(xb, wb, bias=bias, relu=True, out_dtype=torch.float32)
                else:
                    preacts = ops.preacts_dense(xb, wb, bias)
                x_saved = xb
            else:
                preacts = ops.preacts_dense(x_c.float(), weight.detach().float(), bias)
                x_saved = x_c
            if activation == "topk":
                values, indices = ops.topk_rows(preacts, k)
                if wide_k > k:
                    wide = ops.topk_rows(preacts, wide_k)
            else:
                values, indices = ops.groupmax_rows(preacts, k)
        ctx.save_for_backward(x_saved, weight, indices)
        ctx.has_bias = bias is not None
        ctx.weight_bf16 = weight_bf16
        ctx.k = k
        ctx.in_dtype, ctx.w_dtype = input.dtype, weight.dtype
        ctx.b_dtype = bias.dtype if bias is not None else None
        if preacts is None:
            preacts = values.new_empty(0)
        values = values.to(weight.dtype) if not low_precision else values
        if wide is None:
            wide = (values.new_empty(0), indices.new_empty(0))
        ctx.mark_non_differentiable(indices, *wide)
        return values, indices, preacts, wide[0], wide[1]

    @staticmethod
    def backward(ctx, grad_values, grad_indices, grad_preacts, grad_wide_values=None, grad_wide_indices=None):
        x_saved, weight, indices = ctx.saved_tensors
        grad_input = grad_weight = grad_bias = None
        gv = grad_values.detach().to(torch.float32).contiguous()
        M, D = weight.shape
        k = indices.shape[1]

        # --- Grad w.r.t. input: sum_j gv[n,j] * W[idx[n,j]] ---
        if ctx.needs_input_grad[0]:
            w_src = ctx.weight_bf16 if ctx.weight_bf16 is not None else weight
            grad_input = ops.embedding_bag_fwd(indices, gv, w_src).to(ctx.in_dtype)

        # --- Grad w.r.t. weight and bias: per-latent accumulate of gv * x ---
        want_w = ctx.needs_input_grad[1]
        want_b = ctx.has_bias and ctx.needs_input_grad[2]
        if want_w or want_b:
            row_ptr, entries = ops.csr_build(indices, M)
            res = ops.rows_accumulate(row_ptr, entries, k, M, D, gv, x_saved, biasA=want_b)
            if want_w:
                grad_weight = res["gradA"].to(ctx.w_dtype)
            if want_b:
                grad_bias = res["gbiasA"].to(ctx.b_dtype)

        return grad_input, grad_weight, grad_bias, None, None, None, None, None


def fused_encoder(
    input,
    weight,
    bias,
    k: int,
    activation: Literal["groupmax", "topk"],
    *,
    need_pre_acts: bool = True,
    weight_bf16: Tensor | None = None,
) -> EncoderOutput:
    """
    Linear layer followed by `activation` (top-k or groupmax) with a backward
    pass restricted to the selected latents. Same arguments and result as the
    reference's ``fused_encoder``; the keyword-only extras let a caller skip
    the dense ``pre_acts`` and reuse a bf16 weight copy.
    """
    return EncoderOutput(
        *FusedEncoder.apply(input, weight, bias, k, activation, need_pre_acts, weight_bf16)[:3]  # type: ignore
    )
