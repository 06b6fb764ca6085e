"""The training hot path as one autograd function: encode -> top-k -> decode ->
FVU, with a hand-scheduled backward.

It computes what SparseCoder.forward composes from `fused_encoder`,
`decoder_impl` and elementwise torch ops (sparsify/sparse_coder.py:205-271 with
sparsify/fused_encoder.py:52-87 and sparsify/xformers.py:139-185 behind it), for
the common case - inputs that need no gradient; AuxK, the skip connection and
Multi-TopK in the bf16 / mixed precisions - in fewer passes over memory:

* `x - b_dec` and the bf16 cast are one kernel;
* the residual e = y - out and its squared sum are one kernel; the gradient of
  the output is s*e with s = -2*dFVU/tv, and s is folded into the [N,k]
  coefficients instead of being applied to an [N,D] tensor;
* the CSR of the selected latents is built once and one pass produces the
  gradients of W_dec, W_enc and b_enc;
* when the optimiser is a FusedAdam that registered this coder
  (`defer_weight_update`), the weight gradients are handed over in sparse form
  and applied by one kernel that also projects, normalises and refreshes the
  bf16 copies, so the dense [M, D] gradients never exist;
* the encoder's input gradient is never gathered: its column sum, which is all
  that b_dec needs, equals W_enc^T grad_b_enc;
* Multi-TopK (sparsify/sparse_coder.py:256-262) selects the top 4k once in the encoder
  kernel (the top k is its leading part), decodes the k and the 4k set, and hands both
  losses' weight gradients over as one sparse problem over a virtual batch of 2N tokens
  (see `_multi_topk_factors`).
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import ops


def _start_all_gather(t: Tensor, world: int):
    """Asynchronous all-gather of `t` along dim 0: (source, gathered buffer, work handle)."""
    import torch.distributed as dist
    t = t.contiguous()
    out = t.new_empty((world * t.shape[0],) + tuple(t.shape[1:]))
    work = dist.all_gather_into_tensor(out.view(-1), t.view(-1), async_op=True)
    return t, out, work


class FusedSaeStep(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, y: Tensor | None, W_enc: Tensor, b_enc: Tensor, W_dec: Tensor,
                b_dec: Tensor, sae, dead_mask: Tensor | None = None, num_dead: int = 0,
                W_skip: Tensor | None = None):
        cfg = sae.cfg
        lowp = sae._lowp()
        comp = torch.bfloat16 if lowp else torch.float32
        M, D = W_enc.shape
        k = cfg.k
        x = x.detach()
        xe = ops.prep_input(x, None if cfg.transcode else b_dec.detach(), comp)
        # Sharded data-parallel update: the rows every rank will need from every other rank
        # (inputs now, residuals after the decode) start travelling as soon as they exist, so
        # that the exchange runs under the encoder GEMM instead of in front of the update.
        early = None
        shard = getattr(sae, "_shard", None)
        multi = bool(cfg.multi_topk)
        if (shard is not None and sae.defer_weight_update and ctx.needs_input_grad[2] and ctx.needs_input_grad[4]
                and not getattr(sae, "ragged_tokens", False) and sae.precision == "bf16" and not multi):
            early = {"vecB": _start_all_gather(xe, shard[1])}
        sae._early = early
        w_enc_src = sae.shadow("encoder.weight") if lowp else W_enc.detach()
        if multi:
            # the top 4k in descending order; its first k columns are the top k
            acts, idx = ops.encode_topk_tc(xe, w_enc_src, b_enc.detach(), 4 * k)
        elif cfg.activation == "topk" and lowp and ops.tc_encode_supported(D, M, k):
            acts, idx = ops.encode_topk_tc(xe, w_enc_src, b_enc.detach(), k)
        elif cfg.activation == "groupmax" and lowp and ops.tc_groupmax_supported(D, M, k):
            acts, idx = ops.encode_groupmax_tc(xe, w_enc_src, b_enc.detach(), k)
        else:
            if lowp and D % 8 == 0:
                pre = ops.gemm_nt(xe, w_enc_src, bias=b_enc.detach(), relu=True, out_dtype=torch.float32)
            else:
                pre = ops.preacts_dense(xe, w_enc_src, b_enc.detach())
            acts, idx = (ops.topk_rows if cfg.activation == "topk" else ops.groupmax_rows)(pre, k)
            del pre
        sae.wait_decoder()  # a decoder update may still be running under the encoder above
        gather_lp = sae.precision == "bf16" and W_dec.dtype == torch.float32
        w_dec_src = sae.shadow("W_dec") if gather_lp else W_dec.detach()
        target = (x if y is None else y.detach())
        if target.dtype not in (torch.float32, torch.bfloat16):
            target = target.to(torch.float32)
        tv = ops.total_variance(target)
        # In the bf16 configuration the residual is kept as bf16 only (it is gathered and
        # exchanged in that form); AuxK and the other precisions need it in fp32.
        e16_only = sae.precision == "bf16" and num_dead == 0
        ctx.skip = None
        ctx.multi = None
        multi_fvu = None
        dots = None
        if multi:
            # FVU on the leading k, Multi-TopK FVU on all 4k; the returned reconstruction, activations
            # and indices are the 4k ones, as in the reference
            lp = sae.precision == "bf16"
            idx_k, acts_k = idx[:, :k].contiguous(), acts[:, :k].contiguous()
            with_dots = ops.decode_dots_supported(w_dec_src, k)
            res_k = ops.decode_residual(idx_k, acts_k, w_dec_src, b_dec.detach(), target, want_out=False,
                                        want_e32=not lp, want_e16=lp, want_dots=with_dots)
            _, ek32, ek16, sse_k = res_k[:4]
            dots = res_k[4] if with_dots else None
            out, e, e16, sse = ops.decode_residual(idx, acts, w_dec_src, b_dec.detach(), target,
                                                   want_e32=not lp, want_e16=lp)
            multi_fvu = sse / tv
            sse = sse_k
            ctx.multi = (ek16 if lp else ek32,)
        elif W_skip is None and D % 4 == 0:
            # decode, residual and its squared sum in one pass - and, where the kernel exists, the
            # residual's dot product with every gathered row, which is the activation gradient up
            # to a scalar: the backward then has no second gather of the decoder rows to do
            with_dots = ops.decode_dots_supported(w_dec_src, k)
            res = ops.decode_residual(idx, acts, w_dec_src, b_dec.detach(), target, want_e32=not e16_only,
                                      want_e16=sae.precision == "bf16", want_dots=with_dots)
            out, e, e16, sse = res[:4]
            dots = res[4] if with_dots else None
        else:
            out = ops.embedding_bag_fwd(idx, acts, w_dec_src, b_dec.detach())
            if W_skip is not None:
                # out += x W_skip^T (sparsify/sparse_coder.py:221-222): tensor-core GEMM that
                # accumulates onto the decode output in its epilogue
                x_b = x if x.dtype == torch.bfloat16 else ops.prep_input(x, None, torch.bfloat16)
                out = ops.gemm_nt(x_b, W_skip.detach().to(torch.bfloat16), beta=1.0, Cin=out, out_dtype=torch.float32)
                ctx.skip = x_b
            sse, e = ops.sq_err(target.to(torch.float32), out, want_diff=True)
            e16 = ops.prep_input(e, None, torch.bfloat16) if sae.precision == "bf16" else None
        if early is not None and e16 is not None:
            early["vecA"] = _start_all_gather(e16, shard[1])
        fvu = sse / tv

        # ---- AuxK (sparsify/sparse_coder.py:231-249) in compact dense form: the dead
        # latents' pre-activations are one small GEMM over the gathered dead rows of
        # W_enc, the auxiliary reconstruction another over the dead rows of W_dec.
        auxk = fvu.new_zeros(())
        ctx.aux = None
        if num_dead > 0:
            dead_idx = sae.dead_indices(dead_mask)  # no read-back when the mask was prepared
            nd = int(dead_idx.numel())
            pad = (-nd) % 8  # the GEMM wants a multiple of 8 in its contraction dimension
            k_aux = target.shape[-1] // 2
            scale = min(nd / k_aux, 1.0)
            k_aux = min(k_aux, nd)
            We = w_enc_src[dead_idx].to(torch.bfloat16)
            Wd = w_dec_src[dead_idx].to(torch.bfloat16)
            be = b_enc.detach()[dead_idx].to(torch.float32)
            if pad:
                We = torch.cat([We, We.new_zeros(pad, D)])
                Wd = torch.cat([Wd, Wd.new_zeros(pad, D)])
                be = torch.cat([be, be.new_zeros(pad)])
            xe_b = xe if xe.dtype == torch.bfloat16 else xe.to(torch.bfloat16)
            P = ops.gemm_nt(xe_b, We, bias=be, relu=True, out_dtype=torch.float32)  # [N, nd + pad]
            if nd > k_aux:  # keep each row's k_aux largest, zero the rest (one pass, bf16 out)
                Pb = ops.topk_mask_rows(P, k_aux)
            else:
                Pb = P.to(torch.bfloat16)
            e_hat = ops.gemm_nt(Pb, ops.transpose_bf16(Wd), bias=b_dec.detach(), out_dtype=torch.float32)
            sse_aux, diff = ops.sq_err(e_hat, e, want_diff=True)  # diff = e_hat - e
            auxk = scale * sse_aux / tv
            ctx.aux = (Pb, diff, dead_idx, nd, scale)

        ctx.save_for_backward(xe, idx, acts, e if e is not None else e16, tv)
        ctx.e16 = e16
        ctx.dots = dots  # e . W_dec[idx] of the residual as saved (None where it was not computed)
        ctx.w_enc_src, ctx.w_dec_src = w_enc_src, w_dec_src
        ctx.shape = (M, D, k)
        ctx.transcode = cfg.transcode
        ctx.sae = sae
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(idx)
        if multi_fvu is None:
            multi_fvu = fvu.new_zeros(())
        return out, acts, idx, fvu, auxk, multi_fvu

    @staticmethod
    def backward(ctx, g_out, g_acts, g_idx, g_fvu, g_auxk, g_multi=None):
        xe, idx, acts, e, tv = ctx.saved_tensors
        M, D, k = ctx.shape
        dev = e.device
        if ctx.multi is not None:
            return FusedSaeStep._backward_multi_topk(ctx, g_out, g_acts, g_fvu, g_multi)
        # d fvu / d out = -2 e / tv
        s = (-2.0 * g_fvu / tv).to(torch.float32) if g_fvu is not None else torch.zeros((), device=dev)
        if g_out is not None:
            gout = torch.addcmul(g_out.to(torch.float32), e.to(torch.float32), s)  # general case: materialise
            scale = torch.ones((), device=dev)
        else:
            gout, scale = e, s

        if g_out is None and ctx.dots is not None:
            gacts = ctx.dots * scale  # the forward already dotted the residual with the gathered rows
        else:
            gacts = ops.embedding_bag_bwd_acts(idx, gout, ctx.w_dec_src) * scale
        if g_acts is not None:
            gacts = gacts + g_acts
        # ---- AuxK: dense gradient rows for the dead latents, and its share of b_dec ----
        extra = None
        g_b_dec_aux = None
        if ctx.aux is not None and g_auxk is not None:
            Pb, diff, dead_idx, nd, aux_scale = ctx.aux
            coef = (2.0 * aux_scale * g_auxk / tv).to(torch.float32)
            g_ehat = (diff * coef).to(torch.bfloat16)
            N = g_ehat.shape[0]
            if N % 8 == 0:
                rows = ops.gemm_nt(ops.transpose_bf16(Pb), ops.transpose_bf16(g_ehat), out_dtype=torch.float32)
            else:
                rows = Pb.float().T @ g_ehat.float()
            extra = (dead_idx, rows[:nd].contiguous())
            g_b_dec_aux = ops.weighted_colsum(diff) * coef

        g_W_skip = None
        if ctx.skip is not None and ctx.needs_input_grad[9]:
            # grad W_skip = gout^T x = scale * (e^T)(x^T)^T, both operands put into K-major form
            x_b = ctx.skip
            g_b = gout.to(torch.bfloat16)
            if x_b.shape[0] % 8 == 0:
                g_W_skip = ops.gemm_nt(ops.transpose_bf16(g_b), ops.transpose_bf16(x_b), out_dtype=torch.float32)
            else:
                g_W_skip = g_b.float().T @ x_b.float()
            g_W_skip = g_W_skip * scale

        row_ptr, entries = ops.csr_build(idx, M)
        sae = ctx.sae
        if sae._pending is not None:
            sae.materialize_pending()  # a second backward before the optimiser step: go dense
        if sae.defer_weight_update and ctx.needs_input_grad[2] and ctx.needs_input_grad[4]:
            # The optimiser consumes the sparse form directly (sc_rows_adam): keep the
            # CSR and the coefficient / row tensors instead of two dense [M, D] gradients.
            # in the bf16 configuration the residual rows are gathered (and, across ranks,
            # exchanged) as bf16 like every other gathered operand
            if sae.precision != "bf16":
                vecA = gout
            elif g_out is None and ctx.e16 is not None:
                vecA = ctx.e16  # the forward already wrote the residual as bf16
            else:
                vecA = ops.prep_input(gout, None, torch.bfloat16)
            sae._pending = dict(row_ptr=row_ptr, entries=entries, k=k, idx=idx, coefA=acts * scale,
                                vecA=vecA, coefB=gacts, vecB=xe, extra=extra)
            early = getattr(sae, "_early", None)
            if early is not None:
                # sharded update: the small factors (indices and the two coefficient arrays, already
                # divided by the world size) follow the row arrays as soon as they exist, so that the
                # optimiser step finds them gathered
                world = sae._shard[1]
                pend = sae._pending
                early["idx"] = _start_all_gather(idx.to(torch.int32), world)
                early["coefA"] = _start_all_gather((pend["coefA"].to(torch.float32) / world).reshape(idx.shape), world)
                early["coefB"] = _start_all_gather((gacts.to(torch.float32) / world).reshape(idx.shape), world)
            g_W_dec = g_W_enc = None
            g_b_enc = ops.csr_segment_sum(row_ptr, entries, gacts, M)
        else:
            res = ops.rows_accumulate(row_ptr, entries, k, M, D, acts * scale, gout,
                                      coefB=gacts, vecB=xe, biasB=True)
            g_W_dec, g_W_enc, g_b_enc = res["gradA"], res["gradB"], res["gbiasB"]
            if extra is not None:
                g_W_dec.index_add_(0, extra[0], extra[1])
        g_b_dec = ops.weighted_colsum(gout) * scale
        if not ctx.transcode:
            # minus the column sum of the encoder's input gradient
            g_b_dec = g_b_dec - ops.weighted_colsum(ctx.w_enc_src, g_b_enc)
        if g_b_dec_aux is not None:
            g_b_dec = g_b_dec + g_b_dec_aux
        return None, None, g_W_enc, g_b_enc, g_W_dec, g_b_dec, None, None, None, g_W_skip


    @staticmethod
    def _backward_multi_topk(ctx, g_out, g_acts, g_fvu, g_multi):
        """loss = g_fvu * FVU(top k) + g_multi * FVU(top 4k). In the reference the 4k activations are
        taken from `pre_acts`, whose gradient FusedEncoder.backward drops
        (sparsify/fused_encoder.py:52-87): the Multi-TopK term reaches W_dec and b_dec only, the
        encoder learns from the top-k term alone. With r4 = s4 * e4 (+ a gradient arriving through
        the returned reconstruction) and rk = sk * ek (s = -2 g / total variance):
          grad acts[n, j]  = rk[n] . W_dec[idx[n, j]]                     for j < k only
          grad W_dec[m]    = sum over (n, j) with idx = m of acts[n, j] (r4[n] + [j < k] rk[n])
          grad W_enc[m]    = sum of grad acts[n, j] x'[n],   grad b_enc[m] = sum of grad acts[n, j]
        The two vectors per token (r4 for the entries j >= k, u = r4 + rk for j < k) make this one
        sparse problem over 2N virtual tokens with 3k entries each: token n holds the entries
        j >= k with vector e4 (scale folded into the coefficients), token N + n the entries j < k
        (padded with invalid indices, which the CSR build skips) with vector u."""
        xe, idx, acts, e4, tv = ctx.saved_tensors
        (ek,) = ctx.multi
        M, D, k = ctx.shape
        dev = e4.device
        N = idx.shape[0]
        zero = torch.zeros((), device=dev)
        s4 = (-2.0 * g_multi / tv).to(torch.float32) if g_multi is not None else zero
        sk = (-2.0 * g_fvu / tv).to(torch.float32) if g_fvu is not None else zero
        lp = e4.dtype == torch.bfloat16
        if g_out is not None:  # general case: materialise the 4k residual with its incoming gradient
            r4 = torch.addcmul(g_out.to(torch.float32), e4.to(torch.float32), s4)
            r4 = r4.to(torch.bfloat16) if lp else r4
            vec4, scale4 = r4, torch.ones((), device=dev)
        else:
            vec4, scale4 = e4, s4
        idx_k = idx[:, :k].contiguous()
        if ctx.dots is not None:
            gacts_k = ctx.dots * sk                                               # [N, k], from the forward
        else:
            gacts_k = ops.embedding_bag_bwd_acts(idx_k, ek, ctx.w_dec_src) * sk
        u = (vec4.to(torch.float32) * scale4).add_(ek.to(torch.float32) * sk)
        u = u.to(torch.bfloat16) if lp else u
        pad_i = idx.new_full((N, 2 * k), -1)
        pad_f = acts.new_zeros((N, 2 * k))
        idx_v = torch.cat([idx[:, k:], torch.cat([idx_k, pad_i], dim=1)])
        coefA_v = torch.cat([acts[:, k:] * scale4, torch.cat([acts[:, :k], pad_f], dim=1)])
        coefB_v = torch.cat([acts.new_zeros((N, 3 * k)), torch.cat([gacts_k, pad_f], dim=1)])
        vecA_v = torch.cat([vec4, u])
        vecB_v = torch.cat([xe, xe])
        kv = 3 * k
        row_ptr, entries = ops.csr_build(idx_v, M)
        sae = ctx.sae
        if sae._pending is not None:
            sae.materialize_pending()
        if sae.defer_weight_update and ctx.needs_input_grad[2] and ctx.needs_input_grad[4]:
            sae._pending = dict(row_ptr=row_ptr, entries=entries, k=kv, idx=idx_v, coefA=coefA_v, vecA=vecA_v,
                                coefB=coefB_v, vecB=vecB_v, extra=None)
            g_W_dec = g_W_enc = None
            g_b_enc = ops.csr_segment_sum(row_ptr, entries, coefB_v, M)
        else:
            res = ops.rows_accumulate(row_ptr, entries, kv, M, D, coefA_v, vecA_v, coefB=coefB_v, vecB=vecB_v,
                                      biasB=True)
            g_W_dec, g_W_enc, g_b_enc = res["gradA"], res["gradB"], res["gbiasB"]
        g_b_dec = ops.weighted_colsum(vec4) * scale4 + ops.weighted_colsum(ek) * sk
        if not ctx.transcode:
            g_b_dec = g_b_dec - ops.weighted_colsum(ctx.w_enc_src, g_b_enc)
        return None, None, g_W_enc, g_b_enc, g_W_dec, g_b_dec, None, None, None, None


def fused_supported(sae, x: Tensor, num_dead: int) -> bool:
    """The fused function covers the common training case; everything else runs
    the composed path in SparseCoder.forward."""
    return (
        x.is_cuda
        and sae.W_dec is not None
        and (sae.W_skip is None or (sae._lowp() and x.shape[-1] % 8 == 0))
        and (not sae.cfg.multi_topk
             or (sae.cfg.activation == "topk" and sae._lowp() and num_dead == 0 and sae.W_skip is None
                 and ops.tc_encode_supported(x.shape[-1], sae.num_latents, 4 * sae.cfg.k)))
        and (num_dead == 0 or (sae._lowp() and x.shape[-1] % 8 == 0))
        and not x.requires_grad
        and x.shape[-1] % 4 == 0
        and sae.dtype == torch.float32
    )
