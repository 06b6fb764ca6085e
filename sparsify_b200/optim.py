"""Adam on the CUDA kernels, as a torch.optim.Optimizer so that the Trainer can
schedule, checkpoint and resume it exactly like the `torch.optim.Adam` the
reference constructs (sparsify/trainer.py:93-122). State keys (`step`,
`exp_avg`, `exp_avg_sq`) and hyper-parameter names match torch's, so a state
dict written by either loads into the other.

Per parameter one kernel pass does: optional removal of the gradient component
parallel to each parameter row (the reference's
`remove_gradient_parallel_to_decoder_directions`, sparse_coder.py:281-295),
the Adam update, and the refresh of a bf16 shadow copy when one is registered.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import ops


class FusedAdam(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8):
        if lr < 0:
            raise ValueError(f"Invalid learning rate: {lr}")
        defaults = dict(lr=lr, betas=betas, eps=eps)
        super().__init__(params, defaults)
        self._project: set[int] = set()
        self._shadow: dict[int, tuple] = {}
        self._sparse: list = []  # coders whose weight gradients arrive in sparse form

    def project_rows(self, p: Tensor) -> None:
        """Marks `p` (a [M, D] decoder) for gradient projection at every step."""
        self._project.add(id(p))

    def register_shadow(self, p: Tensor, shadow: Tensor, on_refresh=None) -> None:
        """`shadow` (bf16, same shape) is rewritten with the updated value of
        `p` inside the update kernel; `on_refresh()` is called afterwards."""
        self._shadow[id(p)] = (shadow, on_refresh)

    def enable_sparse_update(self, sae) -> bool:
        """Lets `sae` hand its W_enc / W_dec gradients over in sparse form (CSR +
        coefficients) so that one kernel applies them: projection, Adam, decoder
        normalisation and bf16 copies, with no dense gradient in between. Only
        for a single process without gradient accumulation: nothing else may
        need `.grad` of the two matrices. Returns whether it was enabled."""
        W = sae.encoder.weight
        ok = (sae.W_dec is not None and W.is_cuda and W.dtype == torch.float32 and W.shape[1] % 4 == 0
              and W.shape[1] <= 4096 and sae.W_skip is None)
        if ok:
            sae.defer_weight_update = True
            self._sparse.append(sae)
        return ok

    def _group_of(self, p):
        for group in self.param_groups:
            if any(q is p for q in group["params"]):
                return group
        raise KeyError("parameter not in this optimiser")

    def _state_for(self, p):
        state = self.state[p]
        if len(state) == 0:
            state["step"] = torch.tensor(0.0, dtype=torch.float32)
            state["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        return state

    def _sparse_step(self, sae) -> None:
        pend = sae._pending
        W_enc, W_dec = sae.encoder.weight, sae.W_dec
        if W_enc.grad is not None or W_dec.grad is not None:
            sae.materialize_pending()  # dense gradients exist as well: fold and go dense
            return
        sae._pending = None
        hps, states = [], []
        for p in (W_dec, W_enc):
            group, state = self._group_of(p), self._state_for(p)
            state["step"] += 1
            lr = group["lr"]
            hps.append(dict(lr=float(lr), beta1=group["betas"][0], beta2=group["betas"][1],
                            eps=group["eps"], step=int(state["step"])))
            states.append(state)
        shadow_dec = self._shadow.get(id(W_dec), (None, None))
        shadow_enc = self._shadow.get(id(W_enc), (None, None))
        normalize = sae.cfg.normalize_decoder and not sae.cfg.transcode
        ops.rows_adam_(
            pend["row_ptr"], pend["entries"], pend["k"], pend["coefA"], pend["vecA"], pend["coefB"],
            pend["vecB"], pA=W_dec.data, mA=states[0]["exp_avg"], vA=states[0]["exp_avg_sq"],
            shadowA=shadow_dec[0], projectA=id(W_dec) in self._project, normalizeA=normalize,
            norm_eps=torch.finfo(torch.float32).eps, hpA=hps[0], pB=W_enc.data, mB=states[1]["exp_avg"],
            vB=states[1]["exp_avg_sq"], shadowB=shadow_enc[0], hpB=hps[1])
        for _, cb in (shadow_dec, shadow_enc):
            if cb is not None:
                cb()
        if normalize:
            sae._dec_unit_norm = (W_dec.data_ptr(), W_dec._version)

    @torch.no_grad()
    def step(self, closure=None):
        assert closure is None, "Closure is not supported."
        for sae in self._sparse:
            if sae._pending is not None:
                self._sparse_step(sae)
        for group in self.param_groups:
            lr = group["lr"]
            lr = float(lr) if not isinstance(lr, Tensor) else float(lr.item())
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self._state_for(p)
                state["step"] += 1
                g = p.grad
                if g.dtype != torch.float32 or not g.is_contiguous():
                    g = g.to(torch.float32).contiguous()
                shadow, cb = self._shadow.get(id(p), (None, None))
                ops.adam_rows_(
                    p.data, g, state["exp_avg"], state["exp_avg_sq"], lr=lr, beta1=beta1,
                    beta2=beta2, eps=group["eps"], step=int(state["step"]),
                    project=id(p) in self._project and p.dim() == 2, shadow=shadow,
                )
                if cb is not None:
                    cb()
