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

    def project_rows(self, p: Tensor) -> None:
        """Marks `p` (a [M, D] decoder) for gradient projection at every step."""
        self._project.add(id(p))

    def register_shadow(self, p: Tensor, shadow: Tensor, on_refresh=None) -> None:
        """`shadow` (bf16, same shape) is rewritten with the updated value of
        `p` inside the update kernel; `on_refresh()` is called afterwards."""
        self._shadow[id(p)] = (shadow, on_refresh)

    @torch.no_grad()
    def step(self, closure=None):
        assert closure is None, "Closure is not supported."
        for group in self.param_groups:
            lr = group["lr"]
            lr = float(lr) if not isinstance(lr, Tensor) else float(lr.item())
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if len(state) == 0:
                    state["step"] = torch.tensor(0.0, dtype=torch.float32)
                    state["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
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
