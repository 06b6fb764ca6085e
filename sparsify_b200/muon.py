"""Muon (momentum orthogonalised by Newton-Schulz) with the reference's
constructor and update rule (sparsify/muon.py:11-181).

Per matrix: decoupled weight decay, momentum (optionally Nesterov), five quintic
Newton-Schulz iterations in bf16 on the wide orientation, then
p -= lr * 0.2 * sqrt(max(shape)) * update. In data-parallel mode (`ddp=True`
and torch.distributed initialised) rank r orthogonalises matrices r, r+W, ...
and the bf16 updates are exchanged with an asynchronous all-gather while the
next group is being computed; the parameter list must therefore have the same
order in every process (the Trainer passes it sorted by name).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def quintic_newtonschulz(G: Tensor, steps: int) -> Tensor:
    """Approximate orthogonalisation of G: X <- aX + (bA + cA^2)X with A = XX^T,
    starting from G / (||G||_F + 1e-7), in bf16 (sparsify/muon.py:11-40)."""
    assert G.ndim >= 2
    a, b, c = NS_COEFFS
    if G.is_cuda and G.ndim == 2 and G.shape[0] % 8 == 0 and G.shape[1] % 8 == 0:
        return _newtonschulz_tc(G, steps)
    X = G.bfloat16()
    transposed = G.size(-2) > G.size(-1)
    if transposed:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        A = X @ X.mT
        B = torch.addmm(A, A, A, beta=b, alpha=c) if A.ndim == 2 else b * A + c * A @ A
        X = torch.addmm(X, B, X, beta=a) if X.ndim == 2 else a * X + B @ X
    if transposed:
        X = X.mT
    return X


def _newtonschulz_tc(G: Tensor, steps: int) -> Tensor:
    """The same iteration with every product on the tcgen05 GEMM kernel, every
    product written as P Q^T with both operands K-major. The iterate is kept in
    both orientations, wide W = X [r, n] (r <= n) and tall T = X^T [n, r]:

        A  = W W^T                      symmetric: upper tiles computed, rest mirrored
        B  = b A + c A A^T              symmetric (A is)
        T' = a T + T B^T (= T B)        written as T' and, transposed, as W'

    so no transpose pass runs inside the loop, and the result is available in
    the orientation of G without one."""
    from . import ops
    a, b, c = NS_COEFFS
    X = G.bfloat16()
    X = (X / (X.norm() + 1e-7)).contiguous()
    tall_input = G.size(-2) > G.size(-1)
    T = X if tall_input else ops.transpose_bf16(X)
    W = ops.transpose_bf16(X) if tall_input else X
    for _ in range(steps):
        A = ops.gemm_nt(W, W, symmetric=True)
        B = ops.gemm_nt(A, A, alpha=c, beta=b, Cin=A, symmetric=True)
        W_next = torch.empty_like(W)
        T = ops.gemm_nt(T, B, alpha=1.0, beta=a, Cin=T, out_t=W_next)
        W = W_next
    return T if tall_input else W


class Muon(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, momentum: float = 0.95, nesterov: bool = True,
                 weight_decay: float = 0.1, ns_steps: int = 5, ddp: bool = True):
        defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                        weight_decay=weight_decay)
        params = list(params)
        use_dist = dist.is_available() and dist.is_initialized() and ddp
        self.rank = dist.get_rank() if use_dist else 0
        self.world_size = dist.get_world_size() if use_dist else 1

        if use_dist:
            devices = {p.device for p in params}
            assert len(devices) == 1, "Muon does not support model parallelism."
            device = next(iter(devices))
            groups = []
            # one group (and one gather buffer) per distinct matrix size, in first-seen order
            sizes = list(dict.fromkeys(p.numel() for p in params))
            for size in sizes:
                buf = torch.empty(self.world_size, size, dtype=torch.bfloat16, device=device)
                groups.append(dict(
                    params=[p for p in params if p.numel() == size],
                    update_buffer=buf,
                    update_buffer_views=[buf[i] for i in range(self.world_size)],
                ))
            super().__init__(groups, defaults)
        else:
            super().__init__(params, defaults)

    def _orthogonal_update(self, p: Tensor, group: dict) -> Tensor:
        g = p.grad
        assert g is not None
        beta = group["momentum"]
        if beta > 0.0:
            state = self.state[p]
            if "exp_avg" not in state:
                state["exp_avg"] = torch.zeros_like(g)
            buf = state["exp_avg"].lerp_(g, 1 - beta)
            g = g.lerp_(buf, beta) if group["nesterov"] else buf
        if g.ndim == 4:
            g = g.view(len(g), -1)
        return quintic_newtonschulz(g, steps=group["ns_steps"])

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            params: list[Tensor] = group["params"]
            lr = group["lr"]
            if group["weight_decay"] > 0.0:
                for p in params:
                    p.mul_(1 - lr * group["weight_decay"])

            if self.world_size == 1:
                for p in params:
                    upd = self._orthogonal_update(p, group)
                    p.add_(upd.view_as(p), alpha=-lr * 0.2 * max(p.shape) ** 0.5)
                continue

            buffer: Tensor = group["update_buffer"]
            views: list[Tensor] = group["update_buffer_views"]
            inflight = None  # (work handle, parameters the gathered updates belong to)

            def apply(handle, owners):
                handle.wait()
                for p_w, g_w in zip(owners, views):
                    p_w.add_(g_w.view_as(p_w), alpha=-lr * 0.2 * max(p_w.shape) ** 0.5)

            for i in range(0, len(params), self.world_size):
                if i + self.rank < len(params):
                    upd = self._orthogonal_update(params[i + self.rank], group).flatten()
                else:
                    upd = views[self.rank]  # nothing to contribute in a ragged last group
                if inflight is not None:
                    apply(*inflight)  # the previous gather overlapped this group's iterations
                handle = dist.all_gather_into_tensor(buffer.view(-1), upd.contiguous(), async_op=True)
                inflight = (handle, params[i : i + self.world_size])
            if inflight is not None:
                apply(*inflight)
