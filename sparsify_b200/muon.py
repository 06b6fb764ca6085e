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
    starting from G / (||G||_F + 1e-7), in bf16 (sparsify/muon.py:11-40). CUDA
    matrices whose sides are multiples of 8 only: every product runs on the
    tcgen05 GEMM kernel and there is no other path."""
    if G.ndim == 4:  # conv filters, as the reference flattens them
        G = G.view(len(G), -1)
    if not (G.is_cuda and G.ndim == 2):
        raise RuntimeError("quintic_newtonschulz: no CPU path; pass a 2-D CUDA tensor")
    if G.shape[0] % 8 or G.shape[1] % 8:
        raise ValueError(f"quintic_newtonschulz: sides must be multiples of 8, got {tuple(G.shape)}")
    return _newtonschulz_tc(G, steps)


def _newtonschulz_tc(G: Tensor, steps: int, Xb: Tensor | None = None, sumsq: Tensor | None = None) -> Tensor:
    """The same iteration with every product on the tcgen05 GEMM kernel, every
    product written as P Q^T with both operands K-major. The iterate is kept in
    both orientations, wide W = X [r, n] (r <= n) and tall T = X^T [n, r]:

        A  = W W^T                      symmetric: upper tiles computed, rest mirrored
        B  = b A + c A A^T              symmetric (A is)
        T' = a T + T B^T (= T B)        written as T' and, transposed, as W'

    so no transpose pass runs inside the loop, and the result is available in
    the orientation of G without one. Xb / sumsq: the bf16 cast of G and the sum
    of its squares when the caller already has them (the fused momentum pass)."""
    from . import ops
    a, b, c = NS_COEFFS
    if Xb is None:
        Xb = G.bfloat16().contiguous()
        sumsq = torch.linalg.vector_norm(Xb, dtype=torch.float32).square().reshape(1)
    tall_input = Xb.size(-2) > Xb.size(-1)
    # normalisation fused with the one transpose that sets up the two orientations
    if tall_input:
        T, W = ops.scale_transpose_bf16(Xb, sumsq)
    else:
        W, T = ops.scale_transpose_bf16(Xb, sumsq)
    for _ in range(steps):
        A = ops.gemm_nt(W, W, symmetric=True)
        B = ops.gemm_nt(A, A, alpha=c, beta=b, Cin=A, symmetric=True)
        W_next = torch.empty_like(W)
        T = ops.gemm_nt(T, B, alpha=1.0, beta=a, Cin=T, out_t=W_next)
        W = W_next
    return T if tall_input else W


class Muon(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, momentum: float = 0.95, nesterov: bool = True,
                 weight_decay: float = 0.1, ns_steps: int = 5, ddp: bool = True, orthogonalize=None):
        defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                        weight_decay=weight_decay)
        params = list(params)
        self._shadow: dict[int, tuple] = {}
        # `orthogonalize(G, steps)`: replaces the tensor-core Newton-Schulz (tests of the
        # host-side exchange logic on CPU processes inject a CPU implementation here)
        self._orthogonalize = orthogonalize
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

    def register_shadow(self, p: Tensor, shadow: Tensor, on_refresh=None) -> None:
        """`shadow` (bf16, same shape) is rewritten with the updated value of `p`
        inside the update kernel; `on_refresh()` is called afterwards."""
        self._shadow[id(p)] = (shadow, on_refresh)

    def project_rows(self, p: Tensor) -> None:  # the Trainer projects Muon's gradients itself
        raise NotImplementedError("Muon does not project gradients; call "
                                  "remove_gradient_parallel_to_decoder_directions() before step()")

    def _fast(self, p: Tensor, g: Tensor) -> bool:
        return (g.is_cuda and g.ndim == 2 and g.dtype == torch.float32 and g.is_contiguous()
                and p.dtype == torch.float32 and p.is_contiguous()
                and g.shape[0] % 8 == 0 and g.shape[1] % 8 == 0)

    def _orthogonal_update(self, p: Tensor, group: dict) -> Tensor:
        g = p.grad
        assert g is not None
        beta = group["momentum"]
        if beta > 0.0 and self._orthogonalize is None and self._fast(p, g):
            # momentum, Nesterov, bf16 cast and the Frobenius norm in one pass
            from . import ops
            state = self.state[p]
            if "exp_avg" not in state:
                state["exp_avg"] = torch.zeros_like(g)
            xb, sumsq = ops.muon_momentum_(g, state["exp_avg"], beta, group["nesterov"])
            return _newtonschulz_tc(g, group["ns_steps"], xb, sumsq)
        if beta > 0.0:
            state = self.state[p]
            if "exp_avg" not in state:
                state["exp_avg"] = torch.zeros_like(g)
            buf = state["exp_avg"].lerp_(g, 1 - beta)
            g = g.lerp_(buf, beta) if group["nesterov"] else buf
        return (self._orthogonalize or quintic_newtonschulz)(g, group["ns_steps"])

    def _apply(self, p: Tensor, upd: Tensor, lr: float, decay: float) -> None:
        """p = p * decay - lr * 0.2 sqrt(max(shape)) * upd (muon.py:120-123,139-141)."""
        alpha = lr * 0.2 * max(p.shape) ** 0.5
        upd = upd.view_as(p)
        if self._fast(p, p.data) and upd.dtype == torch.bfloat16 and upd.is_contiguous():
            from . import ops
            shadow, cb = self._shadow.get(id(p), (None, None))
            ops.muon_apply_(p.data, upd, decay, alpha, shadow)
            torch.autograd.graph.increment_version(p)  # written through raw pointers
            if cb is not None:
                cb()
        elif self._orthogonalize is not None:
            # injected orthogonaliser (CPU processes testing the exchange logic): plain tensor ops
            if decay != 1.0:
                p.mul_(decay)
            p.add_(upd, alpha=-alpha)
        else:
            raise RuntimeError("Muon: contiguous fp32 CUDA matrices with sides that are multiples of 8 "
                               "only (no CPU path)")

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            params: list[Tensor] = group["params"]
            lr = group["lr"]
            # decoupled weight decay, folded into the pass that applies the update
            decay = 1 - lr * group["weight_decay"] if group["weight_decay"] > 0.0 else 1.0

            if self.world_size == 1:
                for p in params:
                    self._apply(p, self._orthogonal_update(p, group), lr, decay)
                continue

            buffer: Tensor = group["update_buffer"]
            views: list[Tensor] = group["update_buffer_views"]
            inflight = None  # (work handle, parameters the gathered updates belong to)

            def apply(handle, owners):
                handle.wait()
                for p_w, g_w in zip(owners, views):
                    self._apply(p_w, g_w, lr, decay)

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
