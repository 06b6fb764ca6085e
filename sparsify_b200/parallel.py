"""Multi-process plumbing of the Trainer over torch.distributed (NCCL on GPUs,
gloo in CPU tests). Device-agnostic: nothing here launches a kernel of its own.

* data parallel: every rank holds a replica and its own tokens; gradients are
  averaged across ranks (what DistributedDataParallel does for the reference,
  sparsify/trainer.py:457-468). `GradReducer` starts an asynchronous all-reduce
  for each parameter as soon as autograd has accumulated its gradient, so the
  decoder's reduction overlaps the encoder's backward.
* hookpoint sharding (`distribute_modules`, sparsify/trainer.py:630-646): each
  hookpoint is owned by one rank, which receives every rank's activations. The
  reference all-gathers to everyone and lets non-owners drop the data; here
  only the owner receives (gather), an 8x cut of received bytes on 8 ranks,
  with the same concatenation order (rank-major).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor


def is_dist() -> bool:
    return dist.is_available() and dist.is_initialized()


def module_plan(hookpoints: list[str], world_size: int) -> list[list[str]]:
    """Equal contiguous slices of the hookpoint list, one per rank."""
    per_rank, rem = divmod(len(hookpoints), world_size)
    assert rem == 0, "Number of modules must be divisible by world size"
    return [hookpoints[s : s + per_rank] for s in range(0, len(hookpoints), per_rank)]


def owner_of(plan: list[list[str]], name: str) -> int:
    for rank, names in enumerate(plan):
        if name in names:
            return rank
    raise KeyError(name)


def gather_to_owner(t: Tensor, owner: int, group=None, stream=None, after=None) -> Tensor | None:
    """Concatenates `t` from all ranks along dim 0 on rank `owner` (rank-major,
    the layout of all_gather_into_tensor); other ranks get None.

    stream: a CUDA stream to run the exchange on. The calling stream then does
    not wait for the collective unless this rank is the owner, so a rank that
    only contributes its slice is not held back by the owner's queued work, and
    the owners of different hookpoints compute side by side. after: the event
    that marks `t` as complete (default: everything queued on the calling stream)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    t = t.contiguous()
    if stream is None or not t.is_cuda:
        if rank == owner:
            out = t.new_empty(world * t.shape[0], *t.shape[1:])
            parts = list(out.chunk(world, dim=0))
            dist.gather(t, parts, dst=owner, group=group)
            return out
        dist.gather(t, None, dst=owner, group=group)
        return None
    cur = torch.cuda.current_stream(t.device)
    if after is not None:
        stream.wait_event(after)
    else:
        stream.wait_stream(cur)  # the slice is complete
    out = None
    with torch.cuda.stream(stream):
        if rank == owner:
            out = t.new_empty(world * t.shape[0], *t.shape[1:])
            dist.gather(t, list(out.chunk(world, dim=0)), dst=owner, group=group)
        else:
            dist.gather(t, None, dst=owner, group=group)
    t.record_stream(stream)
    if out is not None:
        cur.wait_stream(stream)
        out.record_stream(cur)
    return out


def all_reduce_(x: Tensor, op: str = "mean", group=None) -> Tensor:
    """In-place all-reduce with the reference's op names (trainer.py:614-628)."""
    if not is_dist():
        return x
    if op == "sum":
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
    elif op == "mean":
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
        x /= dist.get_world_size(group)
    elif op == "max":
        if x.dtype == torch.bool:
            y = x.to(torch.uint8)
            dist.all_reduce(y, op=dist.ReduceOp.MAX, group=group)
            x.copy_(y.bool())
        else:
            dist.all_reduce(x, op=dist.ReduceOp.MAX, group=group)
    else:
        raise ValueError(f"Unknown reduction op '{op}'")
    return x


def broadcast_params(params, src: int = 0, group=None) -> None:
    """Replicas start identical (DDP's initial broadcast)."""
    for p in params:
        dist.broadcast(p.data, src=src, group=group)


class GradReducer:
    """Averages gradients across ranks, overlapped with the backward pass.

    attach() registers a post-accumulate hook on every parameter; the hook
    issues an asynchronous SUM all-reduce of that parameter's gradient.
    finish() waits for all of them and divides by the world size. With
    gradient accumulation the caller enables the reducer only for the last
    micro-step: the mean over ranks of the accumulated gradient equals the
    accumulated per-micro-step means that DDP produces for the reference, at
    one exchange per optimiser step instead of one per micro-step."""

    def __init__(self, params, group=None):
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        self.pending: list[tuple] = []
        self.handles = []
        self.enabled = True

    def attach(self) -> "GradReducer":
        for p in self.params:
            self.handles.append(p.register_post_accumulate_grad_hook(self._hook))
        return self

    def detach(self) -> None:
        for h in self.handles:
            h.remove()
        self.handles = []

    def _hook(self, p: Tensor) -> None:
        if not self.enabled or p.grad is None:
            return
        work = dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self.pending.append((work, p))

    def finish(self) -> None:
        world = dist.get_world_size(self.group)
        for work, p in self.pending:
            work.wait()
            p.grad /= world
        self.pending = []
