"""World-size-2 tests of the multi-process plumbing on CPU (gloo): gather to the
owning rank, gradient averaging overlapped with backward, boolean MAX reduce,
and Muon's one-matrix-per-rank mode against the single-process optimiser."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sae_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def run(fn, world=2):
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), fn, out), nprocs=world, join=True)
    return [out[r] for r in range(world)]


def _gather_case(rank, world):
    from sparsify_b200 import parallel
    t = torch.full((2, 3), float(rank))
    got = [parallel.gather_to_owner(t, owner) for owner in range(world)]
    flags = torch.tensor([rank == 0, False, rank == 1])
    parallel.all_reduce_(flags, "max")
    mean = parallel.all_reduce_(torch.tensor([float(rank)]), "mean")
    return [None if g is None else g.tolist() for g in got], flags.tolist(), mean.item()


def test_gather_to_owner_and_reductions():
    res = run(_gather_case)
    full = [[0.0] * 3] * 2 + [[1.0] * 3] * 2
    assert res[0][0] == [full, None] and res[1][0] == [None, full]
    assert res[0][1] == res[1][1] == [True, False, True]
    assert res[0][2] == res[1][2] == 0.5


def _reducer_case(rank, world):
    from sparsify_b200 import parallel
    torch.manual_seed(0)
    lin = torch.nn.Linear(4, 3)
    parallel.broadcast_params(lin.parameters())
    red = parallel.GradReducer(lin.parameters()).attach()
    x = torch.arange(8.0).reshape(2, 4) + rank
    red.enabled = False           # first micro-step accumulates locally
    lin(x).sum().backward()
    red.enabled = True            # last micro-step triggers the exchange
    lin(2 * x).sum().backward()
    red.finish()
    red.detach()
    return lin.weight.grad.tolist()


def test_grad_reducer_matches_mean_of_accumulated_grads():
    res = run(_reducer_case)
    assert res[0] == res[1]
    expect = sum(3 * (torch.arange(8.0).reshape(2, 4) + r).sum(0) for r in range(2)) / 2
    assert torch.allclose(torch.tensor(res[0]), expect.expand(3, 4))


def _muon_case(rank, world):
    from sparsify_b200.muon import Muon
    torch.manual_seed(1)
    params = [torch.nn.Parameter(torch.randn(8, 16)) for _ in range(3)]  # ragged last group
    for i, p in enumerate(params):
        p.grad = torch.randn(8, 16, generator=torch.Generator().manual_seed(10 + i))
    opt = Muon(params, lr=0.01, ddp=True, orthogonalize=O.quintic_newtonschulz)
    assert opt.world_size == world
    opt.step()
    return [p.detach().clone() for p in params]


def test_muon_ddp_equals_single_process():
    from sparsify_b200.muon import Muon
    res = run(_muon_case)
    torch.manual_seed(1)
    params = [torch.nn.Parameter(torch.randn(8, 16)) for _ in range(3)]
    for i, p in enumerate(params):
        p.grad = torch.randn(8, 16, generator=torch.Generator().manual_seed(10 + i))
    Muon(params, lr=0.01, ddp=False, orthogonalize=O.quintic_newtonschulz).step()
    for r in range(2):
        for got, want in zip(res[r], params):
            assert torch.allclose(got, want.detach(), atol=1e-6)
