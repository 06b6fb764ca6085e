"""Two-GPU data parallel: the sharded sparse update (factor exchange, per-rank
latent slices, all-gather of the bf16 copies) must reproduce a single process
that sees both ranks' tokens with the per-rank FVU losses averaged. Skipped on
machines with fewer than two GPUs."""

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

N, D, M, K, STEPS = 512, 256, 2048, 16, 3


def _data(rank, step):
    g = torch.Generator().manual_seed(100 + 10 * step + rank)
    return torch.randn(N, D, generator=g)


def _build(device, multi_topk=False):
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    from sparsify_b200.optim import FusedAdam
    torch.manual_seed(0)
    sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=K, multi_topk=multi_topk), device=device,
                      dtype=torch.float32)
    opt = FusedAdam(sae.parameters(), lr=1e-3)
    sae.attach_optimizer(opt)
    return sae, opt


def _dead_mask():
    g = torch.Generator().manual_seed(5)
    m = torch.zeros(M, dtype=torch.bool)
    m[torch.randperm(M, generator=g)[:96]] = True
    return m


def _loss(o):
    return o.fvu + o.auxk_loss / 32 + o.multi_topk_fvu / 8


def _worker(rank, world, port, out, mode):
    auxk, multi = mode == "auxk", mode == "multi_topk"
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        sae, opt = _build(f"cuda:{rank}", multi)
        assert opt.enable_sparse_update(sae) and sae._shard == (rank, world)
        for step in range(STEPS):
            sae.set_decoder_norm_to_unit_norm()
            out_ = sae(_data(rank, step).cuda(), dead_mask=_dead_mask().cuda() if auxk else None)
            _loss(out_).backward()
            assert sae.W_dec.grad is None and sae._pending is not None  # the sparse, sharded route
            for p in sae.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad)
                    p.grad /= world
            opt.step()
            opt.zero_grad(set_to_none=True)
        opt.sync_masters()
        out[rank] = {n: p.detach().cpu() for n, p in sae.named_parameters()}
        out[f"shadow{rank}"] = sae.shadow("W_dec").cpu()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["plain", "auxk", "multi_topk"])
def test_sharded_sparse_update_matches_single_process(cuda_lib, mode):
    auxk, multi = mode == "auxk", mode == "multi_topk"
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, port, out, mode), nprocs=2, join=True)

    # single process: both ranks' batches per step, losses averaged (DDP's mean of gradients)
    sae, opt = _build("cuda:0", multi)
    for step in range(STEPS):
        sae.set_decoder_norm_to_unit_norm()
        dead = _dead_mask().cuda() if auxk else None
        outs = [sae(_data(r, step).cuda(), dead_mask=dead) for r in range(2)]
        loss = sum(_loss(o) for o in outs) / 2
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
    sae.set_decoder_norm_to_unit_norm()
    ref = {n: p.detach().cpu() for n, p in sae.named_parameters()}
    rel = lambda a, b: float((a.double() - b.double()).norm() / b.double().norm())
    for n in ref:
        assert torch.equal(out[0][n], out[1][n]), f"replicas differ in {n}"
        assert rel(out[0][n], ref[n]) < 2e-3, (n, rel(out[0][n], ref[n]))
    assert torch.equal(out["shadow0"], out["shadow1"])
