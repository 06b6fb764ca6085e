"""The Trainer on two GPUs: data parallel (replicas, sharded sparse update) and
`distribute_modules` (each hookpoint owned by one rank that receives every
rank's activations). Skipped with fewer than two GPUs."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.fake_model import FakeModel, dataset

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]

STEPS, B, T, D, M, K = 4, 4, 32, 64, 512, 8


def _acts(seed):
    g = torch.Generator().manual_seed(seed)
    atoms = torch.nn.functional.normalize(torch.randn(256, D, generator=g), dim=1)
    ids = torch.randint(0, 256, (STEPS, B, T, 5), generator=g)
    coef = torch.rand(STEPS, B, T, 5, 1, generator=g)
    return (atoms[ids] * coef).sum(-2) + 0.05 * torch.randn(STEPS, B, T, D, generator=g)


def _cfg(save_dir, hookpoints, **kw):
    from sparsify_b200 import SparseCoderConfig, TrainConfig
    return TrainConfig(SparseCoderConfig(num_latents=M, k=K), batch_size=B, optimizer="adam", lr=5e-3,
                       lr_warmup_steps=1, hookpoints=hookpoints, log_to_wandb=False, save_dir=save_dir,
                       run_name="run", save_every=10 ** 9, **kw)


def _spawn(fn, tmp):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(fn, args=(2, port, str(tmp), out), nprocs=2, join=True)
    return out


def _init(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))


def _ddp_worker(rank, world, port, tmp, out):
    from sparsify_b200 import Trainer
    _init(rank, world, port)
    try:
        model = FakeModel(_acts(10 + rank), device=f"cuda:{rank}")  # each rank sees its own tokens
        tr = Trainer(_cfg(tmp, ["layers.0"]), dataset(STEPS, B, T), model)
        sae = tr.saes["layers.0"]
        assert getattr(sae, "_shard", None) == (rank, world)  # sharded sparse update is active
        tr.fit()
        out[rank] = {n: p.detach().cpu() for n, p in sae.named_parameters()}
        out[f"fvu{rank}"] = [row["fvu/layers.0"] for row in tr.metrics]
    finally:
        dist.destroy_process_group()


def test_data_parallel_trainer(cuda_lib, tmp_path):
    from sparsify_b200 import SparseCoder
    out = _spawn(_ddp_worker, tmp_path)
    for n in out[0]:
        assert torch.equal(out[0][n], out[1][n]), f"replicas differ in {n}"
    assert out["fvu0"] == out["fvu1"] and len(out["fvu0"]) == STEPS  # metrics are averaged over ranks
    assert all(0 < f < 2 for f in out["fvu0"])
    # rank 0 wrote the checkpoint after the shards were gathered: it equals the replicas
    ckpt = SparseCoder.load_from_disk(tmp_path / "run" / "layers.0")
    for n, p in ckpt.named_parameters():
        assert torch.equal(p.detach(), out[1][n]), n


def _dm_worker(rank, world, port, tmp, out):
    from sparsify_b200 import Trainer
    _init(rank, world, port)
    try:
        acts = [_acts(20 + rank), _acts(30 + rank)]  # two hooked layers, this rank's tokens
        model = FakeModel(acts, device=f"cuda:{rank}")
        tr = Trainer(_cfg(tmp, ["layers.0", "layers.1"], distribute_modules=True), dataset(STEPS, B, T), model)
        assert tr.module_plan == [["layers.0"], ["layers.1"]]
        assert list(tr.saes) == [f"layers.{rank}"]
        tr.fit()
        name = f"layers.{rank}"
        out[name] = {n: p.detach().cpu() for n, p in tr.saes[name].named_parameters()}
    finally:
        dist.destroy_process_group()


def test_distribute_modules_matches_single_process(cuda_lib, tmp_path):
    from sparsify_b200 import Trainer
    out = _spawn(_dm_worker, tmp_path / "dist")
    # single process: every hookpoint sees both ranks' tokens, concatenated rank-major
    acts = [torch.cat([_acts(20), _acts(21)], dim=1), torch.cat([_acts(30), _acts(31)], dim=1)]
    model = FakeModel(acts, device="cuda:0")
    cfg = _cfg(str(tmp_path / "single"), ["layers.0", "layers.1"])
    cfg.batch_size = 2 * B
    tr = Trainer(cfg, dataset(STEPS, 2 * B, T), model)
    tr.fit()
    rel = lambda a, b: float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))
    for name in ("layers.0", "layers.1"):
        for n, p in tr.saes[name].named_parameters():
            assert rel(out[name][n], p.detach().cpu()) < 1e-4, (name, n, rel(out[name][n], p.detach().cpu()))
    for r in (0, 1):
        assert (tmp_path / "dist" / "run" / f"rank_{r}_state.pt").exists()
        assert (tmp_path / "dist" / "run" / f"layers.{r}" / "sae.safetensors").exists()
