"""Host-side logic that needs no GPU: configuration round trips, natural sort,
module plan, learning-rate schedule, checkpoint layout of a CPU-resident coder."""

import json
import os

import pytest
import torch

from sparsify_b200 import SparseCoder, SparseCoderConfig, TrainConfig, TranscoderConfig
from sparsify_b200 import parallel
from sparsify_b200.sparse_coder import natsorted


def test_config_roundtrip_and_validation(tmp_path):
    cfg = TrainConfig(SparseCoderConfig(k=64, transcode=True), batch_size=8, hookpoints=["layers.3"])
    d = cfg.to_dict()
    assert d["sae"]["k"] == 64 and d["init_seeds"] == [0]
    back = TrainConfig.from_dict(json.loads(json.dumps(d)))
    assert back == cfg
    cfg.save_json(tmp_path / "config.json")
    assert TrainConfig.load_json(tmp_path / "config.json") == cfg
    assert TranscoderConfig().transcode is True
    assert SparseCoderConfig.from_dict({"k": 5, "unknown": 1}, drop_extra_fields=True).k == 5
    with pytest.raises(ValueError):
        TrainConfig(SparseCoderConfig(), layers=[1], layer_stride=2)
    with pytest.raises(ValueError):
        TrainConfig(SparseCoderConfig(), distribute_modules=True, loss_fn="ce")
    with pytest.raises(ValueError):
        TrainConfig(SparseCoderConfig(), init_seeds=[])


def test_natsorted_and_plan():
    names = ["layers.10", "layers.2", "layers.1", "layers.21"]
    assert natsorted(names) == ["layers.1", "layers.2", "layers.10", "layers.21"]
    plan = parallel.module_plan(natsorted(names), 2)
    assert plan == [["layers.1", "layers.2"], ["layers.10", "layers.21"]]
    assert parallel.owner_of(plan, "layers.10") == 1
    with pytest.raises(AssertionError):
        parallel.module_plan(names, 3)


def test_lr_schedule_matches_transformers():
    from transformers import get_linear_schedule_with_warmup
    from sparsify_b200.trainer import linear_schedule_with_warmup
    p1, p2 = torch.nn.Parameter(torch.zeros(1)), torch.nn.Parameter(torch.zeros(1))
    o1, o2 = torch.optim.SGD([p1], lr=0.3), torch.optim.SGD([p2], lr=0.3)
    s1, s2 = get_linear_schedule_with_warmup(o1, 5, 20), linear_schedule_with_warmup(o2, 5, 20)
    for _ in range(25):
        assert o1.param_groups[0]["lr"] == pytest.approx(o2.param_groups[0]["lr"])
        o1.step(); o2.step(); s1.step(); s2.step()


def test_checkpoint_layout_cpu(tmp_path):
    """Construction, save and load work on the host (no kernels involved); the
    files carry the reference's tensor names and cfg.json fields."""
    from safetensors import safe_open
    torch.manual_seed(0)
    sae = SparseCoder(16, SparseCoderConfig(num_latents=64, k=4), device="cpu")
    norms = sae.W_dec.data.norm(dim=1)
    assert torch.allclose(norms, torch.ones_like(norms), atol=1e-5)
    sae.save_to_disk(tmp_path / "layers.0")
    with safe_open(str(tmp_path / "layers.0" / "sae.safetensors"), framework="pt") as f:
        assert sorted(f.keys()) == ["W_dec", "b_dec", "encoder.bias", "encoder.weight"]
    cfg = json.load(open(tmp_path / "layers.0" / "cfg.json"))
    assert cfg["d_in"] == 16 and cfg["num_latents"] == 64 and cfg["transcode"] is False
    back = SparseCoder.load_many(str(tmp_path), local=True)["layers.0"]
    assert torch.equal(back.encoder.weight, sae.encoder.weight)
    enc_only = SparseCoder.load_from_disk(tmp_path / "layers.0", decoder=False)
    assert enc_only.W_dec is None


def test_compute_on_cpu_fails_loudly():
    sae = SparseCoder(16, SparseCoderConfig(num_latents=64, k=4), device="cpu")
    with pytest.raises(RuntimeError, match="no CPU path"):
        sae(torch.randn(4, 16))


def test_trainer_construction_k_decay_and_lr_on_host(tmp_path):
    """The Trainer builds its sparse coders, plan, learning rates and k schedule on
    the host (trainer.py:63-145,176-177,229-235); only fit() needs the GPU."""
    from sparsify_b200 import TrainConfig, Trainer
    from tests.fake_model import FakeModel, dataset
    acts = [torch.zeros(2, 2, 8, 16), torch.zeros(2, 2, 8, 16)]
    cfg = TrainConfig(SparseCoderConfig(num_latents=64, k=4), batch_size=2, hookpoints=["layers.1", "layers.0"],
                      k_decay_steps=10, log_to_wandb=False, save_dir=str(tmp_path), run_name="r")
    tr = Trainer(cfg, dataset(2, 2, 8), FakeModel(acts))
    assert list(tr.saes) == ["layers.0", "layers.1"]  # natural order
    assert tr.initial_k == min(64, 16 * 10) and tr.final_k == 4
    ks = []
    for step in (0, 5, 10, 50):
        tr.global_step = step
        ks.append(tr.get_current_k())
    assert ks == [64, round(64 * 0.5 + 4 * 0.5), 4, 4]
    # the default optimiser is "signum": lr rule of trainer.py:152, no scheduler, training mode
    assert tr.lr_schedulers == [] and len(tr.optimizers) == 1
    for g in tr.optimizers[0].param_groups:
        assert abs(g["lr"] - 5e-3 / (64 / 2 ** 14) ** 0.5) < 1e-12 and g["momentum"] == 0.95 and g["train_mode"]
    cfg2 = TrainConfig(SparseCoderConfig(num_latents=64, k=4), batch_size=2, hookpoints=["layers.0"],
                       optimizer="adam", log_to_wandb=False, save_dir=str(tmp_path), run_name="r")
    tr2 = Trainer(cfg2, dataset(2, 2, 8), FakeModel(acts))
    for g in tr2.optimizers[0].param_groups:  # trainer.py:109, scheduler starts at lr 0
        assert abs(g["initial_lr"] - 2e-4 / (64 / 2 ** 14) ** 0.5) < 1e-12 and g["lr"] == 0.0
    with pytest.raises(ValueError):
        Trainer(TrainConfig(SparseCoderConfig(num_latents=64, k=4), batch_size=2, hookpoints=["layers.0"],
                            optimizer="sgd", log_to_wandb=False), dataset(2, 2, 8), FakeModel(acts))


def test_load_many_layers_and_pattern(tmp_path):
    torch.manual_seed(0)
    for name in ("layers.0", "layers.2", "layers.10", "other.1"):
        SparseCoder(8, SparseCoderConfig(num_latents=16, k=2), device="cpu").save_to_disk(tmp_path / name)
    all_ = SparseCoder.load_many(str(tmp_path), local=True)
    assert list(all_) == ["layers.0", "layers.2", "layers.10", "other.1"]
    some = SparseCoder.load_many(str(tmp_path), local=True, layers=["layers.10", "layers.2"])
    assert list(some) == ["layers.2", "layers.10"]
    # as in the reference (sparse_coder.py:87,99-103) the pattern gets "/*" appended for the hub
    # download and is then matched against bare directory names, so locally it selects nothing
    assert SparseCoder.load_many(str(tmp_path), local=True, pattern="layers.1*") == {}
    with pytest.raises(NotImplementedError):
        SparseCoder.load_many("someone/some-repo")


def test_schedulefree_signum_modes_and_state_on_host():
    """train()/eval() convert between the gradient point y and the average x through z and
    invert each other; stepping outside training mode is refused; the state dict carries z
    and the schedule-free counters (host-side logic of sparsify/trainer.py:158-159,652-677)."""
    from sparsify_b200.optim import ScheduleFreeSignum
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(5, 4))
    opt = ScheduleFreeSignum([p], lr=1e-2, momentum=0.95)
    with pytest.raises(RuntimeError, match="train"):
        p.grad = torch.zeros_like(p)
        opt.step()
    opt.train()
    y = p.detach().clone()
    z = torch.randn(5, 4)
    opt.state[p]["z"] = z.clone()
    opt.eval()
    x = p.detach().clone()
    assert torch.allclose(x, torch.lerp(y, z, 1 - 1 / 0.95), atol=1e-6)
    opt.train()
    assert torch.allclose(p.detach(), y, atol=1e-5)
    sd = opt.state_dict()
    assert sd["param_groups"][0]["train_mode"] is True and sd["param_groups"][0]["k"] == 0
    opt2 = ScheduleFreeSignum([torch.nn.Parameter(torch.zeros(5, 4))], lr=1.0)
    opt2.load_state_dict(sd)
    assert opt2.param_groups[0]["momentum"] == 0.95 and opt2.param_groups[0]["lr"] == 1e-2
    assert torch.equal(next(iter(opt2.state.values()))["z"], z)


def test_prepared_dead_mask_is_used_by_identity():
    """A mask prepared ahead of time answers count and indices from the cache - for that
    tensor object only; any other mask is counted afresh."""
    sae = SparseCoder(16, SparseCoderConfig(num_latents=64, k=4), device="cpu")
    mask = torch.zeros(64, dtype=torch.bool)
    mask[[3, 10, 40]] = True
    assert sae.prepare_dead_mask(mask) is mask
    assert sae._count_dead(mask) == 3 and sae.dead_indices(mask).tolist() == [3, 10, 40]
    other = mask.clone()
    other[5] = True
    assert sae._count_dead(other) == 4 and sae.dead_indices(other).tolist() == [3, 5, 10, 40]
    assert sae._count_dead(None) == 0
    sae.prepare_dead_mask(None)
    assert sae._count_dead(mask) == 3


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` (the CPU arm: the vendored reference's own Trainer.fit() on
    the host cores, or the oracle port where the reference is absent) prints one JSON line
    with the metric, the workload and the cpu_baseline / e2e objects, on every host thread even
    under a launcher that exports OMP_NUM_THREADS=1; a rank other than 0 of a multi-process
    launch exits without work."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cmd = [sys.executable, str(root / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
           "--d", "64", "--latents", "512", "--k", "4", "--cpu-tokens", "64", "--atoms", "1024", "--active", "8",
           "--config0-steps", "0"]
    env1 = dict(os.environ, OMP_NUM_THREADS="1")  # what torch.distributed.run exports to its workers
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=root, env=env1)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "sae_train_tokens_per_s"
    assert line["unit"] == "tokens/s" and line["higher_is_better"] is True and line["value"] > 0
    from oracle import ref_loader
    assert line["cpu_baseline"]["kind"] == ("reference" if ref_loader.find_reference() is not None else "port")
    assert line["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"]
    assert "workload" in line["config"]
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run(cmd + ["--gpus", "2"], capture_output=True, text=True, timeout=300, cwd=root, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_sparse_update_is_refused_where_dead_sets_can_diverge():
    """Data parallel + excluded tokens + AuxK: each rank's dead-latent counters advance by its own
    unmasked token count, so the dead sets (the shape of a collective in the sharded update) may
    differ between ranks; that combination must keep the dense, fixed-shape gradient exchange."""
    from sparsify_b200.trainer import sparse_update_allowed
    mk = lambda **kw: TrainConfig(SparseCoderConfig(num_latents=64, k=4), **kw)
    assert sparse_update_allowed(mk(), 1) and sparse_update_allowed(mk(), 8)
    assert sparse_update_allowed(mk(exclude_tokens=[0], auxk_alpha=1 / 32), 1)
    assert sparse_update_allowed(mk(exclude_tokens=[0], auxk_alpha=0.0), 8)
    assert not sparse_update_allowed(mk(exclude_tokens=[0], auxk_alpha=1 / 32), 8)
    assert sparse_update_allowed(mk(exclude_tokens=[0], auxk_alpha=1 / 32, distribute_modules=True), 8)
    assert not sparse_update_allowed(mk(grad_acc_steps=2), 1)
    assert not sparse_update_allowed(mk(loss_fn="ce"), 1)


def test_no_assignment_through_an_index_tensor_on_the_step_path():
    """`t[index_tensor] = value` on a CUDA tensor makes the host wait for everything queued before
    it (measured: the whole training step); `index_fill_` / `index_copy_` do not. The step path -
    the package and the benchmark's step - must not reintroduce such an assignment."""
    import pathlib
    import re
    root = pathlib.Path(__file__).resolve().parent.parent
    pat = re.compile(r"\[[^\[\]\"']*\b\w*(?:idx|indices)\b[^\[\]\"']*\]\s*=(?!=)")
    hits = []
    for f in sorted((root / "sparsify_b200").glob("*.py")) + [root / "bench.py"]:
        for no, line in enumerate(f.read_text().splitlines(), 1):
            if pat.search(line.split("#")[0]):
                hits.append(f"{f.name}:{no}: {line.strip()}")
    assert not hits, hits
