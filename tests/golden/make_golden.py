"""Generates tests/golden/*.safetensors by running the REFERENCE implementation
(EleutherAI/sparsify v1.3.0, unmodified, imported from its source tree) on CPU
with seeded inputs. Run once where the reference tree is available:

    SPARSIFY_REF=/path/to/sparsify python tests/golden/make_golden.py

The reference's non-arithmetic dependencies that are not installed here
(natsort, simple_parsing, accelerate) are replaced by small stand-in modules
(oracle/ref_loader.py) that take no part in the arithmetic that is frozen;
schedulefree's wrapper class, which only the optimizer="signum" fixture uses, is
replaced by the oracle's restatement of its published algorithm. The fixtures
are what the oracle (oracle/sae_oracle.py) is pinned against.
"""

from __future__ import annotations

import dataclasses
import json
import os
import re
import sys
import tempfile
import types
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent


def import_reference():
    """The unmodified reference, imported through oracle/ref_loader.py (which documents the
    stand-ins for its four absent non-arithmetic dependencies). schedulefree's wrapper, which
    only the optimizer="signum" fixture uses, is the oracle's restatement of the published
    algorithm: that fixture pins SignSGD, the learning-rate rule and the Trainer's glue, not
    the wrapper itself."""
    sys.path.insert(0, str(HERE.parent.parent))
    from oracle import ref_loader
    from oracle.sae_oracle import ScheduleFreeWrapperPort
    if ref_loader.find_reference() is None:
        raise SystemExit("set SPARSIFY_REF to a checkout of EleutherAI/sparsify v1.3.0 (or run oracle/make_ref.py)")
    return ref_loader.import_reference(schedulefree_wrapper=ScheduleFreeWrapperPort)


def save(name: str, tensors: dict, meta: dict | None = None):
    from safetensors.torch import save_file
    tensors = {k: v.detach().contiguous().clone() for k, v in tensors.items()}
    save_file(tensors, str(HERE / f"{name}.safetensors"),
              metadata={k: json.dumps(v) for k, v in (meta or {}).items()})
    print(f"wrote {name}.safetensors: {sorted(tensors)}")


def sorted_topk(vals, idx):
    """Canonical order (descending value) so unsorted top-k results compare."""
    order = torch.argsort(vals, dim=-1, descending=True, stable=True)
    return vals.gather(-1, order), idx.gather(-1, order)


def gen_encoder(sparsify):
    from sparsify.fused_encoder import fused_encoder
    for tag, act, (N, D, M, k) in [("topk", "topk", (48, 40, 256, 8)), ("groupmax", "groupmax", (24, 32, 128, 8))]:
        g = torch.Generator().manual_seed(42)
        x = torch.randn(N, D, generator=g, requires_grad=True)
        W = torch.randn(M, D, generator=g, requires_grad=True)
        b = torch.randn(M, generator=g, requires_grad=True)
        coef = torch.randn(N, k, generator=g)
        vals, idx, pre = fused_encoder(x, W, b, k, act)
        # coefficients follow the canonical order so the gradient is order-free
        svals, sidx = sorted_topk(vals, idx)
        order = torch.argsort(vals, dim=-1, descending=True, stable=True)
        loss = (vals.gather(-1, order) * coef).sum()
        loss.backward()
        save(f"encoder_{tag}", dict(x=x, W=W, b=b, coef=coef, vals=svals, idx=sidx, pre=pre,
                                    gx=x.grad, gW=W.grad, gb=b.grad), dict(k=k, activation=act))


def gen_decoder(sparsify):
    from sparsify.utils import eager_decode
    for d_in in (48, 64):
        g = torch.Generator().manual_seed(7 + d_in)
        batch, d_sae, k = 2, 128, 10
        latents = torch.rand(batch, d_sae, generator=g)
        W_dec = torch.randn(d_sae, d_in, generator=g, requires_grad=True)
        vals, idx = latents.topk(k)
        vals = vals.clone().requires_grad_(True)
        out = eager_decode(idx, vals, W_dec.mT)
        gout = torch.randn(batch, d_in, generator=g)
        (out * gout).sum().backward()
        save(f"decoder_d{d_in}", dict(idx=idx, acts=vals, W_dec=W_dec, out=out, gout=gout,
                                      gW=W_dec.grad, gacts=vals.grad), dict(k=k))


def gen_forward(sparsify):
    from sparsify import SparseCoder, SparseCoderConfig
    cases = {
        "sae_plain": dict(cfg=dict(k=4), dead=False),
        "sae_auxk": dict(cfg=dict(k=4), dead=True),
        "sae_multitopk": dict(cfg=dict(k=4, multi_topk=True), dead=True),
        "transcoder_skip": dict(cfg=dict(k=4, transcode=True, skip_connection=True), dead=False),
    }
    N, D, M = 80, 32, 256
    alpha = 1 / 32
    for name, case in cases.items():
        torch.manual_seed(0)
        cfg = SparseCoderConfig(num_latents=M, **case["cfg"])
        sae = SparseCoder(D, cfg, dtype=torch.float32)
        g = torch.Generator().manual_seed(11)
        with torch.no_grad():
            sae.encoder.bias.copy_(0.1 * torch.randn(M, generator=g))
            sae.b_dec.copy_(0.1 * torch.randn(D, generator=g))
            if cfg.transcode:
                sae.W_dec.copy_(0.2 * torch.randn(M, D, generator=g))
                sae.W_skip.copy_(0.1 * torch.randn(D, D, generator=g))
        x = torch.randn(N, D, generator=g)
        y = torch.randn(N, D, generator=g) if cfg.transcode else None
        dead_mask = None
        if case["dead"]:
            dead_mask = torch.zeros(M, dtype=torch.bool)
            dead_mask[torch.randperm(M, generator=g)[:40]] = True
        params = dict(W_enc=sae.encoder.weight, b_enc=sae.encoder.bias, W_dec=sae.W_dec, b_dec=sae.b_dec)
        if sae.W_skip is not None:
            params["W_skip"] = sae.W_skip
        init = {k: v.detach().clone() for k, v in params.items()}
        out = sae(x, y, dead_mask=dead_mask)
        loss = out.fvu + alpha * out.auxk_loss + out.multi_topk_fvu / 8
        loss.backward()
        acts, idx = sorted_topk(out.latent_acts, out.latent_indices)
        t = dict(x=x, sae_out=out.sae_out, latent_acts=acts, latent_indices=idx, fvu=out.fvu,
                 auxk_loss=out.auxk_loss, multi_topk_fvu=out.multi_topk_fvu)
        if y is not None:
            t["y"] = y
        if dead_mask is not None:
            t["dead_mask"] = dead_mask
        for k_, v in init.items():
            t[f"param.{k_}"] = v
        for k_, v in params.items():
            t[f"grad.{k_}"] = v.grad if v.grad is not None else torch.zeros_like(v)
        save(f"forward_{name}", t, dict(cfg=dataclasses.asdict(cfg), auxk_alpha=alpha))


class FakeLayer(torch.nn.Module):
    def __init__(self, owner):
        super().__init__()
        object.__setattr__(self, "_owner", owner)

    def forward(self, h):
        return self._owner.next_activation()


class FakeModel(torch.nn.Module):
    """Stands in for the language model: one hooked layer whose output is the
    next batch of stored activations."""

    def __init__(self, acts):
        super().__init__()
        self.config = types.SimpleNamespace(num_hidden_layers=1)
        self.layers = torch.nn.ModuleList([FakeLayer(self)])
        self.acts = acts  # [steps, B, T, D]
        self.cursor = -1  # the width probe consumes one call
        self.dummy_inputs = {"input_ids": torch.zeros(1, acts.shape[2], dtype=torch.long)}

    @property
    def base_model(self):
        return self

    @property
    def device(self):
        return torch.device("cpu")

    def next_activation(self):
        i = max(self.cursor, 0)
        self.cursor += 1
        return self.acts[min(i, self.acts.shape[0] - 1)]

    def forward(self, input_ids=None, **kw):
        return self.layers[0](input_ids)


def gen_trainer(sparsify):
    """A few optimiser steps of the reference Trainer (Adam, FVU + AuxK, decoder
    normalisation) on stored activations; freezes the per-step FVU and the final
    parameters."""
    from sparsify import SparseCoderConfig, TrainConfig, Trainer
    steps, B, T, D, M, k = 6, 4, 16, 32, 256, 4
    g = torch.Generator().manual_seed(5)
    atoms = torch.nn.functional.normalize(torch.randn(512, D, generator=g), dim=1)
    ids = torch.randint(0, 512, (steps, B, T, 6), generator=g)
    coef = -torch.log1p(-torch.rand(steps, B, T, 6, generator=g))
    acts = (atoms[ids] * coef.unsqueeze(-1)).sum(-2) + 0.05 * torch.randn(steps, B, T, D, generator=g)
    model = FakeModel(acts)
    dataset = [{"input_ids": torch.zeros(T, dtype=torch.long)} for _ in range(steps * B)]
    fvus = []
    with tempfile.TemporaryDirectory() as tmp:
        cfg = TrainConfig(
            SparseCoderConfig(num_latents=M, k=k), batch_size=B, optimizer="adam", lr=1e-2,
            lr_warmup_steps=2, auxk_alpha=1 / 32, dead_feature_threshold=100, hookpoints=["layers.0"],
            log_to_wandb=False, save_dir=tmp, run_name="golden", save_every=10**9,
        )
        trainer = Trainer(cfg, dataset, model)
        sae = trainer.saes["layers.0"]
        init = dict(W_enc=sae.encoder.weight.detach().clone(), b_enc=sae.encoder.bias.detach().clone(),
                    W_dec=sae.W_dec.detach().clone(), b_dec=sae.b_dec.detach().clone())
        orig_forward = sae.forward

        def recording_forward(*a, **kw):
            out = orig_forward(*a, **kw)
            fvus.append(out.fvu.detach().clone())
            return out

        sae.forward = recording_forward
        trainer.fit()
        final = dict(W_enc=sae.encoder.weight, b_enc=sae.encoder.bias, W_dec=sae.W_dec, b_dec=sae.b_dec)
        t = dict(acts=acts, fvu=torch.stack(fvus),
                 num_tokens_since_fired=trainer.num_tokens_since_fired["layers.0"])
        for k_, v in init.items():
            t[f"init.{k_}"] = v
        for k_, v in final.items():
            t[f"final.{k_}"] = v
        save("trainer_adam", t, dict(steps=steps, B=B, T=T, D=D, M=M, k=k, lr=1e-2, warmup=2,
                                     auxk_alpha=1 / 32, dead_feature_threshold=100))


def gen_trainer_muon(sparsify):
    """The reference Trainer with optimizer="muon" (Newton-Schulz in bf16 on the
    two matrices, Adam on the biases) for a few steps on stored activations."""
    from sparsify import SparseCoderConfig, TrainConfig, Trainer
    steps, B, T, D, M, k = 4, 4, 16, 32, 256, 4
    g = torch.Generator().manual_seed(6)
    atoms = torch.nn.functional.normalize(torch.randn(512, D, generator=g), dim=1)
    ids = torch.randint(0, 512, (steps, B, T, 6), generator=g)
    coef = -torch.log1p(-torch.rand(steps, B, T, 6, generator=g))
    acts = (atoms[ids] * coef.unsqueeze(-1)).sum(-2) + 0.05 * torch.randn(steps, B, T, D, generator=g)
    model = FakeModel(acts)
    dataset = [{"input_ids": torch.zeros(T, dtype=torch.long)} for _ in range(steps * B)]
    fvus = []
    with tempfile.TemporaryDirectory() as tmp:
        cfg = TrainConfig(SparseCoderConfig(num_latents=M, k=k), batch_size=B, optimizer="muon", lr=2e-3,
                          lr_warmup_steps=2, hookpoints=["layers.0"], log_to_wandb=False, save_dir=tmp,
                          run_name="golden", save_every=10**9)
        trainer = Trainer(cfg, dataset, model)
        sae = trainer.saes["layers.0"]
        init = dict(W_enc=sae.encoder.weight.detach().clone(), b_enc=sae.encoder.bias.detach().clone(),
                    W_dec=sae.W_dec.detach().clone(), b_dec=sae.b_dec.detach().clone())
        orig_forward = sae.forward

        def recording_forward(*a, **kw):
            out = orig_forward(*a, **kw)
            fvus.append(out.fvu.detach().clone())
            return out

        sae.forward = recording_forward
        trainer.fit()
        t = dict(acts=acts, fvu=torch.stack(fvus))
        for k_, v in init.items():
            t[f"init.{k_}"] = v
        for k_, v in dict(W_enc=sae.encoder.weight, b_enc=sae.encoder.bias, W_dec=sae.W_dec, b_dec=sae.b_dec).items():
            t[f"final.{k_}"] = v
        save("trainer_muon", t, dict(steps=steps, B=B, T=T, D=D, M=M, k=k, lr=2e-3, warmup=2))


def gen_trainer_signum(sparsify):
    """The reference Trainer with optimizer="signum" (its SignSGD inside the
    schedule-free wrapper, here the oracle's restatement of that third-party
    class) for a few steps on stored activations; the final parameters are read
    after the end-of-run checkpoint, i.e. back in training mode (y)."""
    from sparsify import SparseCoderConfig, TrainConfig, Trainer
    from safetensors.torch import load_file
    steps, B, T, D, M, k = 5, 4, 16, 32, 256, 4
    g = torch.Generator().manual_seed(8)
    atoms = torch.nn.functional.normalize(torch.randn(512, D, generator=g), dim=1)
    ids = torch.randint(0, 512, (steps, B, T, 6), generator=g)
    coef = -torch.log1p(-torch.rand(steps, B, T, 6, generator=g))
    acts = (atoms[ids] * coef.unsqueeze(-1)).sum(-2) + 0.05 * torch.randn(steps, B, T, D, generator=g)
    model = FakeModel(acts)
    dataset = [{"input_ids": torch.zeros(T, dtype=torch.long)} for _ in range(steps * B)]
    fvus = []
    with tempfile.TemporaryDirectory() as tmp:
        cfg = TrainConfig(SparseCoderConfig(num_latents=M, k=k), batch_size=B, optimizer="signum", lr=1e-3,
                          hookpoints=["layers.0"], log_to_wandb=False, save_dir=tmp, run_name="golden",
                          save_every=10**9)
        trainer = Trainer(cfg, dataset, model)
        sae = trainer.saes["layers.0"]
        init = dict(W_enc=sae.encoder.weight.detach().clone(), b_enc=sae.encoder.bias.detach().clone(),
                    W_dec=sae.W_dec.detach().clone(), b_dec=sae.b_dec.detach().clone())
        orig_forward = sae.forward

        def recording_forward(*a, **kw):
            out = orig_forward(*a, **kw)
            fvus.append(out.fvu.detach().clone())
            return out

        sae.forward = recording_forward
        trainer.fit()
        saved = load_file(f"{tmp}/golden/layers.0/sae.safetensors")  # averaged parameters (x)
        t = dict(acts=acts, fvu=torch.stack(fvus))
        for k_, v in init.items():
            t[f"init.{k_}"] = v
        for k_, v in dict(W_enc=sae.encoder.weight, b_enc=sae.encoder.bias, W_dec=sae.W_dec, b_dec=sae.b_dec).items():
            t[f"final.{k_}"] = v
        for k_, name in dict(W_enc="encoder.weight", b_enc="encoder.bias", W_dec="W_dec", b_dec="b_dec").items():
            t[f"saved.{k_}"] = saved[name]
        save("trainer_signum", t, dict(steps=steps, B=B, T=T, D=D, M=M, k=k, lr=1e-3))


def gen_trainer_e2e(sparsify):
    """The reference Trainer with the end-to-end objectives (loss_fn="ce" and "kl",
    trainer.py:425-430,478-500) on a small live language model (tests/fake_model.TinyLM):
    the sparse coder is spliced into the model's forward at layers.0 and the model's own
    loss trains it. Freezes the final parameters; inputs and model are rebuilt from seeds."""
    sys.path.insert(0, str(HERE.parent.parent))
    from tests.fake_model import TinyLM, token_dataset
    from sparsify import SparseCoderConfig, TrainConfig, Trainer
    steps, B, T, D, M, k = 4, 4, 16, 32, 256, 4
    for loss_fn in ("ce", "kl"):
        model = TinyLM(d=D, ctx=T)
        with tempfile.TemporaryDirectory() as tmp:
            cfg = TrainConfig(SparseCoderConfig(num_latents=M, k=k), batch_size=B, optimizer="adam", lr=1e-2,
                              lr_warmup_steps=1, loss_fn=loss_fn, hookpoints=["layers.0"], log_to_wandb=False,
                              save_dir=tmp, run_name="golden", save_every=10**9)
            trainer = Trainer(cfg, token_dataset(steps, B, T), model)
            sae = trainer.saes["layers.0"]
            t = {f"init.{n}": p.detach().clone() for n, p in
                 dict(W_enc=sae.encoder.weight, b_enc=sae.encoder.bias, W_dec=sae.W_dec, b_dec=sae.b_dec).items()}
            trainer.fit()
            for n, p in dict(W_enc=sae.encoder.weight, b_enc=sae.encoder.bias, W_dec=sae.W_dec, b_dec=sae.b_dec).items():
                t[f"final.{n}"] = p
            t["best_loss"] = torch.tensor(float(trainer.best_loss))
            save(f"trainer_{loss_fn}", t, dict(steps=steps, B=B, T=T, D=D, M=M, k=k, lr=1e-2, warmup=1))


def gen_trajectory200(sparsify, warmup=10, name="trajectory200"):
    """200 optimiser steps of the reference Trainer at the CPU configuration
    (d_in=768, 24576 latents, k=32, 4096 tokens/step, fp32, Adam, AuxK enabled)
    on the seeded synthetic activations of sparsify_b200.synthetic; only the FVU
    of every step is frozen (the inputs are regenerated from their seeds)."""
    sys.path.insert(0, str(HERE.parent.parent))
    from sparsify_b200.synthetic import SyntheticActivations, batch_seed
    from sparsify import SparseCoderConfig, TrainConfig, Trainer
    steps, B, T, D, M, k = 200, 8, 512, 768, 24576, 32
    gen = SyntheticActivations(D, 65536, 32, device="cpu")
    torch.set_num_threads(8)
    acts = torch.stack([gen.batch(B * T, batch_seed(t)).reshape(B, T, D) for t in range(steps)])
    model = FakeModel(acts)
    dataset = [{"input_ids": torch.zeros(T, dtype=torch.long)} for _ in range(steps * B)]
    fvus = []
    with tempfile.TemporaryDirectory() as tmp:
        cfg = TrainConfig(SparseCoderConfig(num_latents=M, k=k), batch_size=B, optimizer="adam",
                          lr_warmup_steps=warmup, auxk_alpha=1 / 32, hookpoints=["layers.0"], log_to_wandb=False,
                          save_dir=tmp, run_name="golden", save_every=10**9)
        trainer = Trainer(cfg, dataset, model)
        sae = trainer.saes["layers.0"]
        orig_forward = sae.forward

        def recording_forward(*a, **kw):
            out = orig_forward(*a, **kw)
            fvus.append(float(out.fvu))
            return out

        sae.forward = recording_forward
        trainer.fit()
    save(name, dict(fvu=torch.tensor(fvus)),
         dict(steps=steps, B=B, T=T, D=D, M=M, k=k, atoms=65536, active=32, warmup=warmup, auxk_alpha=1 / 32))
    print("fvu first/last:", fvus[0], fvus[-1])


def gen_muon(sparsify):
    from sparsify.muon import quintic_newtonschulz
    g = torch.Generator().manual_seed(3)
    for name, shape in [("wide", (32, 96)), ("tall", (96, 32))]:
        G = torch.randn(*shape, generator=g)
        X = quintic_newtonschulz(G, 5)
        save(f"newtonschulz_{name}", dict(G=G, X=X.float()))


def gen_checkpoints(sparsify):
    """Checkpoint trees written by the reference itself, for the loaders of this package:
    `SparseCoder.save_to_disk` of a small SAE and of a transcoder with a skip connection
    (sparsify/sparse_coder.py:167-179), and the tree `Trainer.save()` leaves after three
    optimiser steps (sparsify/trainer.py:648-699). Stored under tests/golden/ckpt_ref/."""
    import shutil
    from sparsify import SparseCoder, SparseCoderConfig, TrainConfig, Trainer
    root = HERE / "ckpt_ref"
    if root.exists():
        shutil.rmtree(root)
    for name, cfg in (("sae", SparseCoderConfig(num_latents=48, k=4)),
                      ("transcoder", SparseCoderConfig(num_latents=40, k=3, transcode=True, skip_connection=True))):
        torch.manual_seed(31)
        sae = SparseCoder(12, cfg)
        with torch.no_grad():
            for q in sae.parameters():
                q.add_(0.1 * torch.randn_like(q))
        sae.save_to_disk(root / name)
    steps, B, T, D, M, k = 3, 2, 8, 12, 48, 4
    g = torch.Generator().manual_seed(32)
    acts = torch.randn(steps, B, T, D, generator=g)
    model = FakeModel(acts)
    dataset = [{"input_ids": torch.zeros(T, dtype=torch.long)} for _ in range(steps * B)]
    cfg = TrainConfig(SparseCoderConfig(num_latents=M, k=k), batch_size=B, optimizer="adam", lr_warmup_steps=2,
                      auxk_alpha=1 / 32, dead_feature_threshold=20, hookpoints=["layers.0"], log_to_wandb=False,
                      save_dir=str(root), run_name="trainer", save_every=10 ** 9)
    trainer = Trainer(cfg, dataset, model)
    trainer.fit()  # ends with Trainer.save()
    print("wrote", sorted(str(f.relative_to(root)) for f in root.rglob("*") if f.is_file()))


def check_reference_loads_ours(sparsify):
    """The other direction: a tree written by THIS package (SparseCoder.save_to_disk and
    Trainer.save, on the host) read by the reference's own loaders
    (sparsify/sparse_coder.py:134-165, sparsify/trainer.py:186-227). Records the outcome in
    tests/golden/ckpt_interchange.json; tests/test_checkpoint_interchange.py repeats the check
    live wherever the reference is at hand."""
    sys.path.insert(0, str(HERE.parent.parent))
    from tests.test_checkpoint_interchange import reference_reads_our_tree
    with tempfile.TemporaryDirectory() as tmp:
        report = reference_reads_our_tree(sparsify, Path(tmp))
    with open(HERE / "ckpt_interchange.json", "w") as f:
        json.dump(report, f, indent=1)
    print("ckpt_interchange.json:", report)


if __name__ == "__main__":
    ref = import_reference()
    if "--checkpoints" in sys.argv:  # only the checkpoint interchange fixtures
        gen_checkpoints(ref)
        check_reference_loads_ours(ref)
        sys.exit(0)
    torch.set_num_threads(1)  # one summation order
    gen_encoder(ref)
    gen_decoder(ref)
    gen_forward(ref)
    gen_trainer(ref)
    gen_trainer_muon(ref)
    gen_trainer_signum(ref)
    gen_trainer_e2e(ref)
    gen_muon(ref)
    if "--trajectory" in sys.argv:  # about three minutes of CPU time on 8 threads
        gen_trajectory200(ref)
        gen_trajectory200(ref, warmup=1000, name="trajectory200_warmup1000")  # the reference's default
