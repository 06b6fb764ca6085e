"""Trainer with the reference's surface (sparsify/trainer.py:28-728):
``Trainer(cfg, dataset, model)``, ``fit()``, ``save()``, ``load_state(path)``,
``saes``, ``module_plan``, ``local_hookpoints()`` and the same checkpoint tree.

The step it drives per hookpoint is the reference's (trainer.py:340-447,
510-538): mask tokens, step-0 bias initialisation, decoder normalisation,
forward (FVU + AuxK + Multi-TopK), backward, gradient exchange, projection of
the decoder gradient, optimiser step, dead-latent bookkeeping - with the
arithmetic done by the CUDA kernels. Differences, all outside the arithmetic:

* data parallel: gradients are averaged by `parallel.GradReducer`
  (asynchronous all-reduce per parameter, overlapped with backward) instead of
  a DistributedDataParallel wrapper;
* `distribute_modules`: activations go to the owning rank only;
* `loss_fn` "ce"/"kl" (trainer.py:425-430,486-500): the sparse coder's output
  replaces the module's output inside the model's forward and the model's own
  loss is back-propagated; these steps take the composed autograd path (dense
  gradients), since the gradient arrives through `sae_out`;
* Weights & Biases logging is not part of this package; metrics go to
  `metrics.jsonl` in the run directory under the names the reference logs.
"""

from __future__ import annotations

import json
import os
from collections import defaultdict
from fnmatch import fnmatchcase
from glob import glob
from typing import Sized

import torch
import torch.distributed as dist
from safetensors.torch import load_model
from torch import Tensor, nn
from torch.utils.data import DataLoader

from . import parallel
from .config import TrainConfig
from .muon import Muon
from .optim import FusedAdam, ScheduleFreeSignum
from .sparse_coder import SparseCoder, natsorted
from .utils import get_layer_list, resolve_widths


def linear_schedule_with_warmup(optimizer, num_warmup_steps: int, num_training_steps: int):
    """transformers.get_linear_schedule_with_warmup (used at trainer.py:117-121)."""
    def lr_lambda(step: int):
        if step < num_warmup_steps:
            return float(step) / float(max(1, num_warmup_steps))
        return max(0.0, float(num_training_steps - step) / float(max(1, num_training_steps - num_warmup_steps)))
    return torch.optim.lr_scheduler.LambdaLR(optimizer, lr_lambda)


def sparse_update_allowed(cfg: TrainConfig, world_size: int) -> bool:
    """Whether the optimiser may consume the weight gradients in sparse form (and, on several
    data-parallel ranks, shard the update over them).

    Needs: nothing else wants the dense gradients (no accumulation, the plain FVU objective).
    On several data-parallel ranks the sharded update also assumes that every rank holds the
    same set of dead latents, because their AuxK gradient rows are summed with a collective
    whose shape is that set. The dead-latent counters advance by each rank's own unmasked
    token count (sparsify/trainer.py:471-472,529-538), which `exclude_tokens` makes differ
    between ranks: with AuxK enabled the sets can then diverge, so that combination keeps the
    dense gradients, whose all-reduce has a fixed shape (as DistributedDataParallel's has)."""
    if cfg.grad_acc_steps * cfg.micro_acc_steps != 1 or cfg.loss_fn != "fvu":
        return False
    data_parallel = world_size > 1 and not cfg.distribute_modules
    if data_parallel and cfg.exclude_tokens and cfg.auxk_alpha > 0:
        return False
    return True


class Trainer:
    def __init__(self, cfg: TrainConfig, dataset, model: nn.Module):
        self.model = model

        if cfg.hookpoints:
            assert not cfg.layers, "Cannot specify both `hookpoints` and `layers`."
            raw = [name for name, _ in model.base_model.named_modules()
                   if any(fnmatchcase(name, pat) for pat in cfg.hookpoints)]
            cfg.hookpoints = natsorted(raw)
        else:
            if not cfg.layers:
                cfg.layers = list(range(0, model.config.num_hidden_layers))
            layers_name, _ = get_layer_list(model)
            cfg.hookpoints = [f"{layers_name}.{i}" for i in cfg.layers]
        cfg.hookpoints = cfg.hookpoints[:: cfg.layer_stride]

        self.cfg = cfg
        self.dataset = dataset
        self.distribute_modules()

        device = model.device
        if dist.is_initialized() and dist.get_world_size() > 1 and torch.device(device).type == "cuda":
            # collectives run beside the persistent tensor-core kernels: leave NCCL a few SMs
            from . import ops
            ops.set_reserved_sms(int(os.environ.get("SPARSIFY_RESERVED_SMS", "4")))
        input_widths = resolve_widths(model, cfg.hookpoints)
        unique_widths = set(input_widths.values())
        if cfg.distribute_modules and len(unique_widths) > 1:
            raise ValueError(
                f"All modules must output tensors of the same shape when using "
                f"`distribute_modules=True`, got {unique_widths}"
            )
        if cfg.loss_fn not in ("fvu", "ce", "kl"):
            raise ValueError(f"Unknown loss function '{cfg.loss_fn}'")

        print(f"Initializing SAEs with random seed(s) {cfg.init_seeds}")
        self.saes: dict[str, SparseCoder] = {}
        for hook in self.local_hookpoints():
            for seed in cfg.init_seeds:
                torch.manual_seed(seed)
                name = f"{hook}/seed{seed}" if len(cfg.init_seeds) > 1 else hook
                self.saes[name] = SparseCoder(input_widths[hook], cfg.sae, device, dtype=torch.float32)

        assert isinstance(dataset, Sized)
        num_batches = len(dataset) // cfg.batch_size

        match cfg.optimizer:
            case "adam":
                pgs = [dict(params=list(sae.parameters()),
                            lr=cfg.lr or 2e-4 / (sae.num_latents / (2 ** 14)) ** 0.5)
                       for sae in self.saes.values()]
                lrs = [f"{lr:.2e}" for lr in sorted(set(pg["lr"] for pg in pgs))]
                adam = FusedAdam(pgs)
                # (end-to-end losses reach the weights through sae_out: dense gradients)
                no_acc = sparse_update_allowed(cfg, dist.get_world_size() if dist.is_initialized() else 1)
                for sae in self.saes.values():
                    sae.attach_optimizer(adam)
                    sae.ragged_tokens = bool(cfg.exclude_tokens)
                    if no_acc:
                        # Nothing but the optimiser needs the dense weight gradients: hand them
                        # over in sparse form (sharded over ranks when data parallel).
                        adam.enable_sparse_update(sae, data_parallel=not cfg.distribute_modules)
                self.optimizers = [adam]
                self.lr_schedulers = [linear_schedule_with_warmup(adam, cfg.lr_warmup_steps, num_batches)]
            case "muon":
                # name-sorted so that the matrix -> rank assignment is the same in every process
                named = [(f"{n}.{pn}", p) for n, sae in self.saes.items() for pn, p in sae.named_parameters()]
                muon_params = [p for _, p in sorted(named, key=lambda t: t[0]) if p.ndim >= 2]
                other = [p for _, p in named if p.ndim < 2]
                lrs = [f"{cfg.lr or 2e-3:.2e}"]
                self.optimizers = [
                    Muon(muon_params, lr=cfg.lr or 2e-3, ddp=not cfg.distribute_modules),
                    FusedAdam(other, lr=cfg.lr or 2e-3),
                ]
                for sae in self.saes.values():
                    sae.attach_optimizer(self.optimizers[0], project=False)  # bf16 copies only
                self.lr_schedulers = [
                    linear_schedule_with_warmup(self.optimizers[0], 0, num_batches),
                    linear_schedule_with_warmup(self.optimizers[1], cfg.lr_warmup_steps, num_batches),
                ]
            case "signum":
                pgs = [dict(params=list(sae.parameters()),
                            lr=cfg.lr or 5e-3 / (sae.num_latents / (2 ** 14)) ** 0.5)
                       for sae in self.saes.values()]
                lrs = [f"{lr:.2e}" for lr in sorted(set(pg["lr"] for pg in pgs))]
                opt = ScheduleFreeSignum(pgs, momentum=0.95)
                for sae in self.saes.values():
                    sae.attach_optimizer(opt)
                    sae.ragged_tokens = bool(cfg.exclude_tokens)
                opt.train()
                self.optimizers = [opt]
                self.lr_schedulers = []
            case other:
                raise ValueError(f"Unknown optimizer '{other}'")

        print(f"Learning rates: {lrs}" if len(lrs) > 1 else f"Learning rate: {lrs[0]}")
        self.global_step = 0
        self.num_tokens_since_fired = {
            name: torch.zeros(sae.num_latents, device=device, dtype=torch.long)
            for name, sae in self.saes.items()
        }
        self.exclude_tokens = torch.tensor(self.cfg.exclude_tokens, device=device, dtype=torch.long)

        num_latents = list(self.saes.values())[0].num_latents
        self.initial_k = min(num_latents, round(list(input_widths.values())[0] * 10))
        self.final_k = self.cfg.sae.k
        self.best_loss = ({name: float("inf") for name in self.local_hookpoints()}
                          if cfg.loss_fn == "fvu" else float("inf"))  # trainer.py:180-184
        self.metrics: list[dict] = []
        self._tokens_seen = 0  # upper bound of every num_tokens_since_fired counter
        self._dead_masks: dict[str, Tensor] = {}  # next step's dead masks, already read back

    # ------------------------------------------------------------------ state
    def load_state(self, path: str):
        """Load the trainer state from disk (layout of trainer.py:186-227)."""
        device = self.model.device
        train_state = torch.load(f"{path}/state.pt", map_location=device, weights_only=True)
        self.global_step = train_state["global_step"]

        for file in glob(f"{path}/rank_*_state.pt"):
            rank_state = torch.load(file, map_location=device, weights_only=True)
            for k in self.local_hookpoints():
                if k in rank_state["num_tokens_since_fired"]:
                    self.num_tokens_since_fired[k] = rank_state["num_tokens_since_fired"][k]
                    self._tokens_seen = max(self._tokens_seen, int(self.num_tokens_since_fired[k].max()))
                if not isinstance(rank_state["best_loss"], dict):
                    self.best_loss = rank_state["best_loss"]
                elif k in rank_state["best_loss"]:
                    self.best_loss[k] = rank_state["best_loss"][k]

        self._dead_masks.clear()
        print(f"\033[92mResuming training at step {self.global_step} from '{path}'\033[0m")
        for i, scheduler in enumerate(self.lr_schedulers):
            scheduler.load_state_dict(
                torch.load(f"{path}/lr_scheduler_{i}.pt", map_location=device, weights_only=True))
        for i, optimizer in enumerate(self.optimizers):
            optimizer.load_state_dict(
                torch.load(f"{path}/optimizer_{i}.pt", map_location=device, weights_only=True))
        for name, sae in self.saes.items():
            load_model(sae, f"{path}/{name}/sae.safetensors", device=str(device))

    def get_current_k(self) -> int:
        """Linear decay of k from initial_k to final_k (trainer.py:229-235)."""
        if self.global_step >= self.cfg.k_decay_steps:
            return self.final_k
        progress = self.global_step / self.cfg.k_decay_steps
        return round(self.initial_k * (1 - progress) + self.final_k * progress)

    # ------------------------------------------------------------------ training
    def fit(self):
        self.model.requires_grad_(False)
        rank_zero = not dist.is_initialized() or dist.get_rank() == 0
        ddp = dist.is_initialized() and not self.cfg.distribute_modules
        world = dist.get_world_size() if dist.is_initialized() else 1

        num_sae_params = sum(p.numel() for s in self.saes.values() for p in s.parameters())
        print(f"Number of SAE parameters: {num_sae_params:_}")

        if self.global_step > 0:
            assert hasattr(self.dataset, "select"), "Dataset must implement `select`"
            n = self.global_step * self.cfg.batch_size
            ds = self.dataset.select(range(n, len(self.dataset)))
        else:
            ds = self.dataset

        device = self.model.device
        dl = DataLoader(ds, batch_size=self.cfg.batch_size, shuffle=False)

        did_fire = {name: torch.zeros(sae.num_latents, device=device, dtype=torch.bool)
                    for name, sae in self.saes.items()}
        tokens_mask: Tensor

        acc_steps = self.cfg.grad_acc_steps * self.cfg.micro_acc_steps
        denom = acc_steps * self.cfg.wandb_log_frequency
        num_tokens_in_step = 0
        avg_auxk_loss = defaultdict(float)
        avg_fvu = defaultdict(float)
        avg_multi_topk_fvu = defaultdict(float)
        avg_losses = {name: float("inf") for name in self.local_hookpoints()}
        avg_e2e = 0.0  # cross-entropy or KL of the model with the sparse coders spliced in

        name_to_module = {name: self.model.base_model.get_submodule(name) for name in self.cfg.hookpoints}
        module_to_name = {v: k for k, v in name_to_module.items()}
        reducer: parallel.GradReducer | None = None
        # loss scalars stay on the device until the step ends: one host sync per step
        pending_metrics: list[tuple] = []

        e2e = self.cfg.loss_fn in ("ce", "kl")
        # activations travel to their owners on a stream of their own, so a rank that only
        # contributes its slice is not held back by the owner's queued work
        gather_stream = (torch.cuda.Stream(device=device)
                         if self.cfg.distribute_modules and torch.device(device).type == "cuda" else None)
        # ... and the owner trains its coder on a second stream, so that the model's forward
        # (and with it the hooks of later layers, on every rank) is not queued behind it
        sae_stream = torch.cuda.Stream(device=device) if gather_stream is not None else None
        ragged_possible = bool(self.cfg.exclude_tokens)

        # Owners do not train inside the hook: they only start the exchange there and train once
        # the model's forward has returned. A rank's contribution to later hookpoints is then
        # issued at the pace of the model's forward, not after this rank's own training calls
        # (whose host-side work would otherwise delay every later owner).
        deferred: list = []

        def hook(module: nn.Module, inputs, outputs):
            if sae_stream is None:
                return hook_body(module, inputs, outputs, None)
            ready = torch.cuda.Event()
            ready.record()  # the module's output is complete at this point of the model's stream
            with torch.cuda.stream(sae_stream):
                sae_stream.wait_event(ready)
                return hook_body(module, inputs, outputs, ready)

        def hook_body(module: nn.Module, inputs, outputs, ready):
            aux_out = None
            if isinstance(inputs, tuple):
                inputs = inputs[0]
            if isinstance(outputs, tuple):
                outputs, *aux_out = outputs
            mask = tokens_mask
            hookpoint = module_to_name[module]
            out_shape = outputs.shape

            if self.cfg.distribute_modules:
                owner = parallel.owner_of(self.module_plan, hookpoint)
                outputs = parallel.gather_to_owner(outputs, owner, stream=gather_stream, after=ready)
                if self.cfg.sae.transcode:
                    inputs = parallel.gather_to_owner(inputs, owner, stream=gather_stream, after=ready)
                mask = parallel.gather_to_owner(mask.to(torch.uint8), owner, stream=gather_stream)
                if dist.get_rank() != owner:
                    return
                mask = mask.bool()
                if sae_stream is not None:
                    deferred.append((hookpoint, inputs, outputs, mask))
                    return

            return train_hookpoint(hookpoint, inputs, outputs, mask, aux_out, out_shape)

        def train_hookpoint(hookpoint, inputs, outputs, mask, aux_out, out_shape):
            outputs = outputs.flatten(0, 1)
            inputs = inputs.flatten(0, 1) if self.cfg.sae.transcode else outputs
            mask = mask.flatten(0, 1)
            all_outputs = outputs.detach() if e2e else None
            # without excluded tokens the mask is all ones by construction: no read-back
            ragged = ragged_possible and not bool(mask.all())
            if ragged:
                outputs = outputs[mask]
                inputs = inputs[mask] if self.cfg.sae.transcode else outputs

            seeds = self.cfg.init_seeds
            names = [f"{hookpoint}/seed{s}" for s in seeds] if len(seeds) > 1 else [hookpoint]
            for name in names:
                raw = self.saes[name]
                if self.global_step == 0 and not self.cfg.finetune:
                    # centre the pre-activations and the reconstruction (trainer.py:393-404)
                    with torch.no_grad():
                        if self.cfg.sae.transcode:
                            mean = self.maybe_all_reduce(inputs.float().mean(0)).to(raw.dtype)
                            raw.encoder.bias.data = -mean @ raw.encoder.weight.data.T
                        mean = self.maybe_all_reduce(outputs.float().mean(0))
                        raw.b_dec.data = mean.to(raw.dtype)

                if raw.cfg.normalize_decoder and not self.cfg.sae.transcode:
                    raw.set_decoder_norm_to_unit_norm()

                # No counter can exceed the number of tokens this rank has trained on, so
                # until that passes the threshold the mask is known to be empty and is not
                # built (the forward would otherwise read its sum back to the host).
                may_be_dead = self.cfg.auxk_alpha > 0 and self._tokens_seen > self.cfg.dead_feature_threshold
                raw.fused = not e2e  # a gradient arriving through sae_out needs the autograd path
                out = raw(
                    x=inputs,
                    y=outputs,
                    dead_mask=((self._dead_masks[name] if name in self._dead_masks else
                                self.num_tokens_since_fired[name] > self.cfg.dead_feature_threshold)
                               if may_be_dead else None),
                )
                # index_fill_ is queued like any kernel; `mask[indices] = True` makes the host wait
                # for everything queued before it
                did_fire[name].index_fill_(0, out.latent_indices.flatten(), True)
                self.maybe_all_reduce(did_fire[name], "max")

                if e2e:
                    # the sparse coder's output takes the module's place in the model's forward
                    # (trainer.py:425-430); the model's loss is back-propagated by fit()
                    if ragged:
                        output = all_outputs.clone()
                        output[mask] = out.sae_out.type_as(output)
                    else:
                        output = out.sae_out.type_as(all_outputs)
                    output = output.reshape(out_shape)
                    return (output, *aux_out) if aux_out is not None else output

                pending_metrics.append((name, out.fvu.detach(), out.auxk_loss.detach(),
                                        out.multi_topk_fvu.detach()))
                loss = out.fvu + self.cfg.auxk_alpha * out.auxk_loss + out.multi_topk_fvu / 8
                loss.div(acc_steps).backward()

        k = self.get_current_k()
        for sae in self.saes.values():
            sae.cfg.k = k

        for batch in dl:
            x = batch["input_ids"].to(device)
            tokens_mask = torch.isin(x, self.exclude_tokens, invert=True)

            step, substep = divmod(self.global_step + 1, self.cfg.grad_acc_steps)
            if ddp and reducer is None:
                reducer = parallel.GradReducer(
                    [p for sae in self.saes.values() for p in sae.parameters()]).attach()
            if reducer is not None:
                reducer.enabled = substep == 0

            # without excluded tokens every token counts: no read-back of the mask's sum
            N = int(tokens_mask.sum().item()) if self.cfg.exclude_tokens else tokens_mask.numel()
            num_tokens_in_step += N

            # clean next-token distribution for the KL objective (trainer.py:478-483)
            clean_probs = self.model(x).logits.softmax(dim=-1) if self.cfg.loss_fn == "kl" else None

            handles = [mod.register_forward_hook(hook) for mod in name_to_module.values()]
            try:
                match self.cfg.loss_fn:
                    case "ce":
                        ce = self.model(x, labels=x).loss
                        ce.div(acc_steps).backward()
                        avg_e2e += float(self.maybe_all_reduce(ce.detach()) / denom)
                    case "kl":
                        dirty_lps = self.model(x).logits.log_softmax(dim=-1)
                        kl = -torch.sum(clean_probs * dirty_lps, dim=-1).mean()
                        kl.div(acc_steps).backward()
                        avg_e2e += float(self.maybe_all_reduce(kl.detach()) / denom)
                    case _:
                        self.model(x)
            finally:
                for handle in handles:
                    handle.remove()
            if sae_stream is not None:
                with torch.cuda.stream(sae_stream):
                    for job in deferred:  # this rank's hookpoints, in the model's order
                        train_hookpoint(*job, None, None)
                deferred.clear()
                torch.cuda.current_stream(device).wait_stream(sae_stream)  # the coders' work joins here

            # metric reads (one sync for all hookpoints of this batch)
            for name, fvu, auxk, multi in pending_metrics:
                avg_fvu[name] += float(self.maybe_all_reduce(fvu) / denom)
                if self.cfg.auxk_alpha > 0:
                    avg_auxk_loss[name] += float(self.maybe_all_reduce(auxk) / denom)
                if self.cfg.sae.multi_topk:
                    avg_multi_topk_fvu[name] += float(self.maybe_all_reduce(multi) / denom)
            pending_metrics.clear()
            avg_losses = avg_e2e if e2e else dict(avg_fvu)
            if torch.device(device).type == "cuda":
                # the reads above waited for the device: the cheapest place to learn that a
                # bounded wait inside a tensor-core kernel gave up (its results are garbage)
                from . import ops
                ops.check_status(device)

            if substep == 0:
                if reducer is not None:
                    reducer.finish()
                # the decoder-gradient projection (trainer.py:513-515) runs inside
                # FusedAdam's update kernel; Muon needs it applied beforehand
                if self.cfg.optimizer == "muon" and self.cfg.sae.normalize_decoder and not self.cfg.sae.transcode:
                    for sae in self.saes.values():
                        sae.remove_gradient_parallel_to_decoder_directions()

                # Dead-latent bookkeeping (trainer.py:529-538; independent of the optimiser step,
                # done first): the metric reads above have just drained the device queue, so this
                # is where next step's dead latents are read back (their indices, once) - the
                # forward pass then needs no read-back of its own.
                self._tokens_seen += num_tokens_in_step
                with torch.no_grad():
                    for name, counts in self.num_tokens_since_fired.items():
                        counts += num_tokens_in_step
                        counts[did_fire[name]] = 0
                        if self.cfg.auxk_alpha > 0 and self._tokens_seen > self.cfg.dead_feature_threshold:
                            self._dead_masks[name] = self.saes[name].prepare_dead_mask(
                                counts > self.cfg.dead_feature_threshold)
                    num_tokens_in_step = 0
                    for mask in did_fire.values():
                        mask.zero_()

                for optimizer in self.optimizers:
                    optimizer.step()
                    optimizer.zero_grad()
                for scheduler in self.lr_schedulers:
                    scheduler.step()

                k = self.get_current_k()
                for sae in self.saes.values():
                    sae.cfg.k = k

                if (step + 1) % self.cfg.save_every == 0:
                    self.save()
                    if self.cfg.save_best:
                        self.save_best(avg_losses)

                if (step + 1) % self.cfg.wandb_log_frequency == 0:
                    info = {"step": step, "k": k}
                    if e2e:
                        info["ce_loss" if self.cfg.loss_fn == "ce" else "kl_loss"] = avg_e2e
                    for name in self.saes:
                        dead = self.num_tokens_since_fired[name] > self.cfg.dead_feature_threshold
                        info[f"dead_pct/{name}"] = dead.mean(dtype=torch.float32).item()
                        if not e2e:
                            info[f"fvu/{name}"] = avg_fvu[name]
                        if self.cfg.auxk_alpha > 0:
                            info[f"auxk/{name}"] = avg_auxk_loss[name]
                        if self.cfg.sae.multi_topk:
                            info[f"multi_topk_fvu/{name}"] = avg_multi_topk_fvu[name]
                    self.metrics.append(info)

                avg_auxk_loss.clear()
                avg_fvu.clear()
                avg_multi_topk_fvu.clear()
                avg_e2e = 0.0

            self.global_step += 1

        if reducer is not None:
            reducer.detach()
        self.save()
        if self.cfg.save_best:
            self.save_best(avg_losses)

    # ------------------------------------------------------------------ distribution
    def local_hookpoints(self) -> list[str]:
        return self.module_plan[dist.get_rank()] if self.module_plan else self.cfg.hookpoints

    def maybe_all_reduce(self, x: Tensor, op: str = "mean") -> Tensor:
        if not dist.is_initialized() or self.cfg.distribute_modules:
            return x
        return parallel.all_reduce_(x, op)

    def distribute_modules(self):
        """Prepare a plan for distributing modules across ranks."""
        if not self.cfg.distribute_modules:
            self.module_plan = []
            print(f"Training on modules: {self.cfg.hookpoints}")
            return
        self.module_plan = parallel.module_plan(self.cfg.hookpoints, dist.get_world_size())
        for rank, modules in enumerate(self.module_plan):
            print(f"Rank {rank} modules: {modules}")

    # ------------------------------------------------------------------ checkpoints
    def _checkpoint(self, saes: dict[str, SparseCoder], path: str, rank_zero: bool):
        """Layout of trainer.py:648-686: {path}/{name}/sae.safetensors + cfg.json,
        and on rank 0 lr_scheduler_i.pt, optimizer_i.pt, state.pt, config.json; every
        saving rank writes rank_{r}_state.pt."""
        print("Saving checkpoint")
        for optimizer in self.optimizers:
            if isinstance(optimizer, ScheduleFreeSignum):
                optimizer.eval()  # the checkpoint stores the averaged parameters (trainer.py:652-654)
        for name, sae in saes.items():
            assert isinstance(sae, SparseCoder)
            sae.save_to_disk(f"{path}/{name}")

        if rank_zero:
            os.makedirs(path, exist_ok=True)
            for i, scheduler in enumerate(self.lr_schedulers):
                torch.save(scheduler.state_dict(), f"{path}/lr_scheduler_{i}.pt")
            for i, optimizer in enumerate(self.optimizers):
                torch.save(optimizer.state_dict(), f"{path}/optimizer_{i}.pt")
            torch.save({"global_step": self.global_step}, f"{path}/state.pt")
            self.cfg.save_json(f"{path}/config.json")
            if self.metrics:
                with open(f"{path}/metrics.jsonl", "w") as f:
                    for row in self.metrics:
                        f.write(json.dumps(row) + "\n")

        for optimizer in self.optimizers:
            if isinstance(optimizer, ScheduleFreeSignum):
                optimizer.train()

        rank = 0 if rank_zero else dist.get_rank()
        os.makedirs(path, exist_ok=True)
        torch.save(
            {"num_tokens_since_fired": self.num_tokens_since_fired, "best_loss": self.best_loss},
            f"{path}/rank_{rank}_state.pt",
        )

    def save(self):
        """Save the SAEs and training state to disk."""
        path = f'{self.cfg.save_dir}/{self.cfg.run_name or "unnamed"}'
        rank_zero = not dist.is_initialized() or dist.get_rank() == 0
        for opt in self.optimizers:
            if isinstance(opt, FusedAdam):
                opt.sync_masters()  # sharded updates: make every replica whole before writing
        if rank_zero or self.cfg.distribute_modules:
            self._checkpoint(self.saes, path, rank_zero)
        if dist.is_initialized():
            dist.barrier()

    def save_best(self, avg_loss: float | dict[str, float]):
        """Save individual sparse coders to disk if they have the lowest loss (a dict of
        per-hookpoint FVUs, or the model's single loss for the end-to-end objectives)."""
        base_path = f'{self.cfg.save_dir}/{self.cfg.run_name or "unnamed"}/best'
        rank_zero = not dist.is_initialized() or dist.get_rank() == 0
        if isinstance(avg_loss, dict):
            for name in self.saes:
                if avg_loss.get(name, float("inf")) < self.best_loss.get(name, float("inf")):
                    self.best_loss[name] = avg_loss[name]
                    if rank_zero or self.cfg.distribute_modules:
                        self._checkpoint({name: self.saes[name]}, f"{base_path}/{name}", rank_zero)
        else:
            if avg_loss < self.best_loss:
                self.best_loss = avg_loss
                if rank_zero or self.cfg.distribute_modules:
                    self._checkpoint(self.saes, base_path, rank_zero)
        if dist.is_initialized():
            dist.barrier()


# Support old name for compatibility
SaeTrainer = Trainer
