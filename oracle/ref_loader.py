"""Loads and times the REFERENCE implementation itself. TEST INFRASTRUCTURE ONLY.

The reference (EleutherAI/sparsify v1.3.0) is pure Python on top of PyTorch, so
its own code runs on the host CPU wherever its source tree is. Nothing of it is
part of this repository: `oracle/make_ref.py` copies the package directory of a
reference checkout into `oracle/_ref/` (git-ignored, built like a compiled
artefact), and this module imports it from there. Used by

* `tests/golden/make_golden.py` - generates the fixtures the oracle is pinned to,
* `bench.py --impl reference` and the `cpu_baseline` leg of `bench.py` - time the
  reference's own `Trainer.fit()` on the host cores next to the GPU numbers.

Four third-party modules the reference imports are not installed here and do no
arithmetic on the timed path; they are replaced by small stand-ins:
`natsort.natsorted` (sparsify/sparse_coder.py:9,98,107; trainer.py:11,48),
`simple_parsing.Serializable/list_field/field/parse` (config serialisation,
sparsify/config.py:5,85-95; sparse_coder.py:146,175; trainer.py:673),
`accelerate.utils.send_to_device` (sparsify/utils.py:5,54) and the class
`schedulefree.ScheduleFreeWrapper` (an isinstance check, trainer.py:13,653,676;
only optimizer="signum" instantiates it).
"""

from __future__ import annotations

import dataclasses
import json
import os
import re
import sys
import tempfile
import time
import types
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"


def find_reference() -> Path | None:
    """Directory that holds the reference's `sparsify/` package: $SPARSIFY_REF if it
    points at a checkout, else the vendored copy under oracle/_ref."""
    for root in (os.environ.get("SPARSIFY_REF", ""), str(REF_DIR)):
        if root and Path(root, "sparsify", "fused_encoder.py").exists():
            return Path(root)
    return None


def _natsorted(seq, key=None):
    def split(s):
        return [int(t) if t.isdigit() else t for t in re.split(r"(\d+)", str(s))]
    return sorted(seq, key=(lambda v: split(key(v))) if key else split)


class _Serializable:
    def to_dict(self):
        return dataclasses.asdict(self)

    @classmethod
    def from_dict(cls, d, drop_extra_fields=False):
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    def save_json(self, path):
        with open(path, "w") as f:
            json.dump(self.to_dict(), f)


class _NoScheduleFree:
    """Placeholder so that `isinstance(opt, ScheduleFreeWrapper)` is False."""


def import_reference(schedulefree_wrapper=None, triton: bool = False):
    """Imports the reference package and returns the module. triton=False (the CPU arm and the
    fixtures): Triton disabled, as the reference does when SPARSIFY_DISABLE_TRITON=1
    (sparsify/utils.py:94-103); triton=True leaves the reference's own dispatch alone, which
    on a GPU box compiles and uses its Triton decoder kernels (sparsify/xformers.py)."""
    root = find_reference()
    if root is None:
        raise RuntimeError("the reference is not available: run `python oracle/make_ref.py` where a checkout of "
                           "EleutherAI/sparsify v1.3.0 exists, or point SPARSIFY_REF at one")
    if triton:
        os.environ.pop("SPARSIFY_DISABLE_TRITON", None)
    else:
        os.environ["SPARSIFY_DISABLE_TRITON"] = "1"
    import transformers  # noqa: F401  (must be imported before the accelerate stand-in exists)

    natsort = types.ModuleType("natsort")
    natsort.natsorted = _natsorted
    sp = types.ModuleType("simple_parsing")
    sp.Serializable = _Serializable
    sp.list_field = lambda *d: dataclasses.field(default_factory=lambda: list(d))
    sp.field = dataclasses.field
    sp.parse = lambda *a, **k: None
    acc = types.ModuleType("accelerate")
    acc_utils = types.ModuleType("accelerate.utils")
    acc_utils.send_to_device = lambda obj, device: obj
    acc.utils = acc_utils
    sf = types.ModuleType("schedulefree")
    sf.ScheduleFreeWrapper = schedulefree_wrapper or _NoScheduleFree
    for name, mod in [("natsort", natsort), ("simple_parsing", sp), ("accelerate", acc),
                      ("accelerate.utils", acc_utils), ("schedulefree", sf)]:
        sys.modules.setdefault(name, mod)
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    import sparsify
    return sparsify


# ----------------------------------------------------------------------------- timing
class _Layer(torch.nn.Module):
    def __init__(self, owner):
        super().__init__()
        object.__setattr__(self, "_owner", owner)

    def forward(self, h):
        return self._owner.next_activation()


class StoredActivations(torch.nn.Module):
    """What the reference Trainer hooks into instead of a language model: one layer whose
    output is the next stored batch [B, T, D]. Records the wall-clock time of every
    forward call, i.e. of every step boundary of `Trainer.fit()`."""

    def __init__(self, acts: torch.Tensor):
        super().__init__()
        self.config = types.SimpleNamespace(num_hidden_layers=1)
        self.layers = torch.nn.ModuleList([_Layer(self)])
        self.acts = acts  # [steps, B, T, D], on the device the coders are to live on
        self.cursor = -1  # the Trainer's width probe consumes one call
        self.dummy_inputs = {"input_ids": torch.zeros(1, acts.shape[2], dtype=torch.long)}
        self.stamps: list[float] = []

    @property
    def base_model(self):
        return self

    @property
    def device(self):
        return self.acts.device

    def next_activation(self):
        i = max(self.cursor, 0)
        self.cursor += 1
        return self.acts[min(i, self.acts.shape[0] - 1)]

    def forward(self, input_ids=None, **kw):
        if self.cursor >= 0:
            if self.acts.is_cuda:
                torch.cuda.synchronize(self.acts.device)  # the previous step has finished on the device
            self.stamps.append(time.perf_counter())
        return self.layers[0](input_ids)


def time_reference_trainer(acts: torch.Tensor, *, num_latents: int, k: int, warmup_steps: int,
                           auxk_alpha: float = 1 / 32, threads: int | None = None, triton: bool = False) -> dict:
    """Runs the reference's own `Trainer.fit()` (sparsify/trainer.py:237-596: hook, forward,
    backward, decoder normalisation and projection, torch.optim.Adam, schedule, dead-latent
    bookkeeping) over acts [steps, B, T, D] - on the host (fp32 tensors on the CPU) or, for a
    same-box GPU figure, on the device the activations live on (the reference then runs its
    bf16 autocast forward and, with triton=True, its Triton decoder) - and returns the seconds
    of every step after the first `warmup_steps`, measured between consecutive step starts
    (after a device synchronisation for CUDA activations) and the end of the last step (the
    checkpoint fit() would write afterwards is skipped)."""
    sparsify = import_reference(triton=triton)
    from sparsify import SparseCoderConfig, TrainConfig, Trainer
    if threads:
        torch.set_num_threads(threads)
    steps, B, T, D = acts.shape
    model = StoredActivations(acts)
    dataset = [{"input_ids": torch.zeros(T, dtype=torch.long)} for _ in range(steps * B)]
    with tempfile.TemporaryDirectory() as tmp:
        cfg = TrainConfig(SparseCoderConfig(num_latents=num_latents, k=k), batch_size=B, optimizer="adam",
                          auxk_alpha=auxk_alpha, hookpoints=["layers.0"], log_to_wandb=False, save_dir=tmp,
                          run_name="timed", save_every=10 ** 9)
        trainer = Trainer(cfg, dataset, model)
        done = []
        # fit() ends by writing a checkpoint (weights and optimiser state: gigabytes at full width);
        # that write is not part of a step, so this instance records the time instead of saving
        def finished():
            if acts.is_cuda:
                torch.cuda.synchronize(acts.device)
            done.append(time.perf_counter())
        trainer.save = finished
        trainer.fit()
    stamps = model.stamps + done[:1]
    per_step = [b - a for a, b in zip(stamps[:-1], stamps[1:])]
    assert len(per_step) == steps, (len(per_step), steps)
    return {"seconds": per_step[warmup_steps:], "threads": torch.get_num_threads(),
            "version": getattr(sparsify, "__version__", "unknown")}
