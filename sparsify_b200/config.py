"""Configuration dataclasses with the reference's field names and defaults
(sparsify/config.py:8-131), serialisable to the same `cfg.json` / `config.json`
layout. `simple_parsing` is not a dependency: `Serializable` below provides
the three methods the reference's call sites use (`to_dict`, `from_dict`,
`save_json`)."""

from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from functools import partial
from typing import Literal


class Serializable:
    def to_dict(self) -> dict:
        return dataclasses.asdict(self)  # type: ignore[arg-type]

    @classmethod
    def from_dict(cls, d: dict, drop_extra_fields: bool = False):
        names = {f.name: f for f in dataclasses.fields(cls)}  # type: ignore[arg-type]
        kwargs = {}
        for key, value in d.items():
            if key not in names:
                if drop_extra_fields:
                    continue
                raise TypeError(f"{cls.__name__} has no field '{key}'")
            f = names[key]
            if isinstance(value, dict) and dataclasses.is_dataclass(_resolve(f.type)):
                value = _resolve(f.type).from_dict(value, drop_extra_fields=drop_extra_fields)
            kwargs[key] = value
        return cls(**kwargs)

    def save_json(self, path) -> None:
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=2)

    @classmethod
    def load_json(cls, path, drop_extra_fields: bool = True):
        with open(path) as f:
            return cls.from_dict(json.load(f), drop_extra_fields=drop_extra_fields)


def _resolve(tp):
    if isinstance(tp, str):
        return globals().get(tp)
    return tp


def list_field(*defaults):
    return field(default_factory=lambda: list(defaults))


@dataclass
class SparseCoderConfig(Serializable):
    """Configuration of a sparse coder (sparsify/config.py:8-39)."""

    activation: Literal["groupmax", "topk"] = "topk"
    expansion_factor: int = 32
    normalize_decoder: bool = True
    num_latents: int = 0
    k: int = 32
    multi_topk: bool = False
    skip_connection: bool = False
    transcode: bool = False


SaeConfig = SparseCoderConfig
TranscoderConfig = partial(SparseCoderConfig, transcode=True)


@dataclass
class TrainConfig(Serializable):
    """Training configuration (sparsify/config.py:47-131)."""

    sae: SparseCoderConfig

    batch_size: int = 32
    grad_acc_steps: int = 1
    micro_acc_steps: int = 1
    loss_fn: Literal["ce", "fvu", "kl"] = "fvu"
    optimizer: Literal["adam", "muon", "signum"] = "signum"
    lr: float | None = None
    lr_warmup_steps: int = 1000
    k_decay_steps: int = 0
    auxk_alpha: float = 0.0
    dead_feature_threshold: int = 10_000_000
    exclude_tokens: list[int] = list_field()
    hookpoints: list[str] = list_field()
    init_seeds: list[int] = list_field(0)
    layers: list[int] = list_field()
    layer_stride: int = 1
    distribute_modules: bool = False
    save_every: int = 1000
    save_best: bool = False
    finetune: str | None = None
    log_to_wandb: bool = True
    run_name: str | None = None
    wandb_log_frequency: int = 1
    save_dir: str = "checkpoints"

    def __post_init__(self):
        if isinstance(self.sae, dict):
            self.sae = SparseCoderConfig.from_dict(self.sae, drop_extra_fields=True)
        if self.layers and self.layer_stride != 1:
            raise ValueError("Cannot specify both `layers` and `layer_stride`.")
        if self.distribute_modules and self.loss_fn in ("ce", "kl"):
            raise ValueError(
                "Distributing modules across ranks is not compatible with the "
                "cross-entropy or KL divergence losses."
            )
        if not self.init_seeds:
            raise ValueError("Must specify at least one random seed.")
