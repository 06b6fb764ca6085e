"""Seeded synthetic activations standing in for language-model activations.

x = (sum of `active` unit-norm atoms with Exp(1) coefficients + N(0, 0.05^2)
noise) * per-dimension scale, where the scale is LogNormal(0, 0.5) with two
outlier dimensions multiplied by 20. The dictionary and the scales depend only
on (n_atoms, d, seed); each batch depends on its own seed. Generation runs on
whatever device is asked for (CPU for parity fixtures, GPU for throughput)."""

from __future__ import annotations

import torch
from torch import Tensor


class SyntheticActivations:
    def __init__(self, d: int, n_atoms: int, active: int, seed: int = 1234,
                 device: str | torch.device = "cpu"):
        self.d, self.n_atoms, self.active = d, n_atoms, active
        self.device = torch.device(device)
        g = torch.Generator(device="cpu").manual_seed(seed)
        # the dictionary is drawn in chunks so that large ones need no 2x peak
        chunks = []
        for lo in range(0, n_atoms, 65536):
            a = torch.randn(min(65536, n_atoms - lo), d, generator=g)
            chunks.append(torch.nn.functional.normalize(a, dim=1).to(self.device))
        self.atoms = torch.cat(chunks)
        scale = torch.exp(0.5 * torch.randn(d, generator=g))
        outliers = torch.randperm(d, generator=g)[:2]
        scale[outliers] *= 20
        self.scale = scale.to(self.device)

    def batch(self, n: int, seed: int, dtype: torch.dtype = torch.float32) -> Tensor:
        dev = self.device
        g = torch.Generator(device=dev).manual_seed(seed)
        ids = torch.randint(0, self.n_atoms, (n, self.active), generator=g, device=dev)
        # without replacement: redraw the rows that hold a duplicate
        for _ in range(64):
            s = ids.sort(dim=1).values
            dup = (s[:, 1:] == s[:, :-1]).any(dim=1)
            if not bool(dup.any()):
                break
            m = int(dup.sum())
            ids[dup] = torch.randint(0, self.n_atoms, (m, self.active), generator=g, device=dev)
        coef = -torch.log1p(-torch.rand(n, self.active, generator=g, device=dev))
        x = torch.zeros(n, self.d, device=dev)
        for lo in range(0, n, 2048):  # bounded gather temporaries
            hi = min(n, lo + 2048)
            x[lo:hi] = torch.einsum("nad,na->nd", self.atoms[ids[lo:hi]], coef[lo:hi])
        x += 0.05 * torch.randn(n, self.d, generator=g, device=dev)
        x *= self.scale
        return x.to(dtype)


def batch_seed(step: int, rank: int = 0, world: int = 1, hookpoint: int = 0) -> int:
    return 10_000 * hookpoint + step * world + rank
