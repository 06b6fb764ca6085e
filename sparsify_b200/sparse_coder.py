"""SparseCoder with the reference's surface (sparsify/sparse_coder.py:38-299):
same parameters (`encoder.weight`, `encoder.bias`, `W_dec`, `b_dec`, `W_skip`),
`encode` / `decode` / `forward`, the `sae.safetensors` + `cfg.json` checkpoint
layout, and the decoder-norm utilities - computed by the CUDA kernels of
libsparsecoder instead of eager PyTorch / Triton.

Precision. The reference runs `forward` under a CUDA bf16 autocast
(sparsify/sparse_coder.py:205-209) with fp32 parameters. Here the attribute
`precision` selects:
  "bf16"  encoder GEMM on bf16 copies of x and W_enc (tensor cores, fp32
          accumulate) and bf16 copies of W_dec / W_enc for the row gathers;
  "mixed" bf16 encoder GEMM, fp32 rows for the gathers (what autocast does);
  "fp32"  everything in fp32 (what the reference computes on CPU).
The bf16 copies ("shadows") are cached per parameter and re-cast only when the
parameter's version counter has moved.
"""

from __future__ import annotations

import json
import re
from fnmatch import fnmatch
from pathlib import Path
from typing import NamedTuple

import torch
from safetensors import safe_open
from safetensors.torch import load_model, save_model
from torch import Tensor, nn

from . import ops
from .config import SparseCoderConfig
from .dense import linear_nt
from .fused_encoder import EncoderOutput, FusedEncoder, fused_encoder
from .fused_step import FusedSaeStep, fused_supported
from .utils import decoder_impl


def natsorted(seq, key=None):
    """Natural sort (digit runs compare as numbers), as natsort.natsorted does
    for the hookpoint names the reference sorts (sparsify/trainer.py:48)."""
    def split(s):
        return [int(t) if t.isdigit() else t for t in re.split(r"(\d+)", str(s))]
    return sorted(seq, key=(lambda v: split(key(v))) if key else split)


class ForwardOutput(NamedTuple):
    sae_out: Tensor

    latent_acts: Tensor
    """Activations of the top-k latents."""

    latent_indices: Tensor
    """Indices of the top-k features."""

    fvu: Tensor
    """Fraction of variance unexplained."""

    auxk_loss: Tensor
    """AuxK loss, if applicable."""

    multi_topk_fvu: Tensor
    """Multi-TopK FVU, if applicable."""


class SparseCoder(nn.Module):
    default_precision = "bf16"
    """Precision new instances start with ("bf16", "mixed" or "fp32")."""

    def __init__(
        self,
        d_in: int,
        cfg: SparseCoderConfig,
        device: str | torch.device = "cpu",
        dtype: torch.dtype | None = None,
        *,
        decoder: bool = True,
    ):
        super().__init__()
        self.cfg = cfg
        self.d_in = d_in
        self.num_latents = cfg.num_latents or d_in * cfg.expansion_factor
        self.precision = type(self).default_precision
        self.fused = True  # use the single-function training path when it applies
        self.defer_weight_update = False  # set by FusedAdam.enable_sparse_update
        self._pending: dict | None = None  # weight gradients in sparse form, awaiting the optimiser
        self._dec_unit_norm: tuple | None = None  # (data_ptr, version) at which W_dec rows had unit norm
        self._dec_event = None  # completion of a decoder update running on a side stream
        self._dec_work = None  # asynchronous all-gather of the decoder's bf16 copy
        self._enc_work = None  # the same for the encoder's copy
        self._shadows: dict[str, tuple[int, int, Tensor]] = {}

        self.encoder = nn.Linear(d_in, self.num_latents, device=device, dtype=dtype)
        self.encoder.bias.data.zero_()

        if decoder:
            if cfg.transcode:
                # transcoder: decoder starts at zero (sparsify/sparse_coder.py:57-59)
                self.W_dec = nn.Parameter(torch.zeros_like(self.encoder.weight.data))
            else:
                # autoencoder: decoder starts as the (row-normalised) encoder
                self.W_dec = nn.Parameter(self.encoder.weight.data.clone())
                if self.cfg.normalize_decoder:
                    self.set_decoder_norm_to_unit_norm()
        else:
            self.W_dec = None

        self.b_dec = nn.Parameter(torch.zeros(d_in, dtype=dtype, device=device))
        self.W_skip = (
            nn.Parameter(torch.zeros(d_in, d_in, device=device, dtype=dtype))
            if cfg.skip_connection
            else None
        )

    # ------------------------------------------------------------------ loading
    @staticmethod
    def load_many(
        name: str,
        local: bool = False,
        layers: list[str] | None = None,
        device: str | torch.device = "cpu",
        *,
        decoder: bool = True,
        pattern: str | None = None,
    ) -> dict[str, "SparseCoder"]:
        """Load sparse coders for several hookpoints from one directory tree."""
        pattern = pattern + "/*" if pattern is not None else None
        if not local:
            raise NotImplementedError(
                "Downloading from the HuggingFace Hub is outside this package; "
                "fetch the repository yourself and pass local=True."
            )
        repo_path = Path(name)
        if layers is not None:
            return {
                layer: SparseCoder.load_from_disk(repo_path / layer, device=device, decoder=decoder)
                for layer in natsorted(layers)
            }
        files = [
            f for f in repo_path.iterdir()
            if f.is_dir() and (pattern is None or fnmatch(f.name, pattern))
        ]
        return {
            f.name: SparseCoder.load_from_disk(f, device=device, decoder=decoder)
            for f in natsorted(files, key=lambda f: f.name)
        }

    @staticmethod
    def load_from_disk(
        path: Path | str,
        device: str | torch.device = "cpu",
        *,
        decoder: bool = True,
    ) -> "SparseCoder":
        path = Path(path)
        with open(path / "cfg.json", "r") as f:
            cfg_dict = json.load(f)
            d_in = cfg_dict.pop("d_in")
            cfg = SparseCoderConfig.from_dict(cfg_dict, drop_extra_fields=True)

        safetensors_path = str(path / "sae.safetensors")
        with safe_open(safetensors_path, framework="pt", device="cpu") as f:
            first_key = next(iter(f.keys()))
            reference_dtype = f.get_tensor(first_key).dtype

        sae = SparseCoder(d_in, cfg, device=device, decoder=decoder, dtype=reference_dtype)
        load_model(model=sae, filename=safetensors_path, device=str(device), strict=decoder)
        return sae

    def save_to_disk(self, path: Path | str):
        self.wait_decoder()
        path = Path(path)
        path.mkdir(parents=True, exist_ok=True)
        save_model(self, str(path / "sae.safetensors"))
        with open(path / "cfg.json", "w") as f:
            json.dump({**self.cfg.to_dict(), "d_in": self.d_in}, f)

    @property
    def device(self):
        return self.encoder.weight.device

    @property
    def dtype(self):
        return self.encoder.weight.dtype

    # ------------------------------------------------------------------ shadows
    def shadow(self, name: str) -> Tensor | None:
        """bf16 copy of parameter `name` ("encoder.weight" or "W_dec"), re-cast
        when the parameter was modified in place since the copy was made."""
        p = self.encoder.weight if name == "encoder.weight" else getattr(self, name)
        if p is None:
            return None
        if name == "encoder.weight":
            self.wait_encoder()
        if p.dtype == torch.bfloat16:
            return p.detach()
        hit = self._shadows.get(name)
        if hit is not None and hit[0] == p.data_ptr() and hit[1] == p._version:
            return hit[2]
        buf = hit[2] if hit is not None and hit[2].shape == p.shape and hit[2].device == p.device else None
        buf = ops.cast_bf16(p.detach().contiguous(), buf)
        self._shadows[name] = (p.data_ptr(), p._version, buf)
        return buf

    def mark_shadow_fresh(self, name: str, buf: Tensor) -> None:
        """Records that `buf` holds the bf16 image of the parameter's current
        value (a fused update kernel wrote both)."""
        p = self.encoder.weight if name == "encoder.weight" else getattr(self, name)
        self._shadows[name] = (p.data_ptr(), p._version, buf)

    def _lowp(self) -> bool:
        return self.precision in ("bf16", "mixed") and self.dtype == torch.float32 or self.dtype == torch.bfloat16

    # ------------------------------------------------------------------ compute
    def encode(self, x: Tensor, *, need_pre_acts: bool = True) -> EncoderOutput:
        """Encode the input and select the top-k latents."""
        return self._encode(x, need_pre_acts, 0)[0]

    def _encode(self, x: Tensor, need_pre_acts: bool, wide_k: int):
        """encode() that can also return the top-`wide_k` set (see FusedEncoder)."""
        if not self.cfg.transcode:
            x = x - self.b_dec
        lowp = self._lowp()
        if lowp:
            w_lp = self.shadow("encoder.weight")
        else:
            w_lp = None
            x = x.to(torch.float32)
        res = FusedEncoder.apply(x, self.encoder.weight, self.encoder.bias, self.cfg.k, self.cfg.activation,
                                 need_pre_acts, w_lp, wide_k)
        return EncoderOutput(*res[:3]), res[3], res[4]

    def decode(self, top_acts: Tensor, top_indices: Tensor) -> Tensor:
        assert self.W_dec is not None, "Decoder weight was not initialized."
        self.wait_decoder()
        w_lp = self.shadow("W_dec") if (self.precision == "bf16" and self.dtype == torch.float32) else None
        y = decoder_impl(top_indices, top_acts.to(self.dtype), self.W_dec.mT, w_lp)
        return y + self.b_dec

    def forward(
        self, x: Tensor, y: Tensor | None = None, *, dead_mask: Tensor | None = None
    ) -> ForwardOutput:
        num_dead = self._count_dead(dead_mask)
        if self.fused and fused_supported(self, x, num_dead):
            sae_out, top_acts, top_indices, fvu, auxk_loss, multi_topk_fvu = FusedSaeStep.apply(
                x, y, self.encoder.weight, self.encoder.bias, self.W_dec, self.b_dec, self, dead_mask, num_dead,
                self.W_skip)
            return ForwardOutput(sae_out, top_acts, top_indices, fvu, auxk_loss, multi_topk_fvu)
        # Multi-TopK alone needs no dense pre-activations: the encoder kernel selects
        # the top 4k once and the top k is its leading part.
        wide_k = 4 * self.cfg.k if self.cfg.multi_topk and self.cfg.activation == "topk" else 0
        wide_on_chip = (wide_k > 0 and num_dead == 0 and self._lowp() and x.is_cuda
                        and ops.tc_encode_supported(self.d_in, self.num_latents, wide_k))
        need_dense = (self.cfg.multi_topk and not wide_on_chip) or num_dead > 0
        (top_acts, top_indices, pre_acts), wide_acts, wide_indices = self._encode(x, need_dense, wide_k)

        # If we aren't given a distinct target, we're autoencoding
        if y is None:
            y = x
        y = y.to(torch.float32)

        sae_out = self.decode(top_acts, top_indices)
        if self.W_skip is not None:
            D = self.d_in
            if self._lowp() and x.is_cuda and D % 8 == 0:
                sae_out = sae_out + linear_nt(x, self.W_skip)  # tensor-core GEMM, bf16 operands
            else:
                sae_out += x.to(self.dtype) @ self.W_skip.mT

        e = y - sae_out

        # Used as a denominator for putting everything on a reasonable scale
        total_variance = ops.total_variance(y.detach())

        if num_dead > 0:
            # Heuristic from Appendix B.1 of the TopK SAE paper, as in the reference
            k_aux = y.shape[-1] // 2
            scale = min(num_dead / k_aux, 1.0)
            k_aux = min(k_aux, num_dead)

            # top-k_aux among dead latents only; no gradient reaches the encoder
            auxk_acts, auxk_indices = ops.topk_rows(pre_acts, k_aux, col_mask=dead_mask)

            e_hat = self.decode(auxk_acts, auxk_indices)
            auxk_loss = (e_hat - e.detach()).pow(2).sum()
            auxk_loss = scale * auxk_loss / total_variance
        else:
            auxk_loss = sae_out.new_zeros(())  # filled on the device: no host round trip

        l2_loss = e.pow(2).sum()
        fvu = l2_loss / total_variance

        if self.cfg.multi_topk:
            if wide_k > 0:
                top_acts, top_indices = wide_acts, wide_indices
            else:
                top_acts, top_indices = ops.topk_rows(pre_acts, 4 * self.cfg.k)
            sae_out = self.decode(top_acts, top_indices)
            multi_topk_fvu = (sae_out - y).pow(2).sum() / total_variance
        else:
            multi_topk_fvu = sae_out.new_zeros(())

        return ForwardOutput(sae_out, top_acts, top_indices, fvu, auxk_loss, multi_topk_fvu)

    # ------------------------------------------------------------------ dead latents
    def prepare_dead_mask(self, dead_mask: Tensor | None) -> Tensor | None:
        """Reads the dead latents of `dead_mask` back once (their indices, hence their
        number) and remembers them for the forward call that receives this very tensor.
        A caller that knows the mask ahead of time - the Trainer, at the end of the
        previous step, where it reads its metrics anyway - calls this there, and the
        forward pass then runs without any device read-back."""
        if dead_mask is None:
            self._dead_cache = None
            return None
        dead_idx = dead_mask.nonzero().squeeze(1)
        self._dead_cache = (dead_mask, int(dead_idx.numel()), dead_idx)
        return dead_mask

    def _count_dead(self, dead_mask: Tensor | None) -> int:
        if dead_mask is None:
            return 0
        cache = getattr(self, "_dead_cache", None)
        if cache is not None and cache[0] is dead_mask:
            return cache[1]
        return int(dead_mask.sum())

    def dead_indices(self, dead_mask: Tensor) -> Tensor:
        cache = getattr(self, "_dead_cache", None)
        if cache is not None and cache[0] is dead_mask:
            return cache[2]
        return dead_mask.nonzero().squeeze(1)

    # ------------------------------------------------------------------ decoder norm
    @torch.no_grad()
    def set_decoder_norm_to_unit_norm(self):
        assert self.W_dec is not None, "Decoder weight was not initialized."
        eps = torch.finfo(self.W_dec.dtype).eps
        W = self.W_dec.data
        if self._dec_unit_norm == (W.data_ptr(), self.W_dec._version):
            return  # the last fused update already left the rows at unit norm
        self.wait_decoder()
        if W.is_cuda and W.dtype == torch.float32 and W.is_contiguous():
            # the kernel writes through raw pointers (no version bump): refresh the
            # cached bf16 copy in the same pass, or drop it
            hit = self._shadows.pop("W_dec", None)
            buf = hit[2] if hit is not None and hit[2].shape == W.shape and hit[2].device == W.device else None
            ops.normalize_rows_(W, eps, buf)
            torch.autograd.graph.increment_version(self.W_dec)
            if buf is not None:
                self.mark_shadow_fresh("W_dec", buf)
            self._dec_unit_norm = (W.data_ptr(), self.W_dec._version)
        else:
            # construction / checkpoint handling on the host before .to("cuda")
            norm = torch.norm(W, dim=1, keepdim=True)
            self.W_dec.data /= norm + eps

    def wait_encoder(self) -> None:
        """Makes the current stream wait for the all-gather of the encoder's bf16
        copy that a sharded update left in flight."""
        work, self._enc_work = getattr(self, "_enc_work", None), None
        if work is not None:
            with ops.span("x_wait_encoder_copy", self.device):
                work.wait()
            self._enc_work_src = None

    def wait_decoder(self) -> None:
        """Makes the current stream wait for decoder work that FusedAdam left in
        flight (an update on its side stream with `overlap_decoder`, the
        all-gather of the bf16 copy in sharded mode). Call before reading `W_dec`
        or its bf16 copy outside this package's own methods."""
        event, self._dec_event = self._dec_event, None
        if event is not None:
            torch.cuda.current_stream(self.device).wait_event(event)
        work, self._dec_work = self._dec_work, None
        if work is not None:
            with ops.span("x_wait_decoder_copy", self.device):
                work.wait()  # asynchronous all-gather of the decoder's bf16 copy (sharded update)

    def materialize_pending(self) -> None:
        """Turns a deferred sparse weight gradient into dense .grad tensors
        (accumulating), for consumers that need them."""
        pend, self._pending = self._pending, None
        if pend is None:
            return
        M, D = self.encoder.weight.shape
        res = ops.rows_accumulate(pend["row_ptr"], pend["entries"], pend["k"], M, D, pend["coefA"],
                                  pend["vecA"], coefB=pend["coefB"], vecB=pend["vecB"])
        if pend.get("extra") is not None:
            res["gradA"].index_add_(0, pend["extra"][0], pend["extra"][1])
        for p, g in ((self.W_dec, res["gradA"]), (self.encoder.weight, res["gradB"])):
            p.grad = g if p.grad is None else p.grad + g

    def attach_optimizer(self, opt, project: bool = True) -> None:
        """Lets an optimiser of this package keep the bf16 copies current inside
        its update kernel and (project=True) fold the decoder-gradient
        projection into the same pass."""
        lowp = self._lowp() and self.dtype == torch.float32
        names = ["encoder.weight"] + (["W_dec"] if self.precision == "bf16" and self.W_dec is not None else [])
        if lowp and self.device.type == "cuda":
            for name in names:
                p = self.encoder.weight if name == "encoder.weight" else self.W_dec
                buf = self.shadow(name)
                opt.register_shadow(p, buf, lambda name=name, buf=buf: self.mark_shadow_fresh(name, buf))
        if project and self.W_dec is not None and self.cfg.normalize_decoder and not self.cfg.transcode:
            opt.project_rows(self.W_dec)

    @torch.no_grad()
    def remove_gradient_parallel_to_decoder_directions(self):
        assert self.W_dec is not None, "Decoder weight was not initialized."
        assert self.W_dec.grad is not None
        g, w = self.W_dec.grad, self.W_dec.data
        if not (g.is_contiguous() and w.is_contiguous() and g.dtype == torch.float32):
            raise RuntimeError("remove_gradient_parallel_to_decoder_directions: contiguous fp32 tensors only")
        ops.project_rows_(g, w)  # raises for tensors that are not on a CUDA device: no CPU path


# Allow for alternate naming conventions
Sae = SparseCoder
