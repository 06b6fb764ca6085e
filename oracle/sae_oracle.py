"""CPU oracle for the TopK sparse-coder training step. TEST INFRASTRUCTURE ONLY.

This file restates, with explicit formulas on CPU tensors and hand-written
gradients (no autograd), the arithmetic of EleutherAI/sparsify v1.3.0 on the
path the CUDA library accelerates. Only `tests/`, `__graft_entry__.smoke()` and
`bench.py`'s CPU-baseline / `--impl reference` legs may import it; nothing in
`sparsify_b200/` does, and the product never falls back to it.

Pinning. The reference's own tests hold no stored known answers for this path
(both are differential: sparsify tests/test_encode.py, tests/test_decode.py).
The oracle is therefore pinned against outputs of the reference itself: the
script `tests/golden/make_golden.py` imports the reference and freezes its
results on seeded inputs into `tests/golden/*.safetensors`, and
`tests/test_oracle_golden.py` checks every function below against them.

Each function cites the reference lines it follows.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
from torch import Tensor


# ----------------------------------------------------------------------------- encoder
def preacts(x: Tensor, W: Tensor, b: Tensor | None) -> Tensor:
    """relu(x W^T + b)  -- sparsify/fused_encoder.py:29."""
    out = x @ W.T
    if b is not None:
        out = out + b
    return out.clamp_min(0)


def topk(pre: Tensor, k: int) -> tuple[Tensor, Tensor]:
    """Largest k entries of each row -- sparsify/fused_encoder.py:33."""
    vals, idx = torch.topk(pre, k, dim=-1, sorted=True)
    return vals, idx


def groupmax(pre: Tensor, k: int) -> tuple[Tensor, Tensor]:
    """Max inside each of k contiguous groups -- sparsify/fused_encoder.py:34-43."""
    N, M = pre.shape
    g = M // k
    vals, local = pre.reshape(N, k, g).max(dim=-1)
    idx = local + torch.arange(0, M, g).unsqueeze(0)
    return vals, idx


def encoder_forward(x, W, b, k, activation="topk"):
    pre = preacts(x, W, b)
    if activation == "topk":
        vals, idx = topk(pre, k)
    elif activation == "groupmax":
        vals, idx = groupmax(pre, k)
    else:
        raise ValueError(f"Unknown activation: {activation}")
    return vals, idx, pre


def encoder_backward(x: Tensor, W: Tensor, idx: Tensor, grad_vals: Tensor):
    """Gradients of the selected activations -- sparsify/fused_encoder.py:52-87.
    Returns (grad_x, grad_W, grad_b). The ReLU mask is not applied (the
    reference does not apply it either) and grad_preacts is ignored."""
    N, k = idx.shape
    M, D = W.shape
    gx = torch.zeros(N, D, dtype=W.dtype)
    for j in range(k):
        gx += grad_vals[:, j : j + 1] * W[idx[:, j]]
    gW = torch.zeros(M, D, dtype=W.dtype)
    contrib = grad_vals.unsqueeze(2) * x.unsqueeze(1)  # [N,k,D]
    gW.index_add_(0, idx.reshape(-1), contrib.reshape(-1, D))
    gb = torch.zeros(M, dtype=W.dtype)
    gb.index_add_(0, idx.reshape(-1), grad_vals.reshape(-1))
    return gx, gW, gb


# ----------------------------------------------------------------------------- decoder
def decode(idx: Tensor, acts: Tensor, W_dec: Tensor, b_dec: Tensor | None = None) -> Tensor:
    """sum_j acts[n,j] W_dec[idx[n,j]] (+ b_dec), ascending j, --
    sparsify/xformers.py:9-30, sparsify/utils.py:82-85, sparse_coder.py:198-202."""
    N, k = idx.shape
    out = torch.zeros(N, W_dec.shape[1], dtype=W_dec.dtype)
    for j in range(k):
        out += acts[:, j : j + 1] * W_dec[idx[:, j]]
    if b_dec is not None:
        out = out + b_dec
    return out


def decode_backward(idx: Tensor, acts: Tensor, W_dec: Tensor, grad_out: Tensor):
    """(grad_W_dec, grad_acts) -- sparsify/xformers.py:88-136."""
    N, k = idx.shape
    M, D = W_dec.shape
    gW = torch.zeros(M, D, dtype=W_dec.dtype)
    contrib = acts.unsqueeze(2) * grad_out.unsqueeze(1)
    gW.index_add_(0, idx.reshape(-1), contrib.reshape(-1, D))
    gacts = torch.empty(N, k, dtype=W_dec.dtype)
    for j in range(k):
        gacts[:, j] = (grad_out * W_dec[idx[:, j]]).sum(-1)
    return gW, gacts


def csr_by_latent(idx: Tensor, M: int):
    """Latent-major CSR with ascending flat positions -- the structure
    sparsify/xformers.py:146-163 builds (there in arbitrary intra-latent order)."""
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=M)
    row_ptr = torch.zeros(M + 1, dtype=torch.int64)
    row_ptr[1:] = torch.cumsum(counts, 0)
    return row_ptr, order


# ----------------------------------------------------------------------------- model
@dataclass
class OracleCfg:
    k: int = 32
    activation: str = "topk"
    normalize_decoder: bool = True
    multi_topk: bool = False
    skip_connection: bool = False
    transcode: bool = False


@dataclass
class ForwardResult:
    sae_out: Tensor
    latent_acts: Tensor
    latent_indices: Tensor
    fvu: Tensor
    auxk_loss: Tensor
    multi_topk_fvu: Tensor
    grads: dict = field(default_factory=dict)


def normalize_decoder_(W_dec: Tensor) -> None:
    """sparsify/sparse_coder.py:273-279."""
    eps = torch.finfo(W_dec.dtype).eps
    W_dec /= W_dec.norm(dim=1, keepdim=True) + eps


def project_out_parallel_(grad: Tensor, W_dec: Tensor) -> None:
    """sparsify/sparse_coder.py:281-295."""
    par = (grad * W_dec).sum(1, keepdim=True)
    grad -= par * W_dec


def sae_forward_backward(
    params: dict,
    x: Tensor,
    y: Tensor | None = None,
    dead_mask: Tensor | None = None,
    cfg: OracleCfg = OracleCfg(),
    auxk_alpha: float = 0.0,
    loss_scale: float = 1.0,
    round_operands=None,
) -> ForwardResult:
    """SparseCoder.forward (sparsify/sparse_coder.py:205-271) and the gradients
    of loss = (fvu + auxk_alpha*auxk + multi_topk_fvu/8) * loss_scale
    (sparsify/trainer.py:444-447) with respect to every parameter.

    params: {"W_enc" [M,D], "b_enc" [M], "W_dec" [M,D], "b_dec" [D], "W_skip" [D,D] or absent}.
    round_operands: optional callable applied to the operands of the encoder
    GEMM and to the rows that are gathered (e.g. a bf16 round trip), to state the
    reduced-precision configurations with the same formulas."""
    rnd = round_operands or (lambda t: t)
    W_enc, b_enc, W_dec, b_dec = params["W_enc"], params["b_enc"], params["W_dec"], params["b_dec"]
    W_skip = params.get("W_skip")
    M, D = W_enc.shape
    N = x.shape[0]
    if y is None:
        y = x
    xe = x if cfg.transcode else x - b_dec                     # sparse_coder.py:191-192
    xe_r, W_enc_r, W_dec_r = rnd(xe), rnd(W_enc), rnd(W_dec)
    acts, idx, pre = encoder_forward(xe_r, W_enc_r, b_enc, cfg.k, cfg.activation)
    out = decode(idx, acts, W_dec_r, b_dec)                    # sparse_coder.py:216
    if W_skip is not None:
        out = out + x @ W_skip.T                               # sparse_coder.py:221-222
    e = y - out                                                # :225
    tv = (y - y.mean(0)).pow(2).sum()                          # :228
    fvu = e.pow(2).sum() / tv                                  # :253-254

    grads = {n: torch.zeros_like(p) for n, p in params.items()}
    # d fvu / d out
    g_out = (-2.0 * loss_scale / tv) * e
    gWd, g_acts = decode_backward(idx, acts, W_dec_r, g_out)
    grads["W_dec"] += gWd
    grads["b_dec"] += g_out.sum(0)
    if W_skip is not None:
        grads["W_skip"] += g_out.T @ x
    gx, gWe, gbe = encoder_backward(xe_r, W_enc_r, idx, g_acts)
    grads["W_enc"] += gWe
    grads["b_enc"] += gbe
    if not cfg.transcode:
        grads["b_dec"] -= gx.sum(0)                            # through x - b_dec

    auxk = torch.zeros(())
    num_dead = int(dead_mask.sum()) if dead_mask is not None else 0
    if num_dead > 0:                                           # :231-249
        k_aux = y.shape[-1] // 2
        scale = min(num_dead / k_aux, 1.0)
        k_aux = min(k_aux, num_dead)
        masked = torch.where(dead_mask[None], pre, torch.full_like(pre, -math.inf))
        a_acts, a_idx = torch.topk(masked, k_aux, sorted=True)
        e_hat = decode(a_idx, a_acts, W_dec_r, b_dec)
        diff = e_hat - e
        auxk = scale * diff.pow(2).sum() / tv
        g_ehat = (2.0 * scale * auxk_alpha * loss_scale / tv) * diff
        gWd2, _ = decode_backward(a_idx, a_acts, W_dec_r, g_ehat)  # encoder gets no gradient
        grads["W_dec"] += gWd2
        grads["b_dec"] += g_ehat.sum(0)

    multi = torch.zeros(())
    out_acts, out_idx, sae_out = acts, idx, out
    if cfg.multi_topk:                                         # :256-262
        m_acts, m_idx = torch.topk(pre, 4 * cfg.k, sorted=True)
        m_out = decode(m_idx, m_acts, W_dec_r, b_dec)
        diff = m_out - y
        multi = diff.pow(2).sum() / tv
        g_m = (2.0 * loss_scale / 8.0 / tv) * diff
        gWd3, _ = decode_backward(m_idx, m_acts, W_dec_r, g_m)
        grads["W_dec"] += gWd3
        grads["b_dec"] += g_m.sum(0)
        out_acts, out_idx, sae_out = m_acts, m_idx, m_out

    return ForwardResult(sae_out, out_acts, out_idx, fvu, auxk, multi, grads)


# ----------------------------------------------------------------------------- optimiser
def adam_step_(p: Tensor, g: Tensor, m: Tensor, v: Tensor, step: int, lr: float,
               beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8) -> None:
    """torch.optim.Adam defaults (sparsify/trainer.py:99-116), `step` 1-based."""
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = v.sqrt() / math.sqrt(bc2) + eps
    p.addcdiv_(m, denom, value=-lr / bc1)


def linear_warmup_lr(base_lr: float, step: int, warmup: int, total: int) -> float:
    """transformers.get_linear_schedule_with_warmup as used at
    sparsify/trainer.py:117-121; `step` is the number of scheduler steps taken."""
    if step < warmup:
        return base_lr * step / max(1, warmup)
    return base_lr * max(0.0, (total - step) / max(1, total - warmup))


def default_adam_lr(num_latents: int) -> float:
    """sparsify/trainer.py:109."""
    return 2e-4 / (num_latents / (2 ** 14)) ** 0.5


def quintic_newtonschulz(G: Tensor, steps: int = 5) -> Tensor:
    """sparsify/muon.py:11-40, with bf16 rounding of every product."""
    a, b, c = (3.4445, -4.7750, 2.0315)
    X = G.bfloat16()
    transposed = G.size(-2) > G.size(-1)
    if transposed:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        A = X @ X.mT
        B = b * A + c * A @ A
        X = a * X + B @ X
    if transposed:
        X = X.mT
    return X



# ----------------------------------------------------------------------------- signum
def default_signum_lr(num_latents: int) -> float:
    """sparsify/trainer.py:152: lr = 5e-3 / sqrt(num_latents / 2**14)."""
    return 5e-3 / (num_latents / 2 ** 14) ** 0.5


def sign_sgd_step_(p: Tensor, g: Tensor, lr: float) -> None:
    """sparsify/sign_sgd.py:18-26."""
    p.add_(g.sign(), alpha=-lr)


class ScheduleFreeWrapperPort:
    """Restatement of ``schedulefree.ScheduleFreeWrapper`` (third-party package
    "schedulefree", facebookresearch/schedule_free; the reference lists it
    unpinned in pyproject.toml and it is not available offline, so this follows
    the published algorithm of Defazio et al. 2024, "The Road Less Scheduled",
    in the wrapper form the reference calls at sparsify/trainer.py:158-159,
    652-654,675-677). PARITY UNPINNED for this class: there is no copy of the
    package to check it against; SignSGD, the learning-rate rule and the
    Trainer's use of train()/eval() are the reference's own code.

    The wrapped optimiser's parameters hold y while training; state z is the
    base optimiser's iterate; x = y + (1 - 1/beta)(z - y) is the average.
    """

    def __init__(self, base, weight_decay_at_y: float = 0.0, momentum: float = 0.9,
                 weight_lr_power: float = 2.0, r: float = 0.0):
        self.base = base
        self.state: dict = {}
        for group in self.param_groups:
            group.update(weight_decay_at_y=weight_decay_at_y, momentum=momentum,
                         weight_lr_power=weight_lr_power, r=r, k=0, lr_max=-1.0, weight_sum=0.0,
                         train_mode=False)

    @property
    def param_groups(self):
        return self.base.param_groups

    def zero_grad(self, set_to_none: bool = True):
        return self.base.zero_grad(set_to_none)

    def state_dict(self):
        return {"z": [self.state[p]["z"] for g in self.param_groups for p in g["params"] if p in self.state],
                "groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    @torch.no_grad()
    def eval(self):
        for group in self.param_groups:
            if group["train_mode"]:
                for p in group["params"]:
                    if p in self.state:
                        p.lerp_(end=self.state[p]["z"], weight=1 - 1 / group["momentum"])  # y -> x
                group["train_mode"] = False

    @torch.no_grad()
    def train(self):
        for group in self.param_groups:
            if not group["train_mode"]:
                for p in group["params"]:
                    if p in self.state:
                        p.lerp_(end=self.state[p]["z"], weight=1 - group["momentum"])      # x -> y
                group["train_mode"] = True

    @torch.no_grad()
    def step(self, closure=None):
        assert closure is None
        for group in self.param_groups:
            assert group["train_mode"], "call .train() first"
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state.setdefault(p, {})
                if "z" not in st:
                    st["z"] = p.detach().clone()
                z = st["z"]
                if group["weight_decay_at_y"] != 0.0:
                    wd = group["lr"] * group["weight_decay_at_y"]
                    z.sub_(p, alpha=wd)
                    p.sub_(p, alpha=wd * (1 - group["momentum"]))
                p.lerp_(end=z, weight=1 - 1 / group["momentum"])       # y -> x
                tmp = p.detach().clone()                                # p <- z, z-buffer <- x
                p.copy_(z)
                z.copy_(tmp)
        self.base.step()                                                # the wrapped step acts on z
        for group in self.param_groups:
            k, lr = group["k"], group["lr"]
            lr_max = group["lr_max"] = max(lr, group["lr_max"])
            weight = ((k + 1) ** group["r"]) * (lr_max ** group["weight_lr_power"])
            weight_sum = group["weight_sum"] = group["weight_sum"] + weight
            ckp1 = weight / weight_sum if weight_sum != 0 else 0.0
            for p in group["params"]:
                if p.grad is None:
                    continue
                z = self.state[p]["z"]
                tmp = p.detach().clone()                                # p <- x, z-buffer <- new z
                p.copy_(z)
                z.copy_(tmp)
                p.lerp_(end=z, weight=ckp1)                             # x <- x + c (z - x)
                p.lerp_(end=z, weight=1 - group["momentum"])            # y
            group["k"] = k + 1


def signum_schedulefree_step_(y: Tensor, z: Tensor, g: Tensor, lr: float, momentum: float, ckp1: float) -> None:
    """One step of ScheduleFreeWrapperPort(SignSGD) on a single tensor, in place on (y, z)."""
    x = torch.lerp(y, z, 1 - 1 / momentum)
    sign_sgd_step_(z, g, lr)
    x.lerp_(z, ckp1)
    y.copy_(torch.lerp(x, z, 1 - momentum))


class OracleTrainer:
    """One SAE trained the way sparsify/trainer.py:340-447,510-538 does it with
    loss_fn="fvu" and Adam: step-0 b_dec init, decoder normalisation before each
    forward, gradient projection before each optimiser step, linear warmup,
    dead-latent bookkeeping."""

    def __init__(self, params: dict, cfg: OracleCfg, *, lr: float | None = None, warmup: int = 1000,
                 total_steps: int = 1000, auxk_alpha: float = 0.0, dead_threshold: int = 10_000_000,
                 round_operands=None, optimizer: str = "adam", momentum: float = 0.95):
        self.p = params
        self.cfg = cfg
        M = params["W_enc"].shape[0]
        self.optimizer = optimizer
        self.momentum = momentum
        if optimizer == "signum":  # trainer.py:146-161: no scheduler, constant lr
            self.base_lr = lr or default_signum_lr(M)
            self.z = {n: None for n in params}
            self.weight_sum = 0.0
        else:
            self.base_lr = lr or default_adam_lr(M)
        self.warmup, self.total = warmup, total_steps
        self.auxk_alpha = auxk_alpha
        self.dead_threshold = dead_threshold
        self.m = {n: torch.zeros_like(t) for n, t in params.items()}
        self.v = {n: torch.zeros_like(t) for n, t in params.items()}
        self.global_step = 0
        self.num_tokens_since_fired = torch.zeros(M, dtype=torch.long)
        self.rnd = round_operands

    def step(self, x: Tensor, y: Tensor | None = None) -> ForwardResult:
        target = x if y is None else y
        if self.global_step == 0:
            if self.cfg.transcode:
                self.p["b_enc"].copy_(-(x.mean(0)) @ self.p["W_enc"].T)   # trainer.py:398-401
            self.p["b_dec"].copy_(target.mean(0))                          # trainer.py:403-404
        if self.cfg.normalize_decoder and not self.cfg.transcode:
            normalize_decoder_(self.p["W_dec"])                            # trainer.py:407-408
        dead = (self.num_tokens_since_fired > self.dead_threshold) if self.auxk_alpha > 0 else None
        res = sae_forward_backward(self.p, x, y, dead, self.cfg, self.auxk_alpha,
                                   round_operands=self.rnd)
        if self.cfg.normalize_decoder and not self.cfg.transcode:
            project_out_parallel_(res.grads["W_dec"], self.p["W_dec"])     # trainer.py:513-515
        if self.optimizer == "signum":
            lr = self.base_lr
            self.weight_sum += lr ** 2          # weight_lr_power=2, r=0, constant lr
            for n in self.p:
                if self.z[n] is None:
                    self.z[n] = self.p[n].clone()
                signum_schedulefree_step_(self.p[n], self.z[n], res.grads[n], lr, self.momentum,
                                          lr ** 2 / self.weight_sum)
        else:
            lr = linear_warmup_lr(self.base_lr, self.global_step, self.warmup, self.total)
            for n in self.p:
                adam_step_(self.p[n], res.grads[n], self.m[n], self.v[n], self.global_step + 1, lr)
        fired = torch.zeros_like(self.num_tokens_since_fired, dtype=torch.bool)
        fired[res.latent_indices.reshape(-1)] = True
        self.num_tokens_since_fired += x.shape[0]                          # trainer.py:529-533
        self.num_tokens_since_fired[fired] = 0
        self.global_step += 1
        return res
