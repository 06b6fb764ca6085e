"""Adam on the CUDA kernels, as a torch.optim.Optimizer so that the Trainer can
schedule, checkpoint and resume it exactly like the `torch.optim.Adam` the
reference constructs (sparsify/trainer.py:93-122). State keys (`step`,
`exp_avg`, `exp_avg_sq`) and hyper-parameter names match torch's, so a state
dict written by either loads into the other.

Per parameter one kernel pass does: optional removal of the gradient component
parallel to each parameter row (the reference's
`remove_gradient_parallel_to_decoder_directions`, sparse_coder.py:281-295),
the Adam update, and the refresh of a bf16 shadow copy when one is registered.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch import Tensor

from . import ops


def _touched(p: Tensor) -> None:
    """The kernels write parameters through raw pointers; this moves the tensor's
    version counter so that anything cached against it (bf16 copies, the
    unit-norm marker) is seen as out of date unless it is re-marked afterwards."""
    torch.autograd.graph.increment_version(p)


class FusedAdam(torch.optim.Optimizer):
    # torch.optim.Adam's remaining hyper-parameters at the values this optimiser implements.
    # They are stored in every parameter group so that a state dict written here has the keys
    # torch.optim.Adam.load_state_dict installs (and its step() then reads) in the reference
    # Trainer, and one written by torch.optim.Adam is checked against them when loaded here.
    _TORCH_ADAM_FIXED = dict(weight_decay=0, amsgrad=False, maximize=False, foreach=None, capturable=False,
                             differentiable=False, fused=None, decoupled_weight_decay=False)

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8):
        if lr < 0:
            raise ValueError(f"Invalid learning rate: {lr}")
        defaults = dict(lr=lr, betas=betas, eps=eps, **self._TORCH_ADAM_FIXED)
        super().__init__(params, defaults)
        self._project: set[int] = set()
        self._shadow: dict[int, tuple] = {}
        self._sparse: list = []  # coders whose weight gradients arrive in sparse form

    def load_state_dict(self, state_dict) -> None:
        """Accepts state dicts written by this class and by torch.optim.Adam (the reference
        Trainer's optimizer_0.pt, sparsify/trainer.py:219-223); refuses Adam variants this
        optimiser does not implement instead of silently ignoring them."""
        for group in state_dict["param_groups"]:
            if group.get("weight_decay", 0) != 0 or group.get("amsgrad", False) or group.get("maximize", False):
                raise ValueError("FusedAdam implements plain Adam only (weight_decay=0, amsgrad=False, maximize=False)")
        super().load_state_dict(state_dict)
        for group in self.param_groups:  # the execution-strategy flags of torch's Adam mean nothing here
            for key, val in self._TORCH_ADAM_FIXED.items():
                group[key] = val if key in ("foreach", "capturable", "differentiable", "fused") else group.get(key, val)

    def project_rows(self, p: Tensor) -> None:
        """Marks `p` (a [M, D] decoder) for gradient projection at every step."""
        self._project.add(id(p))

    def register_shadow(self, p: Tensor, shadow: Tensor, on_refresh=None) -> None:
        """`shadow` (bf16, same shape) is rewritten with the updated value of
        `p` inside the update kernel; `on_refresh()` is called afterwards."""
        self._shadow[id(p)] = (shadow, on_refresh)

    def enable_sparse_update(self, sae, data_parallel: bool = True, overlap_decoder: bool = False) -> bool:
        """Lets `sae` hand its W_enc / W_dec gradients over in sparse form (CSR +
        coefficients) so that one kernel applies them: projection, Adam, decoder
        normalisation and bf16 copies, with no dense gradient in between. Only
        for a single process without gradient accumulation: nothing else may
        need `.grad` of the two matrices. With torch.distributed initialised and
        `data_parallel` (replicas on every rank) the update is sharded over ranks;
        pass data_parallel=False for a coder that lives on one rank only.
        overlap_decoder=True runs the decoder half of the update on a second
        stream, so that it may overlap the next forward's encoder GEMM (which does
        not read W_dec); readers of W_dec inside this package wait for it, code
        that reads `sae.W_dec` directly must call `sae.wait_decoder()` first.
        (Measured on B200 at d=4096, 131072 latents: no gain - the background
        kernel slows the encoder by more than it hides; off by default.)
        Returns whether it was enabled."""
        W = sae.encoder.weight
        ok = (sae.W_dec is not None and W.is_cuda and W.dtype == torch.float32 and W.shape[1] % 4 == 0
              and W.shape[1] <= 8192)
        if ok and data_parallel and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            # Data parallel: ranks exchange the sparse factors (indices, coefficients,
            # residual and input rows) instead of dense gradients and each rank updates
            # only its slice of the latents, then the bf16 copies are all-gathered.
            ok = W.shape[0] % dist.get_world_size() == 0 and sae.precision == "bf16"
            if ok:
                sae._shard = (dist.get_rank(), dist.get_world_size())
        if ok:
            sae.defer_weight_update = True
            sae._overlap_decoder = bool(overlap_decoder) and getattr(sae, "_shard", None) is None
            sae._overlap_ctas_per_sm = int(os.environ.get("SC_OVERLAP_CTAS_PER_SM", "0"))
            self._sparse.append(sae)
        return ok

    def sync_masters(self, sae=None) -> None:
        """In sharded data-parallel mode a rank keeps the fp32 values and Adam
        moments of its own latent slice current; this all-gathers them so that
        every rank holds the full tensors again (before a checkpoint or a dense
        update)."""
        for s_ in ([sae] if sae is not None else self._sparse):
            if getattr(s_, "_shard", None) is None or not getattr(s_, "_masters_stale", False):
                continue
            rank, world = s_._shard
            for p in (s_.W_dec, s_.encoder.weight):
                rows = p.shape[0] // world
                state = self._state_for(p)
                for t in (p.data, state["exp_avg"], state["exp_avg_sq"]):
                    mine = t[rank * rows:(rank + 1) * rows].clone()
                    dist.all_gather_into_tensor(t.view(-1), mine.view(-1))
            s_._masters_stale = False

    def _group_of(self, p):
        for group in self.param_groups:
            if any(q is p for q in group["params"]):
                return group
        raise KeyError("parameter not in this optimiser")

    def _state_for(self, p):
        state = self.state[p]
        if len(state) == 0:
            state["step"] = torch.tensor(0.0, dtype=torch.float32)
            state["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        return state

    def _sparse_step(self, sae) -> None:
        pend = sae._pending
        W_enc, W_dec = sae.encoder.weight, sae.W_dec
        if W_enc.grad is not None or W_dec.grad is not None:
            sae.materialize_pending()  # dense gradients exist as well: fold and go dense
            self.sync_masters(sae)
            return
        sae._pending = None
        shard = getattr(sae, "_shard", None)
        late_vecA = None
        if shard is not None:
            # (the gathered residual rows may still be travelling: the encoder half of the update
            # does not need them, so they are waited for only in front of the decoder half)
            pend, late_vecA = self._exchange_factors(sae, pend, shard)
        hps, states = [], []
        for p in (W_dec, W_enc):
            group, state = self._group_of(p), self._state_for(p)
            state["step"] += 1
            lr = group["lr"]
            hps.append(dict(lr=float(lr), beta1=group["betas"][0], beta2=group["betas"][1],
                            eps=group["eps"], step=int(state["step"])))
            states.append(state)
        shadow_dec = self._shadow.get(id(W_dec), (None, None))
        shadow_enc = self._shadow.get(id(W_enc), (None, None))
        normalize = sae.cfg.normalize_decoder and not sae.cfg.transcode
        rows = slice(None)
        if shard is not None:
            per = W_dec.shape[0] // shard[1]
            rows = slice(shard[0] * per, (shard[0] + 1) * per)
        sl = lambda t: None if t is None else t[rows]
        kw = dict(pA=W_dec.data[rows], mA=states[0]["exp_avg"][rows], vA=states[0]["exp_avg_sq"][rows],
                  shadowA=sl(shadow_dec[0]), projectA=id(W_dec) in self._project, normalizeA=normalize,
                  norm_eps=torch.finfo(torch.float32).eps, hpA=hps[0], pB=W_enc.data[rows],
                  mB=states[1]["exp_avg"][rows], vB=states[1]["exp_avg_sq"][rows], shadowB=sl(shadow_enc[0]),
                  hpB=hps[1])
        args = (pend["row_ptr"], pend["entries"], pend["k"], pend["coefA"], pend["vecA"], pend["coefB"],
                pend["vecB"])
        extra = pend.get("extra")
        if extra is not None:
            # AuxK: dense gradient rows of the dead latents; a rank map tells the kernel which
            # latent owns which row (restricted to this rank's slice when sharded)
            dead_idx, extra_rows = extra
            if shard is not None:
                dist.all_reduce(extra_rows)  # dead sets are identical on every rank
                extra_rows /= shard[1]
            rank_map = torch.full((W_dec.shape[0],), -1, dtype=torch.int32, device=W_dec.device)
            rank_map.index_copy_(0, dead_idx, torch.arange(dead_idx.numel(), dtype=torch.int32, device=W_dec.device))
            kw.update(extraA=extra_rows, extra_rank=rank_map[rows].contiguous())
        if getattr(sae, "_overlap_decoder", False):
            # Encoder half now; decoder half on a side stream, where it can run under the
            # next forward's encoder GEMM. Consumers of W_dec wait on the recorded event.
            sae.wait_decoder()
            main = torch.cuda.current_stream(W_dec.device)
            ops.rows_adam_(*args, parts=2, **kw)
            if getattr(sae, "_side_stream", None) is None:
                sae._side_stream = torch.cuda.Stream(device=W_dec.device)
            side = sae._side_stream
            side.wait_stream(main)
            with torch.cuda.stream(side):
                # optionally a small persistent grid (SC_OVERLAP_CTAS_PER_SM > 0), which leaves
                # room on every SM for the encoder kernel launched after it
                sms = torch.cuda.get_device_properties(W_dec.device).multi_processor_count
                ops.rows_adam_(*args, parts=1, max_ctas=sms * sae._overlap_ctas_per_sm, **kw)
                event = torch.cuda.Event()
                event.record(side)
            for t in args:
                if isinstance(t, Tensor):
                    t.record_stream(side)  # allocated on the main stream, still in use on the side stream
            sae._dec_event = event
        else:
            # one launch per matrix: each then gathers from a single [N, D] bf16 array (134 MB at
            # d=4096, 16384 tokens), which L2 holds far better than both at once (-0.3 ms per step)
            ops.rows_adam_(*args, parts=2, **kw)
            if shard is not None:
                # everyone needs every row of the encoder copy for the next forward: its
                # all-gather runs while the decoder half of the update is computed
                mine = shadow_enc[0][rows].clone()
                sae._enc_work = dist.all_gather_into_tensor(shadow_enc[0].view(-1), mine.view(-1), async_op=True)
                sae._enc_work_src = mine
            if late_vecA is not None:
                args = args[:4] + (late_vecA(),) + args[5:]  # the residual rows of every rank, now needed
            ops.rows_adam_(*args, parts=1, **kw)
        if shard is not None:
            if getattr(sae, "_overlap_decoder", False):
                mine = shadow_enc[0][rows].clone()
                dist.all_gather_into_tensor(shadow_enc[0].view(-1), mine.view(-1))
            # the decoder copy is needed only at decode time: its all-gather runs under the
            # encoder GEMM of the next forward
            mine_dec = shadow_dec[0][rows].clone()
            sae.wait_decoder()
            sae._dec_work = dist.all_gather_into_tensor(shadow_dec[0].view(-1), mine_dec.view(-1), async_op=True)
            sae._dec_work_src = mine_dec  # keep the send buffer alive until the wait
            sae._masters_stale = True
        for q in (W_dec, W_enc):
            _touched(q)
        for _, cb in (shadow_dec, shadow_enc):
            if cb is not None:
                cb()
        if normalize:
            sae._dec_unit_norm = (W_dec.data_ptr(), W_dec._version)

    def _exchange_factors(self, sae, pend: dict, shard) -> dict:
        """All-gathers the sparse gradient factors of every rank and builds the CSR
        of this rank's latent slice over the concatenated tokens. Coefficients are
        divided by the world size: the result is the mean of the per-rank
        gradients, as DistributedDataParallel averages them."""
        rank, world = shard
        idx = pend["idx"].to(torch.int32)
        N, k = idx.shape
        coefA = (pend["coefA"].to(torch.float32) / world).reshape(N, k)
        coefB = (pend["coefB"].to(torch.float32) / world).reshape(N, k)
        vecA, vecB = pend["vecA"].contiguous(), pend["vecB"].contiguous()
        if getattr(sae, "ragged_tokens", False):
            # ranks may hold different token counts: pad to the maximum with inert rows
            n_max = torch.tensor([N], device=idx.device)
            dist.all_reduce(n_max, op=dist.ReduceOp.MAX)
            n_max = int(n_max)
            if n_max > N:
                pad = n_max - N
                idx = torch.cat([idx, idx.new_full((pad, k), -1)])
                coefA = torch.cat([coefA, coefA.new_zeros(pad, k)])
                coefB = torch.cat([coefB, coefB.new_zeros(pad, k)])
                vecA = torch.cat([vecA, vecA.new_zeros(pad, vecA.shape[1])])
                vecB = torch.cat([vecB, vecB.new_zeros(pad, vecB.shape[1])])
                N = n_max

        def gather(t):
            out = t.new_empty((world * t.shape[0],) + tuple(t.shape[1:]))
            dist.all_gather_into_tensor(out.view(-1), t.contiguous().view(-1))
            return out

        # the arrays may already be on their way (started by the forward and backward passes)
        early = getattr(sae, "_early", None) or {}
        sae._early = None
        dev = idx.device

        def take(name, t):
            if name in early:
                src, out, work = early[name]
                work.wait()
                if src.shape == t.shape and src.dtype == t.dtype:
                    return out
            return gather(t)

        with ops.span("x_wait_rows", dev):
            vecB_all = take("vecB", vecB)   # same order on every rank: issued first, waited first
        late = None
        if "vecA" in early and early["vecA"][0].shape == vecA.shape:
            def late():  # waited for in front of the decoder half of the update
                with ops.span("x_wait_residual_rows", dev):
                    early["vecA"][2].wait()
                return early["vecA"][1]
            vecA_all = vecA  # placeholder with a valid address: the encoder half never reads it
        else:
            vecA_all = gather(vecA)
        with ops.span("x_gather_factors", dev):
            idx_all, coefA_all, coefB_all = take("idx", idx), take("coefA", coefA), take("coefB", coefB)
        per = sae.encoder.weight.shape[0] // world
        with ops.span("x_csr_slice", dev):
            # indices relative to this rank's slice; the CSR build skips the ones outside [0, per)
            local = idx_all.to(torch.int64) - rank * per
            row_ptr, entries = ops.csr_build(local, per)
        return dict(row_ptr=row_ptr, entries=entries, k=k, coefA=coefA_all, vecA=vecA_all, coefB=coefB_all,
                    vecB=vecB_all, extra=pend.get("extra")), late

    @torch.no_grad()
    def step(self, closure=None):
        assert closure is None, "Closure is not supported."
        for sae in self._sparse:
            had_pending = sae._pending is not None
            if had_pending:
                self._sparse_step(sae)
            if sae.W_dec.grad is not None:
                sae.wait_decoder()  # a dense update of W_dec must not race the side stream
            if not had_pending and getattr(sae, "_masters_stale", False) and (
                    sae.W_dec.grad is not None or sae.encoder.weight.grad is not None):
                self.sync_masters(sae)  # a dense update of a sharded matrix needs full replicas
        for group in self.param_groups:
            lr = group["lr"]
            lr = float(lr) if not isinstance(lr, Tensor) else float(lr.item())
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self._state_for(p)
                state["step"] += 1
                g = p.grad
                if g.dtype != torch.float32 or not g.is_contiguous():
                    g = g.to(torch.float32).contiguous()
                shadow, cb = self._shadow.get(id(p), (None, None))
                ops.adam_rows_(
                    p.data, g, state["exp_avg"], state["exp_avg_sq"], lr=lr, beta1=beta1,
                    beta2=beta2, eps=group["eps"], step=int(state["step"]),
                    project=id(p) in self._project and p.dim() == 2, shadow=shadow,
                )
                _touched(p)
                if cb is not None:
                    cb()


class ScheduleFreeSignum(torch.optim.Optimizer):
    """optimizer="signum" of the reference Trainer (sparsify/trainer.py:146-161):
    ``ScheduleFreeWrapper(SignSGD(params), momentum=0.95)`` as one optimiser
    whose step is a single fused kernel per parameter.

    SignSGD is the reference's own (sparsify/sign_sgd.py:18-26): p -= lr*sign(g).
    The wrapper comes from the third-party ``schedulefree`` package (Defazio et
    al., "The Road Less Scheduled", 2024; the reference does not pin a version),
    restated here from its published algorithm: the parameter tensor holds the
    gradient-evaluation point y while training, ``state["z"]`` the wrapped
    optimiser's iterate, and the running average x is implied by the two:

        x = y + (1 - 1/momentum)(z - y)            # un-extrapolate
        z = z - lr * sign(grad(y))                 # the wrapped step
        x = x + c_{k+1} (z - x),  c = w_k / sum w  # w_k = (k+1)^r * lr_max^weight_lr_power
        y = x + (1 - momentum)(z - x)              # extrapolate

    ``eval()`` turns the parameters into x (what a checkpoint stores), ``train()``
    back into y. Gradients projected by ``project_rows`` lose their component
    along the parameter rows before the sign is taken.
    """

    def __init__(self, params, lr: float = 1e-3, momentum: float = 0.9, weight_lr_power: float = 2.0,
                 r: float = 0.0):
        if lr <= 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if not 0.0 < momentum <= 1.0:
            raise ValueError(f"Invalid momentum: {momentum}")
        defaults = dict(lr=lr, momentum=momentum, weight_lr_power=weight_lr_power, r=r, k=0, lr_max=-1.0,
                        weight_sum=0.0, train_mode=False)
        super().__init__(params, defaults)
        self._project: set[int] = set()
        self._shadow: dict[int, tuple] = {}

    project_rows = FusedAdam.project_rows
    register_shadow = FusedAdam.register_shadow

    @torch.no_grad()
    def eval(self):
        for group in self.param_groups:
            if group["train_mode"]:
                for p in group["params"]:
                    if "z" in self.state[p]:
                        p.lerp_(end=self.state[p]["z"], weight=1 - 1 / group["momentum"])  # y -> x
                group["train_mode"] = False

    @torch.no_grad()
    def train(self):
        for group in self.param_groups:
            if not group["train_mode"]:
                for p in group["params"]:
                    if "z" in self.state[p]:
                        p.lerp_(end=self.state[p]["z"], weight=1 - group["momentum"])  # x -> y
                group["train_mode"] = True

    @torch.no_grad()
    def step(self, closure=None):
        assert closure is None, "Closure is not supported."
        for group in self.param_groups:
            if not group["train_mode"]:
                raise RuntimeError("Not in train mode: call .train() before stepping (and .eval() to "
                                   "read the averaged parameters)")
            lr = group["lr"]
            lr = float(lr) if not isinstance(lr, Tensor) else float(lr.item())
            k = group["k"]
            lr_max = group["lr_max"] = max(lr, group["lr_max"])
            weight = ((k + 1) ** group["r"]) * (lr_max ** group["weight_lr_power"])
            weight_sum = group["weight_sum"] = group["weight_sum"] + weight
            ckp1 = weight / weight_sum if weight_sum != 0 else 0.0
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if "z" not in state:
                    state["z"] = torch.clone(p.data, memory_format=torch.contiguous_format)
                g = p.grad
                if g.dtype != torch.float32 or not g.is_contiguous():
                    g = g.to(torch.float32).contiguous()
                if id(p) in self._project and p.dim() == 2:
                    ops.project_rows_(g, p.data)
                shadow, cb = self._shadow.get(id(p), (None, None))
                ops.signum_schedulefree_(p.data, state["z"], g, lr, group["momentum"], ckp1, shadow)
                _touched(p)
                if cb is not None:
                    cb()
            group["k"] = k + 1
