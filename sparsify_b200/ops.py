"""Thin functional wrappers over the C ABI: allocate outputs and workspaces as
torch tensors, pass raw device pointers and the current stream. No autograd
here; see fused_encoder.py and embedding_bag.py for the differentiable ops."""

from __future__ import annotations

import torch
from torch import Tensor

from . import _lib
from ._lib import call, dtype_code, ptr


# When set to a dict, selected ops append (start, end) CUDA-event pairs under
# their name, recorded on the launching stream (used by the benchmark to time
# the dominant kernel inside the step).
timers: dict | None = None


def _timed(name: str, device):
    if timers is None:
        return None
    s = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    timers.setdefault(name, []).append((s, e))
    s.record(torch.cuda.current_stream(device))
    return e


class span:
    """Context manager: when `timers` is set, brackets the enclosed work on the current stream
    of `device` with a CUDA-event pair filed under `name` (e.g. how long the compute stream
    waits for an exchange that should have finished in the background)."""

    def __init__(self, name: str, device):
        self.name, self.device, self.end = name, device, None

    def __enter__(self):
        self.end = _timed(self.name, self.device)
        return self

    def __exit__(self, *exc):
        if self.end is not None:
            self.end.record(torch.cuda.current_stream(self.device))
        return False


def _stream(t: Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def _ws(nbytes: int, device) -> Tensor:
    # torch's caching allocator returns 512-byte aligned blocks
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


# One status word per device, shared by every kernel that has bounded waits (the
# tensor-core encoder and GEMM). A wait that gives up stores its code there and
# the word keeps the first code until check_status() reads and clears it.
_status_words: dict[int, Tensor] = {}


def status_word(device) -> Tensor:
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(index)
    if word is None:
        word = _status_words[index] = torch.zeros(8, dtype=torch.int32, device=torch.device("cuda", index))
    return word


def check_status(device=None) -> None:
    """Raises SparseCoderLibError(SC_ERR_TIMEOUT) if a bounded device-side wait of a
    tensor-core kernel gave up since the last check (its outputs are then invalid).
    Reads one word back, i.e. synchronises: call it where the host waits for the
    device anyway (the Trainer does so once per step, with its metric reads)."""
    words = [status_word(device)] if device is not None else list(_status_words.values())
    for word in words:
        code = int(word[0].item())
        if code != 0:
            word.zero_()
            raise _lib.SparseCoderLibError(
                "device wait", _lib.SC_ERR_TIMEOUT,
                f"a bounded wait inside a tensor-core kernel on {word.device} gave up (wait code {code}); "
                "the results of the calls since the last check are invalid")


def selftest_wait_timeout(device, limit_ms: float = 2.0) -> None:
    """Launches the library's wait self-test: a kernel whose only wait can never be
    satisfied and runs out after limit_ms. check_status() must raise afterwards."""
    word = status_word(device)
    with torch.cuda.device(word.device):
        call("sc_selftest_wait_timeout", ptr(word), int(limit_ms * 1e6),
             torch.cuda.current_stream(word.device).cuda_stream)


def _check_cuda(*ts: Tensor | None):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "sparsify_b200 runs on CUDA tensors only; there is no CPU path "
                f"(got a tensor on {t.device})"
            )


def prep_input(x: Tensor, b_dec: Tensor | None, out_dtype: torch.dtype) -> Tensor:
    """x - b_dec (row broadcast) cast to out_dtype."""
    _check_cuda(x, b_dec)
    x = x.contiguous()
    N, D = x.shape
    out = torch.empty(N, D, dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        call("sc_prep_input", ptr(x), dtype_code(x), ptr(_f32(b_dec)), N, D, ptr(out),
             dtype_code(out), _stream(x))
    return out


def _f32(t: Tensor | None) -> Tensor | None:
    if t is None:
        return None
    return t.detach().to(torch.float32).contiguous()


def preacts_dense(x: Tensor, W: Tensor, bias: Tensor | None, out_dtype=torch.float32) -> Tensor:
    _check_cuda(x, W, bias)
    x, W = x.detach().contiguous(), W.detach().contiguous()
    N, D = x.shape
    M = W.shape[0]
    pre = torch.empty(N, M, dtype=out_dtype, device=x.device)
    with torch.cuda.device(x.device):
        call("sc_preacts_dense", ptr(x), dtype_code(x), ptr(W), dtype_code(W), ptr(_f32(bias)),
             N, D, M, ptr(pre), dtype_code(pre), _stream(x))
    return pre


def topk_rows(pre: Tensor, k: int, col_mask: Tensor | None = None) -> tuple[Tensor, Tensor]:
    _check_cuda(pre, col_mask)
    pre = pre.detach().to(torch.float32).contiguous()
    N, M = pre.shape
    vals = torch.empty(N, k, dtype=torch.float32, device=pre.device)
    idx = torch.empty(N, k, dtype=torch.int64, device=pre.device)
    mask = None
    if col_mask is not None:
        mask = col_mask.to(torch.uint8).contiguous()
    with torch.cuda.device(pre.device):
        call("sc_topk_rows", ptr(pre), N, M, int(k), ptr(mask), ptr(vals), ptr(idx), _stream(pre))
    return vals, idx


def topk_mask_rows(pre: Tensor, k: int, col_mask: Tensor | None = None) -> Tensor:
    """bf16 copy of `pre` with everything outside each row's k largest entries zeroed."""
    _check_cuda(pre, col_mask)
    pre = pre.detach().to(torch.float32).contiguous()
    N, M = pre.shape
    out = torch.empty(N, M, dtype=torch.bfloat16, device=pre.device)
    mask = col_mask.to(torch.uint8).contiguous() if col_mask is not None else None
    with torch.cuda.device(pre.device):
        call("sc_topk_mask_rows", ptr(pre), N, M, int(k), ptr(mask), ptr(out), _stream(pre))
    return out


def groupmax_rows(pre: Tensor, k: int) -> tuple[Tensor, Tensor]:
    _check_cuda(pre)
    pre = pre.detach().to(torch.float32).contiguous()
    N, M = pre.shape
    vals = torch.empty(N, k, dtype=torch.float32, device=pre.device)
    idx = torch.empty(N, k, dtype=torch.int64, device=pre.device)
    with torch.cuda.device(pre.device):
        call("sc_groupmax_rows", ptr(pre), N, M, int(k), ptr(vals), ptr(idx), _stream(pre))
    return vals, idx


def set_reserved_sms(n: int) -> None:
    """Leaves `n` SMs free of the persistent tensor-core kernels (for collectives that
    should run beside them); see sc_set_reserved_sms."""
    call("sc_set_reserved_sms", int(n))


def set_cta_pairs(on: bool | None) -> None:
    """Form of the tensor-core encoder: True = CTA pairs (tcgen05 cta_group::2), False = one CTA per
    tile, None = chosen per shape (the default); see sc_set_cta_pairs."""
    call("sc_set_cta_pairs", -1 if on is None else int(bool(on)))


def tc_encode_supported(D: int, M: int, k: int) -> bool:
    return D % 8 == 0 and 0 < k <= 128 and k <= M


def encode_topk_tc(x_bf16: Tensor, W_bf16: Tensor, bias: Tensor, k: int) -> tuple[Tensor, Tensor]:
    """Tensor-core encoder: relu(x W^T + b) and exact per-row top-k, never
    materialising the [N, M] matrix. Values come out in descending order."""
    _check_cuda(x_bf16, W_bf16, bias)
    assert x_bf16.dtype == torch.bfloat16 and W_bf16.dtype == torch.bfloat16
    x_bf16, W_bf16 = x_bf16.contiguous(), W_bf16.contiguous()
    N, D = x_bf16.shape
    M = W_bf16.shape[0]
    dev = x_bf16.device
    vals = torch.empty(N, k, dtype=torch.float32, device=dev)
    idx = torch.empty(N, k, dtype=torch.int64, device=dev)
    nbytes = _lib.lib().sc_encode_topk_workspace_bytes(N, D, M, int(k))
    ws = _ws(nbytes, dev)
    status = status_word(dev)  # [0] wait-timeout code (sticky), [1:] diagnostics builds only
    bias32 = _f32(bias)
    with torch.cuda.device(dev):
        end = _timed("encode_topk", dev)
        call("sc_encode_topk", ptr(x_bf16), ptr(W_bf16), ptr(bias32), N, D, M, int(k),
             ptr(vals), ptr(idx), ptr(ws), ws.numel(), ptr(status), _stream(x_bf16))
        if end is not None:
            end.record(torch.cuda.current_stream(dev))
    encode_topk_tc.last_status = status
    return vals, idx


def tc_groupmax_supported(D: int, M: int, k: int) -> bool:
    if D % 8 or k <= 0 or M % k:
        return False
    g = M // k
    return g % 32 == 0 and (g % 256 == 0 or 256 % g == 0)


def encode_groupmax_tc(x_bf16: Tensor, W_bf16: Tensor, bias: Tensor, k: int) -> tuple[Tensor, Tensor]:
    """Tensor-core encoder with the groupmax activation: per row, the largest post-ReLU
    pre-activation of each of the k groups of M/k consecutive latents, in group order."""
    _check_cuda(x_bf16, W_bf16, bias)
    assert x_bf16.dtype == torch.bfloat16 and W_bf16.dtype == torch.bfloat16
    x_bf16, W_bf16 = x_bf16.contiguous(), W_bf16.contiguous()
    N, D = x_bf16.shape
    M = W_bf16.shape[0]
    dev = x_bf16.device
    vals = torch.empty(N, k, dtype=torch.float32, device=dev)
    idx = torch.empty(N, k, dtype=torch.int64, device=dev)
    status = status_word(dev)
    bias32 = _f32(bias)
    with torch.cuda.device(dev):
        call("sc_encode_groupmax", ptr(x_bf16), ptr(W_bf16), ptr(bias32), N, D, M, int(k),
             ptr(vals), ptr(idx), ptr(status), _stream(x_bf16))
    encode_groupmax_tc.last_status = status
    return vals, idx


def embedding_bag_fwd(idx: Tensor, acts: Tensor, W: Tensor, bias: Tensor | None = None) -> Tensor:
    """out[n] = bias + sum_j acts[n, j] * W[idx[n, j]], fp32."""
    _check_cuda(idx, acts, W, bias)
    idx = idx.contiguous()
    acts = _f32(acts)
    W = W.detach().contiguous()
    N, k = idx.shape
    M, D = W.shape
    out = torch.empty(N, D, dtype=torch.float32, device=W.device)
    with torch.cuda.device(W.device):
        call("sc_embedding_bag_fwd", ptr(idx), ptr(acts), ptr(W), dtype_code(W), ptr(_f32(bias)),
             N, D, M, int(k), ptr(out), _stream(W))
    return out


def embedding_bag_bwd_acts(idx: Tensor, grad_out: Tensor, W: Tensor) -> Tensor:
    _check_cuda(idx, grad_out, W)
    idx = idx.contiguous()
    grad_out = grad_out.detach().contiguous()
    if grad_out.dtype not in (torch.float32, torch.bfloat16):
        grad_out = grad_out.to(torch.float32)
    W = W.detach().contiguous()
    N, k = idx.shape
    M, D = W.shape
    gacts = torch.empty(N, k, dtype=torch.float32, device=W.device)
    with torch.cuda.device(W.device):
        call("sc_embedding_bag_bwd_acts", ptr(idx), ptr(grad_out), dtype_code(grad_out), ptr(W),
             dtype_code(W), N, D, M, int(k), ptr(gacts), _stream(W))
    return gacts


def decode_dots_supported(W: Tensor, k: int) -> bool:
    """Whether `decode_residual(..., want_dots=True)` has a kernel for this case."""
    D = W.shape[-1]
    return W.dtype == torch.bfloat16 and k <= 32 and D % 4 == 0


def decode_residual(idx: Tensor, acts: Tensor, W: Tensor, bias: Tensor | None, y: Tensor, *,
                    want_out: bool = True, want_e32: bool = False, want_e16: bool = False,
                    want_dots: bool = False):
    """(out, e_f32, e_bf16, sse): decode, residual e = y - out and sum(e^2) in one pass.
    want_dots=True (see `decode_dots_supported`) appends dots[N, k] = e . W[idx], computed from
    the same gathered rows: the activation gradient of the decode up to the scalar that turns
    e into the gradient of the output."""
    _check_cuda(idx, acts, W, bias, y)
    idx, acts = idx.contiguous(), _f32(acts)
    W, y = W.detach().contiguous(), y.detach().contiguous()
    if y.dtype not in (torch.float32, torch.bfloat16):
        y = y.to(torch.float32)
    N, k = idx.shape
    M, D = W.shape
    dev = W.device
    out = torch.empty(N, D, dtype=torch.float32, device=dev) if want_out else None
    e32 = torch.empty(N, D, dtype=torch.float32, device=dev) if want_e32 else None
    e16 = torch.empty(N, D, dtype=torch.bfloat16, device=dev) if want_e16 else None
    sse = torch.empty((), dtype=torch.float32, device=dev)
    ws = _ws(_lib.lib().sc_decode_residual_workspace_bytes(N), dev)
    bias32 = _f32(bias)
    if want_dots:
        dots = torch.empty(N, k, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            call("sc_decode_residual_dots", ptr(idx), ptr(acts), ptr(W), dtype_code(W), ptr(bias32), ptr(y),
                 dtype_code(y), N, D, M, int(k), ptr(out), ptr(e32), ptr(e16), ptr(sse), ptr(dots), ptr(ws),
                 ws.numel(), _stream(W))
        return out, e32, e16, sse, dots
    with torch.cuda.device(dev):
        call("sc_decode_residual", ptr(idx), ptr(acts), ptr(W), dtype_code(W), ptr(bias32), ptr(y),
             dtype_code(y), N, D, M, int(k), ptr(out), ptr(e32), ptr(e16), ptr(sse), ptr(ws), ws.numel(),
             _stream(W))
    return out, e32, e16, sse


def csr_build(idx: Tensor, M: int) -> tuple[Tensor, Tensor]:
    """Latent-major CSR (row_ptr[M+1], entries[N*k]) of an [N, k] index matrix."""
    _check_cuda(idx)
    idx = idx.contiguous()
    N, k = idx.shape
    dev = idx.device
    row_ptr = torch.empty(M + 1, dtype=torch.int32, device=dev)
    entries = torch.empty(max(N * k, 1), dtype=torch.int32, device=dev)
    ws = _ws(_lib.lib().sc_csr_workspace_bytes(M), dev)
    with torch.cuda.device(dev):
        call("sc_csr_build", ptr(idx), N, int(k), int(M), ptr(row_ptr), ptr(entries), ptr(ws),
             ws.numel(), _stream(idx))
    return row_ptr, entries


def rows_accumulate(
    row_ptr: Tensor,
    entries: Tensor,
    k: int,
    M: int,
    D: int,
    coefA: Tensor,
    vecA: Tensor,
    *,
    biasA: bool = False,
    coefB: Tensor | None = None,
    vecB: Tensor | None = None,
    biasB: bool = False,
    lat_range: tuple[int, int] | None = None,
    out: dict | None = None,
) -> dict:
    """Per-latent sums of coef * vec rows; returns {"gradA", "gbiasA", "gradB", "gbiasB"}.
    `out` may supply preallocated [M, D] / [M] tensors under the same keys (used
    when the gradient is produced chunk by chunk over latent ranges)."""
    _check_cuda(row_ptr, entries, coefA, vecA, coefB, vecB)
    dev = vecA.device
    out = dict(out or {})
    coefA = _f32(coefA).reshape(-1)
    vecA = vecA.detach().contiguous()
    has_b = coefB is not None
    if has_b:
        coefB = _f32(coefB).reshape(-1)
        vecB = vecB.detach().contiguous()
    def buf(name, shape, want):
        if not want:
            return None
        if out.get(name) is None:
            out[name] = torch.empty(shape, dtype=torch.float32, device=dev)
        return out[name]
    gA = buf("gradA", (M, D), True)
    gbA = buf("gbiasA", (M,), biasA)
    gB = buf("gradB", (M, D), has_b)
    gbB = buf("gbiasB", (M,), has_b and biasB)
    lo, hi = lat_range if lat_range is not None else (0, M)
    with torch.cuda.device(dev):
        call("sc_rows_accumulate", ptr(row_ptr), ptr(entries), int(k), ptr(coefA), ptr(vecA),
             dtype_code(vecA), ptr(gA), ptr(gbA), ptr(coefB), ptr(vecB),
             dtype_code(vecB) if has_b else 0, ptr(gB), ptr(gbB), int(M), int(D), int(lo), int(hi),
             _stream(vecA))
    return out


def csr_segment_sum(row_ptr: Tensor, entries: Tensor, coef: Tensor, M: int) -> Tensor:
    """out[m] = sum of coef over the CSR entries of latent m."""
    _check_cuda(row_ptr, entries, coef)
    coef = _f32(coef).reshape(-1)
    out = torch.empty(M, dtype=torch.float32, device=coef.device)
    with torch.cuda.device(coef.device):
        call("sc_csr_segment_sum", ptr(row_ptr), ptr(entries), ptr(coef), int(M), ptr(out), _stream(coef))
    return out


def rows_adam_(row_ptr: Tensor, entries: Tensor, k: int, coefA: Tensor, vecA: Tensor, coefB: Tensor,
               vecB: Tensor, *, pA: Tensor, mA: Tensor, vA: Tensor, shadowA: Tensor | None, projectA: bool,
               normalizeA: bool, norm_eps: float, hpA: dict, pB: Tensor, mB: Tensor, vB: Tensor,
               shadowB: Tensor | None, hpB: dict, parts: int = 3, max_ctas: int = 0,
               extraA: Tensor | None = None, extra_rank: Tensor | None = None) -> None:
    """Sparse gradients of the decoder (A) and encoder (B) applied straight to the
    parameters: projection, Adam, decoder normalisation and bf16 shadows in one pass.
    hpA / hpB: dict(lr, beta1, beta2, eps, step)."""
    import ctypes
    _check_cuda(row_ptr, entries, coefA, vecA, coefB, vecB, pA, mA, vA, pB, mB, vB, shadowA, shadowB)
    M, D = pA.shape
    coefA, coefB = _f32(coefA).reshape(-1), _f32(coefB).reshape(-1)
    vecA, vecB = vecA.detach().contiguous(), vecB.detach().contiguous()
    for t in (pA, mA, vA, pB, mB, vB):
        assert t.dtype == torch.float32 and t.is_contiguous()
    ha = _lib.AdamHparams(hpA["lr"], hpA["beta1"], hpA["beta2"], hpA["eps"], hpA["step"])
    hb = _lib.AdamHparams(hpB["lr"], hpB["beta1"], hpB["beta2"], hpB["eps"], hpB["step"])
    with torch.cuda.device(pA.device):
        end = _timed("rows_adam", pA.device)
        call("sc_rows_adam", ptr(row_ptr), ptr(entries), int(k), ptr(coefA), ptr(vecA), dtype_code(vecA),
             ptr(coefB), ptr(vecB), dtype_code(vecB), int(M), int(D), ptr(pA), ptr(mA), ptr(vA), ptr(shadowA),
             int(bool(projectA)), int(bool(normalizeA)), float(norm_eps), ctypes.byref(ha), ptr(pB), ptr(mB),
             ptr(vB), ptr(shadowB), ctypes.byref(hb), ptr(extraA), ptr(extra_rank), int(parts), int(max_ctas), _stream(pA))
        if end is not None:
            end.record(torch.cuda.current_stream(pA.device))


def total_variance(y: Tensor) -> Tensor:
    """sum((y - y.mean(0))**2) as a 0-d fp32 device tensor."""
    _check_cuda(y)
    y = y.detach().contiguous()
    if y.dtype not in (torch.float32, torch.bfloat16):
        y = y.to(torch.float32)
    N, D = y.shape
    tv = torch.empty((), dtype=torch.float32, device=y.device)
    ws = _ws(_lib.lib().sc_loss_workspace_bytes(D), y.device)
    with torch.cuda.device(y.device):
        call("sc_total_variance", ptr(y), dtype_code(y), N, D, ptr(tv), ptr(ws), ws.numel(), _stream(y))
    return tv


def sq_err(a: Tensor, b: Tensor, want_diff: bool = False) -> tuple[Tensor, Tensor | None]:
    """(sum((a-b)**2), a-b or None)."""
    _check_cuda(a, b)
    a, b = _f32(a), _f32(b)
    assert a.shape == b.shape
    sse = torch.empty((), dtype=torch.float32, device=a.device)
    diff = torch.empty_like(a) if want_diff else None
    ws = _ws(4096, a.device)
    with torch.cuda.device(a.device):
        call("sc_sq_err", ptr(a), ptr(b), a.numel(), ptr(diff), ptr(sse), ptr(ws), ws.numel(),
             _stream(a))
    return sse, diff


def weighted_colsum(Y: Tensor, w: Tensor | None = None) -> Tensor:
    """sum_r w[r] * Y[r, :] (w=None: column sums) as an fp32 [D] tensor."""
    _check_cuda(Y, w)
    Y = Y.detach().contiguous()
    R, D = Y.shape
    out = torch.empty(D, dtype=torch.float32, device=Y.device)
    ws = _ws(_lib.lib().sc_loss_workspace_bytes(D), Y.device)
    w32 = _f32(w)
    with torch.cuda.device(Y.device):
        call("sc_weighted_colsum", ptr(Y), dtype_code(Y), ptr(w32), R, D, ptr(out), ptr(ws),
             ws.numel(), _stream(Y))
    return out


def normalize_rows_(W: Tensor, eps: float, shadow: Tensor | None = None) -> None:
    """In place W[m] /= ||W[m]|| + eps; optionally refreshes a bf16 shadow."""
    _check_cuda(W, shadow)
    assert W.dtype == torch.float32 and W.is_contiguous()
    M, D = W.shape
    with torch.cuda.device(W.device):
        call("sc_normalize_rows", ptr(W), M, D, float(eps), ptr(shadow), _stream(W))


def adam_rows_(p: Tensor, g: Tensor, m: Tensor, v: Tensor, *, lr: float, beta1: float, beta2: float,
               eps: float, step: int, project: bool = False, shadow: Tensor | None = None) -> None:
    """One Adam step on p (any shape; rows = leading dim) with optional removal of
    the gradient component parallel to each row of p, optional bf16 shadow refresh."""
    _check_cuda(p, g, m, v, shadow)
    for t in (p, g, m, v):
        assert t.dtype == torch.float32 and t.is_contiguous()
    if p.dim() >= 2:
        M, D = p.shape[0], p.numel() // p.shape[0]
    else:
        M, D = 1, p.numel()
    with torch.cuda.device(p.device):
        call("sc_adam_rows", ptr(p), ptr(g), ptr(m), ptr(v), M, D, float(lr), float(beta1),
             float(beta2), float(eps), int(step), int(bool(project)), ptr(shadow), _stream(p))


def muon_momentum_(g: Tensor, buf: Tensor, beta: float, nesterov: bool) -> tuple[Tensor, Tensor]:
    """Momentum (+ Nesterov) of sparsify/muon.py:150-156 in one pass: updates `buf` in place
    and returns the bf16 cast of the result together with the sum of its squares."""
    _check_cuda(g, buf)
    assert g.dtype == buf.dtype == torch.float32 and g.is_contiguous() and buf.is_contiguous() and g.shape == buf.shape
    out = torch.empty(g.shape, dtype=torch.bfloat16, device=g.device)
    sumsq = torch.empty(1, dtype=torch.float32, device=g.device)
    ws = _ws(_lib.lib().sc_muon_workspace_bytes(), g.device)
    with torch.cuda.device(g.device):
        call("sc_muon_momentum", ptr(g), ptr(buf), g.numel(), float(beta), int(bool(nesterov)), ptr(out),
             ptr(sumsq), ptr(ws), ws.numel(), _stream(g))
    return out, sumsq


def scale_transpose_bf16(x: Tensor, sumsq: Tensor | None, *, scaled: bool = True, transposed: bool = True):
    """x / (||x||_F + 1e-7) with bf16 roundings as torch applies them (sumsq = sum of squares of
    x, None for no scaling), in x's orientation and / or transposed, in one pass."""
    _check_cuda(x, sumsq)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    R, C = x.shape
    out_s = torch.empty(R, C, dtype=torch.bfloat16, device=x.device) if scaled else None
    out_t = torch.empty(C, R, dtype=torch.bfloat16, device=x.device) if transposed else None
    with torch.cuda.device(x.device):
        call("sc_scale_transpose_bf16", ptr(x), R, C, ptr(sumsq), ptr(out_s), ptr(out_t), _stream(x))
    return out_s, out_t


def muon_apply_(p: Tensor, upd: Tensor, decay: float, alpha: float, shadow: Tensor | None = None) -> None:
    """p = p * decay - alpha * upd (bf16), in place; optional bf16 copy of the result
    (sparsify/muon.py:120-123,139-141,176-178 in one pass)."""
    _check_cuda(p, upd, shadow)
    assert p.dtype == torch.float32 and upd.dtype == torch.bfloat16 and p.is_contiguous() and upd.is_contiguous()
    assert p.numel() == upd.numel()
    with torch.cuda.device(p.device):
        call("sc_muon_apply", ptr(p), ptr(upd), p.numel(), float(decay), float(alpha), ptr(shadow), _stream(p))


def project_rows_(g: Tensor, w: Tensor) -> None:
    """g[m] -= (g[m] . w[m]) w[m] in place (sparsify/sparse_coder.py:281-295)."""
    _check_cuda(g, w)
    assert g.dtype == w.dtype == torch.float32 and g.is_contiguous() and w.is_contiguous() and g.shape == w.shape
    M, D = g.shape
    with torch.cuda.device(g.device):
        call("sc_project_rows", ptr(g), ptr(w), M, D, _stream(g))


def signum_schedulefree_(p: Tensor, z: Tensor, g: Tensor, lr: float, momentum: float, ckp1: float,
                         shadow: Tensor | None = None) -> None:
    """One schedule-free sign-descent step in place on (p, z); see sc_signum_schedulefree."""
    _check_cuda(p, z, g, shadow)
    for t in (p, z, g):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() == p.numel()
    if shadow is not None:
        assert shadow.dtype == torch.bfloat16 and shadow.is_contiguous() and shadow.numel() == p.numel()
    with torch.cuda.device(p.device):
        call("sc_signum_schedulefree", ptr(p), ptr(z), ptr(g), p.numel(), float(lr), float(momentum),
             float(ckp1), ptr(shadow), _stream(p))


def cast_bf16(src: Tensor, dst: Tensor | None = None) -> Tensor:
    _check_cuda(src, dst)
    src = src.detach()
    assert src.dtype == torch.float32 and src.is_contiguous()
    if dst is None:
        dst = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
    with torch.cuda.device(src.device):
        call("sc_cast_bf16", ptr(src), ptr(dst), src.numel(), _stream(src))
    return dst


def gemm_nt(A: Tensor, B: Tensor, *, alpha: float = 1.0, beta: float = 0.0, Cin: Tensor | None = None,
            bias: Tensor | None = None, relu: bool = False, out_dtype: torch.dtype = torch.bfloat16,
            out: Tensor | None = None, symmetric: bool = False, out_t: Tensor | None = None) -> Tensor:
    """act(alpha * A @ B.T + beta * Cin + bias) on the tensor cores; A [M,K], B [N,K] bf16.
    symmetric: B is A and the result is symmetric (only the tiles reaching the upper
    triangle are computed, the rest mirrored). out_t: also receives the result transposed."""
    _check_cuda(A, B, Cin, bias, out, out_t)
    assert A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16 and A.shape[1] == B.shape[1]
    if symmetric:
        assert B is A or (B.data_ptr() == A.data_ptr() and B.shape == A.shape)
        A = B = A.contiguous()
    else:
        A, B = A.contiguous(), B.contiguous()
    M, K = A.shape
    N = B.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=A.device)
    assert out.shape == (M, N) and out.is_contiguous()
    if Cin is not None:
        Cin = Cin.contiguous()
        assert Cin.shape == (M, N)
    if out_t is not None:
        assert out_t.shape == (N, M) and out_t.is_contiguous() and out_t.dtype == out.dtype
    bias32 = _f32(bias)
    status = status_word(A.device)
    with torch.cuda.device(A.device):
        call("sc_gemm_bf16_nt", ptr(A), ptr(B), M, N, K, float(alpha), float(beta), ptr(Cin),
             dtype_code(Cin) if Cin is not None else 0, ptr(bias32), int(bool(relu)), ptr(out),
             dtype_code(out), int(bool(symmetric)), ptr(out_t), ptr(status), _stream(A))
    gemm_nt.last_status = status
    return out


def transpose_bf16(x: Tensor) -> Tensor:
    _check_cuda(x)
    assert x.dtype == torch.bfloat16 and x.dim() == 2
    x = x.contiguous()
    R, C = x.shape
    out = torch.empty(C, R, dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        call("sc_transpose_bf16", ptr(x), R, C, ptr(out), _stream(x))
    return out
