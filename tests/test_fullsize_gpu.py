"""Parity at the sizes the benchmark runs, where the oracle cannot finish a whole
problem in seconds: the encoder's 17.6 TFLOP contraction is checked on sampled
rows (fp64 pre-activations of just those rows, computed by the oracle on the
host), everything after the selection - decode, FVU, every gradient, projection,
Adam, decoder normalisation - is checked with the oracle's own functions, run on
all tokens in chunks over compacted weight tables, for sampled latents' rows and
for the whole bias vectors.

Shapes (tokens, d_in, latents, k): (16384, 4096, 131072, 32) SAE,
(16384, 4096, 131072, 64) transcoder width, (8192, 4096, 65536, 32) one hookpoint
of the sharded multi-hookpoint workload. Inputs are the seeded synthetic
activations of sparsify_b200.synthetic; weights are SparseCoder's own seeded
initialisation (sparsify/sparse_coder.py:53-65).
"""

import pytest
import torch

from oracle import sae_oracle as O
from tests.conftest import rel_l2
from tests.test_kernels_gpu import ACT_TOL, GRAD_TOL, check_topk_sets

pytestmark = pytest.mark.gpu

N_FULL, D_FULL, M_FULL = 16384, 4096, 131072
ROW_SAMPLES = 256


def bf16_round(t):
    return t.to(torch.bfloat16).to(torch.float32)


def sample_rows(n_rows: int, count: int, seed: int) -> torch.Tensor:
    """Rows at both ends of every 128- and 256-row block that starts or ends a block
    of 4096 rows (the encoder schedules row blocks in groups), plus random rows."""
    rows = set()
    for base in range(0, n_rows, 4096):
        for off in (0, 127, 128, 255, 256, 3839, 3840, 3967, 3968, 4095):
            if base + off < n_rows:
                rows.add(base + off)
    g = torch.Generator().manual_seed(seed)
    # random rows, drawn alternately from the lower and the upper half so that a problem that
    # uses only the first half of the tokens still sees half of the samples
    half = n_rows // 2
    lower, upper = torch.randperm(half, generator=g).tolist(), (torch.randperm(n_rows - half, generator=g) + half).tolist()
    for lo_r, up_r in zip(lower, upper):
        if len(rows) >= count:
            break
        rows.add(lo_r)
        rows.add(up_r)
    return torch.tensor(sorted(rows))


@pytest.fixture(scope="module")
def full_problem(cuda_lib):
    """x [16384, 4096] bf16 (synthetic activations), W [131072, 4096] bf16, b [131072] on
    the GPU, and the oracle's fp64 pre-activations of the sampled rows on the host."""
    from sparsify_b200.synthetic import SyntheticActivations
    dev = torch.device("cuda")
    gen = SyntheticActivations(D_FULL, 65536, 64, device=dev)
    x = gen.batch(N_FULL, seed=11, dtype=torch.bfloat16)
    x = (x.float() - x.float().mean(0)).to(torch.bfloat16)  # what the encoder sees: x - b_dec
    del gen
    torch.cuda.empty_cache()
    g = torch.Generator(device=dev).manual_seed(12)
    bound = 1.0 / D_FULL ** 0.5
    W = ((torch.rand(M_FULL, D_FULL, device=dev, generator=g) * 2 - 1) * bound).to(torch.bfloat16)
    b = 0.05 * torch.randn(M_FULL, device=dev, generator=g)
    rows = sample_rows(N_FULL, ROW_SAMPLES, seed=13)
    xs = x[rows.cuda()].cpu().double()
    pre = torch.empty(len(rows), M_FULL, dtype=torch.float32)
    for lo in range(0, M_FULL, 8192):  # the oracle, chunked over the latents
        hi = lo + 8192
        pre[:, lo:hi] = O.preacts(xs, W[lo:hi].cpu().double(), b[lo:hi].cpu().double()).float()
    return dict(x=x, W=W, b=b, rows=rows, pre=pre)


@pytest.mark.parametrize("N,M,k", [
    (16384, 131072, 32),   # the headline shape
    (16384, 131072, 64),   # transcoder workload's k
    (8192, 65536, 32),     # one hookpoint of the multi-hookpoint workload
])
def test_encoder_fullsize_sampled_rows(full_problem, N, M, k):
    from sparsify_b200 import ops
    p = full_problem
    vals, idx = ops.encode_topk_tc(p["x"][:N], p["W"][:M], p["b"][:M], k)
    torch.cuda.synchronize()
    ops.check_status(vals.device)  # no bounded wait gave up
    keep = p["rows"] < N
    rows = p["rows"][keep]
    assert len(rows) >= 100
    check_topk_sets(vals[rows.cuda()], idx[rows.cuda()], p["pre"][keep][:, :M], k)
    # every row, cheaply: k distinct in-range indices, values descending and non-negative
    assert bool(((idx >= 0) & (idx < M)).all())
    assert bool((idx.sort(dim=1).values.diff(dim=1) > 0).all())
    assert bool((vals.diff(dim=1) <= 0).all()) and bool((vals >= 0).all())


def test_fused_step_fullsize_vs_oracle(cuda_lib):
    """One optimiser step of the headline workload through SparseCoder + FusedAdam (sparse
    update), against the oracle's decode / backward / projection / Adam / normalisation."""
    from sparsify_b200 import SparseCoder, SparseCoderConfig, ops
    from sparsify_b200.optim import FusedAdam
    from sparsify_b200.synthetic import SyntheticActivations

    dev = torch.device("cuda")
    N, D, M, k = N_FULL, D_FULL, M_FULL, 32
    lr, b1, b2 = 7e-5, 0.9, 0.999
    torch.manual_seed(0)
    sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=k), device=dev, dtype=torch.float32)
    gen = SyntheticActivations(D, 65536, 64, device=dev)
    x = gen.batch(N, seed=21, dtype=torch.bfloat16)
    del gen
    torch.cuda.empty_cache()
    with torch.no_grad():
        sae.b_dec.copy_(x.float().mean(0))
        sae.encoder.bias.copy_(0.01 * torch.randn(M, device=dev))
    opt = FusedAdam(sae.parameters(), lr=lr, betas=(b1, b2))
    sae.attach_optimizer(opt)
    assert opt.enable_sparse_update(sae)
    sae.set_decoder_norm_to_unit_norm()
    old = {n: p.detach().cpu().clone() for n, p in
           (("W_enc", sae.encoder.weight), ("b_enc", sae.encoder.bias), ("W_dec", sae.W_dec), ("b_dec", sae.b_dec))}

    out = sae(x)
    out.fvu.backward()
    opt.step()
    torch.cuda.synchronize()
    ops.check_status(dev)

    idx = out.latent_indices.cpu()
    acts = out.latent_acts.detach().cpu().float()
    xf = x.cpu().float()
    y = xf
    xe = bf16_round(xf - old["b_dec"])          # sparsify/sparse_coder.py:191-192, bf16 GEMM operand
    Wd_r, We_r = bf16_round(old["W_dec"]), bf16_round(old["W_enc"])
    tv = (y - y.mean(0)).pow(2).sum()           # sparse_coder.py:228

    g = torch.Generator().manual_seed(22)
    counts = torch.bincount(idx.reshape(-1), minlength=M)
    fired = counts.nonzero().squeeze(1)
    sampled = set(fired[torch.randperm(len(fired), generator=g)[:200]].tolist())
    sampled |= {int(counts.argmax()), int(fired[0]), int(fired[-1])}
    never = (counts == 0).nonzero().squeeze(1)[:8].tolist()  # rows with a zero gradient still take an Adam step
    sampled = torch.tensor(sorted(sampled | set(never)))
    slot = torch.full((M,), -1, dtype=torch.long)
    slot[sampled] = torch.arange(len(sampled))
    gWd_s = torch.zeros(len(sampled), D)
    gWe_s = torch.zeros(len(sampled), D)
    gb_enc = torch.zeros(M)
    gb_dec = torch.zeros(D)
    sse = torch.zeros((), dtype=torch.float64)
    tok = sample_rows(N, 128, seed=23)
    out_ref = {}
    CH = 512
    for lo in range(0, N, CH):
        sl = slice(lo, lo + CH)
        uniq, inv = torch.unique(idx[sl], return_inverse=True)   # compact weight tables of this chunk
        Wd_c, We_c = Wd_r[uniq], We_r[uniq]
        o = O.decode(inv, acts[sl], Wd_c, old["b_dec"])
        e = y[sl] - o
        sse += e.double().pow(2).sum()
        g_out = (-2.0 / tv) * e                                  # d fvu / d out
        gWd_c, g_acts = O.decode_backward(inv, acts[sl], Wd_c, g_out)
        gx, gWe_c, gbe_c = O.encoder_backward(xe[sl], We_c, inv, g_acts)
        gb_enc[uniq] += gbe_c
        gb_dec += g_out.sum(0) - gx.sum(0)
        s = slot[uniq]
        hit = s >= 0
        gWd_s[s[hit]] += gWd_c[hit]
        gWe_s[s[hit]] += gWe_c[hit]
        for t in tok[(tok >= lo) & (tok < lo + CH)].tolist():
            out_ref[t] = o[t - lo]
    fvu_ref = float(sse / tv.double())

    # forward: reconstruction rows and the loss
    tok_ids = sorted(out_ref)
    ref_rows = torch.stack([out_ref[t] for t in tok_ids])
    assert rel_l2(out.sae_out.detach()[torch.tensor(tok_ids).cuda()], ref_rows) < ACT_TOL
    assert abs(float(out.fvu.detach()) - fvu_ref) <= 1e-3 * fvu_ref

    # gradients, read back from Adam's first moment after step 1: exp_avg = (1 - beta1) g
    st_enc, st_dec = opt.state[sae.encoder.weight], opt.state[sae.W_dec]
    sc = sampled.cuda()
    gWe_gpu = st_enc["exp_avg"][sc].cpu() / (1 - b1)
    assert rel_l2(gWe_gpu, gWe_s) < GRAD_TOL
    gWd_proj = gWd_s.clone()
    O.project_out_parallel_(gWd_proj, old["W_dec"][sampled])   # sparse_coder.py:281-295
    gWd_gpu = st_dec["exp_avg"][sc].cpu() / (1 - b1)
    assert rel_l2(gWd_gpu, gWd_proj) < GRAD_TOL
    assert rel_l2(opt.state[sae.encoder.bias]["exp_avg"].cpu() / (1 - b1), gb_enc) < GRAD_TOL
    assert rel_l2(opt.state[sae.b_dec]["exp_avg"].cpu() / (1 - b1), gb_dec) < GRAD_TOL

    # Parameters after Adam (and the decoder's re-normalisation). At step 1 Adam moves every
    # element by lr * g / (|g| + eps): a sign-like function of g, so the update is checked as
    # arithmetic - the oracle's Adam applied to the gradient the GPU used (read back from its
    # first moment, itself checked against the oracle above) - and the change must then agree
    # to fp32 rounding.
    def adam_rows(p_old, grad):
        p, m, v = p_old.clone(), torch.zeros_like(p_old), torch.zeros_like(p_old)
        O.adam_step_(p, grad, m, v, step=1, lr=lr, beta1=b1, beta2=b2)
        return p
    We_new = adam_rows(old["W_enc"][sampled], gWe_gpu)
    Wd_new = adam_rows(old["W_dec"][sampled], gWd_gpu)
    O.normalize_decoder_(Wd_new)                                # applied at the end of the step here
    d_enc = sae.encoder.weight.detach()[sc].cpu() - old["W_enc"][sampled]
    d_dec = sae.W_dec.detach()[sc].cpu() - old["W_dec"][sampled]
    assert rel_l2(d_enc, We_new - old["W_enc"][sampled]) < 1e-3
    assert rel_l2(d_dec, Wd_new - old["W_dec"][sampled]) < 1e-3
    assert rel_l2(sae.W_dec.detach()[sc].cpu().norm(dim=1), torch.ones(len(sampled))) < 1e-6
    for name, p in (("b_enc", sae.encoder.bias), ("b_dec", sae.b_dec)):
        g_gpu = opt.state[p]["exp_avg"].cpu() / (1 - b1)
        assert rel_l2(p.detach().cpu() - old[name], adam_rows(old[name], g_gpu) - old[name]) < 1e-3, name
    # the bf16 copies the next forward reads are the rounded new parameters
    assert torch.equal(sae.shadow("encoder.weight")[sc].cpu(), sae.encoder.weight.detach()[sc].cpu().to(torch.bfloat16))
    assert torch.equal(sae.shadow("W_dec")[sc].cpu(), sae.W_dec.detach()[sc].cpu().to(torch.bfloat16))


def test_wait_that_runs_out_is_reported(cuda_lib):
    """A bounded device-side wait that nothing satisfies gives up after its limit, leaves its
    code in the status word, and the host raises SC_ERR_TIMEOUT where it checks; the context
    stays usable (no fault, no hang)."""
    from sparsify_b200 import _lib, ops
    dev = torch.device("cuda")
    ops.check_status(dev)
    ops.selftest_wait_timeout(dev, limit_ms=2.0)
    torch.cuda.synchronize()
    with pytest.raises(_lib.SparseCoderLibError) as err:
        ops.check_status(dev)
    assert err.value.status == _lib.SC_ERR_TIMEOUT and "199" in str(err.value)
    ops.check_status(dev)  # cleared by the read
    a = torch.randn(64, 64, device=dev).bfloat16()
    assert rel_l2(ops.gemm_nt(a, a, out_dtype=torch.float32), a.float() @ a.float().T) < 1e-2
    ops.check_status(dev)
