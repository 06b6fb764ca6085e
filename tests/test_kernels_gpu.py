"""Parity of each CUDA entry point with the CPU oracle on the same seeded
inputs, and with the reference-generated golden fixtures. Integer results
(indices, CSR) must match exactly; floating point within the stated tolerance.
"""

import pytest
import torch

from oracle import sae_oracle as O
from tests.conftest import load_golden, rel_l2, sort_topk

pytestmark = pytest.mark.gpu

F32_TOL = 2e-5     # fp32 kernels vs fp32 oracle (summation order differs)
ACT_TOL = 1e-3     # selected activations / decode output (north-star tolerance)
GRAD_TOL = 1e-2    # gradients in the bf16 configuration (north-star tolerance)


def dev(t):
    return t.cuda() if t is not None else None


def bf16_round(t):
    return t.to(torch.bfloat16).to(torch.float32)


def check_topk_sets(vals_gpu, idx_gpu, pre_ref, k, rel_gap=1e-3):
    """Index sets must agree row by row except where the k-th and (k+1)-th
    reference pre-activations are closer than rel_gap (relative)."""
    vals_gpu, idx_gpu = vals_gpu.cpu(), idx_gpu.cpu()
    top = torch.topk(pre_ref, min(k + 1, pre_ref.shape[1]), dim=-1).values
    bad = 0
    for n in range(pre_ref.shape[0]):
        got = set(idx_gpu[n].tolist())
        assert len(got) == k, f"row {n}: duplicate indices"
        want = set(torch.topk(pre_ref[n], k).indices.tolist())
        if got != want:
            kth = float(top[n, k - 1])
            nxt = float(top[n, k]) if top.shape[1] > k else kth
            if abs(kth - nxt) > rel_gap * max(abs(kth), 1e-12):
                bad += 1
    assert bad == 0, f"{bad} rows differ beyond the tie rule"
    # the reported values are the pre-activations at the reported indices
    picked = pre_ref.gather(1, idx_gpu)
    assert rel_l2(vals_gpu, picked) < ACT_TOL


# ----------------------------------------------------------------------------- decode
@pytest.mark.parametrize("d_in", [48, 64])
def test_decode_golden(cuda_lib, d_in):
    from sparsify_b200 import ops
    t, _ = load_golden(f"decoder_d{d_in}")
    out = ops.embedding_bag_fwd(dev(t["idx"]), dev(t["acts"]), dev(t["W_dec"]))
    assert rel_l2(out, t["out"]) < F32_TOL
    gacts = ops.embedding_bag_bwd_acts(dev(t["idx"]), dev(t["gout"]), dev(t["W_dec"]))
    assert rel_l2(gacts, t["gacts"]) < F32_TOL
    M, D = t["W_dec"].shape
    row_ptr, entries = ops.csr_build(dev(t["idx"]), M)
    res = ops.rows_accumulate(row_ptr, entries, t["idx"].shape[1], M, D, dev(t["acts"]), dev(t["gout"]))
    assert rel_l2(res["gradA"], t["gW"]) < F32_TOL


@pytest.mark.parametrize("N,D,M,k,wdtype", [
    (257, 768, 4096, 32, torch.float32),
    (300, 4096, 8192, 32, torch.bfloat16),
    (64, 1024, 2048, 64, torch.bfloat16),
    (5, 52, 96, 3, torch.float32),
    (33, 520, 300, 7, torch.bfloat16),      # k below one register group, ragged width
    (40, 1024, 4096, 100, torch.bfloat16),  # several register groups, the last one partial
    (3, 256, 4096, 1100, torch.bfloat16),   # more entries than the register-staged kernel stages
])
def test_decode_oracle(cuda_lib, N, D, M, k, wdtype):
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(1)
    W = torch.randn(M, D, generator=g)
    if wdtype == torch.bfloat16:
        W = bf16_round(W)
    b = torch.randn(D, generator=g)
    acts = torch.rand(N, k, generator=g)
    idx = torch.stack([torch.randperm(M, generator=g)[:k] for _ in range(N)])
    gout = torch.randn(N, D, generator=g)
    Wd = W.cuda().to(wdtype)
    out = ops.embedding_bag_fwd(idx.cuda(), acts.cuda(), Wd, b.cuda())
    assert rel_l2(out, O.decode(idx, acts, W, b)) < F32_TOL
    gW_ref, gacts_ref = O.decode_backward(idx, acts, W, gout)
    gacts = ops.embedding_bag_bwd_acts(idx.cuda(), gout.cuda(), Wd)
    assert rel_l2(gacts, gacts_ref) < F32_TOL
    row_ptr, entries = ops.csr_build(idx.cuda(), M)
    res = ops.rows_accumulate(row_ptr, entries, k, M, D, acts.cuda(), gout.cuda(), biasA=True)
    assert rel_l2(res["gradA"], gW_ref) < F32_TOL
    gb_ref = torch.zeros(M).index_add_(0, idx.reshape(-1), acts.reshape(-1))
    assert rel_l2(res["gbiasA"], gb_ref) < F32_TOL


def test_csr_exact(cuda_lib):
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(2)
    N, k, M = 3000, 16, 512
    idx = torch.stack([torch.randperm(M, generator=g)[:k] for _ in range(N)])
    idx[:, 0] = 7  # one very hot latent (N entries > the in-kernel sort limit)
    rest = idx[:, 1:]
    rest[rest == 7] = 8  # (duplicates inside a row are harmless for the CSR)
    row_ptr, entries = ops.csr_build(idx.cuda(), M)
    ref_ptr, ref_order = O.csr_by_latent(idx, M)
    assert torch.equal(row_ptr.cpu().long(), ref_ptr)
    entries = entries.cpu().long()
    for m in range(M):
        lo, hi = int(ref_ptr[m]), int(ref_ptr[m + 1])
        seg = entries[lo:hi]
        assert torch.equal(seg, ref_order[lo:hi]), m  # ascending flat positions, long segments too


def test_csr_long_segments_exact(cuda_lib):
    """Latents hit by more tokens than the in-warp sort holds (2048): lengths just above the limit,
    a non-power-of-two length and one latent that every token selects."""
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(21)
    N, k, M = 70000, 4, 64
    idx = torch.randint(8, M, (N, k), generator=g)
    idx[:, 0] = 3                       # N entries
    idx[:2049, 1] = 5                   # one above the limit
    idx[10000:15001, 2] = 6             # 5001 entries
    row_ptr, entries = ops.csr_build(idx.cuda(), M)
    ref_ptr, ref_order = O.csr_by_latent(idx, M)
    assert torch.equal(row_ptr.cpu().long(), ref_ptr)
    assert torch.equal(entries.cpu().long(), ref_order)


def test_csr_empty_and_ragged(cuda_lib):
    from sparsify_b200 import ops
    idx = torch.zeros(0, 4, dtype=torch.int64, device="cuda")
    row_ptr, _ = ops.csr_build(idx, 16)
    assert int(row_ptr.abs().sum()) == 0
    out = ops.embedding_bag_fwd(idx, torch.zeros(0, 4, device="cuda"), torch.randn(16, 8, device="cuda"))
    assert out.shape == (0, 8)


# ----------------------------------------------------------------------------- encoder
def test_encoder_dense_golden(cuda_lib):
    from sparsify_b200 import ops
    t, meta = load_golden("encoder_topk")
    pre = ops.preacts_dense(dev(t["x"]), dev(t["W"]), dev(t["b"]))
    assert rel_l2(pre, t["pre"]) < F32_TOL
    vals, idx = ops.topk_rows(pre, meta["k"])
    vals, idx = sort_topk(vals.cpu(), idx.cpu())
    assert torch.equal(idx, t["idx"])
    assert rel_l2(vals, t["vals"]) < F32_TOL
    t, meta = load_golden("encoder_groupmax")
    pre = ops.preacts_dense(dev(t["x"]), dev(t["W"]), dev(t["b"]))
    vals, idx = ops.groupmax_rows(pre, meta["k"])
    vals, idx = sort_topk(vals.cpu(), idx.cpu())
    assert torch.equal(idx, t["idx"])


def test_topk_rows_masked(cuda_lib):
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(3)
    N, M, k = 37, 5000, 200
    pre = torch.randn(N, M, generator=g).clamp_min(0)  # many exact zeros (ties)
    mask = torch.rand(M, generator=g) < 0.3
    vals, idx = ops.topk_rows(pre.cuda(), k, col_mask=mask.cuda())
    vals, idx = vals.cpu(), idx.cpu()
    masked = torch.where(mask[None], pre, torch.full_like(pre, -float("inf")))
    ref_vals = torch.topk(masked, k).values
    assert torch.equal(vals.sort(-1, descending=True).values, ref_vals)
    assert bool(mask[idx].all())
    assert torch.equal(pre.gather(1, idx), vals)
    for n in range(N):
        assert len(set(idx[n].tolist())) == k


@pytest.mark.parametrize("N,D,M,k", [
    (128, 64, 256, 8),       # one tile, one k-chunk
    (200, 256, 1024, 32),    # ragged rows, several tiles
    (384, 1024, 4352, 32),   # ragged last column tile (4352 = 17 * 256)
    (130, 72, 520, 64),      # D not a multiple of 64, M not a multiple of 256
    (1024, 4096, 16384, 32), # config-1 width, reduced N and M
    (77, 64, 300, 5),        # k not a multiple of the list group size
    (256, 128, 2048, 128),   # largest k of the fused path (Multi-TopK of k=32)
    (64, 64, 40, 40),        # k == M: every latent is selected
])
def test_encoder_tc_vs_oracle(cuda_lib, N, D, M, k):
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(4)
    x = bf16_round(torch.randn(N, D, generator=g))
    W = bf16_round(torch.randn(M, D, generator=g) / D ** 0.5)
    b = 0.1 * torch.randn(M, generator=g)
    vals, idx = ops.encode_topk_tc(x.cuda().bfloat16(), W.cuda().bfloat16(), b.cuda(), k)
    torch.cuda.synchronize()
    assert int(ops.encode_topk_tc.last_status[0].item()) == 0
    pre = O.preacts(x.double(), W.double(), b.double()).float()
    check_topk_sets(vals, idx, pre, k)


@pytest.mark.parametrize("N,D,M,k", [
    (200, 256, 1024, 32),
    (384, 1024, 4352, 32),
    (1024, 4096, 16384, 32),
    (300, 128, 2048, 128),
])
def test_encoder_tc_cta_pair_form(cuda_lib, N, D, M, k):
    """The encoder's CTA-pair form (tcgen05 cta_group::2) must give the answer of the default form."""
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(40)
    x = bf16_round(torch.randn(N, D, generator=g)).cuda().bfloat16()
    W = bf16_round(torch.randn(M, D, generator=g) / D ** 0.5).cuda().bfloat16()
    b = (0.1 * torch.randn(M, generator=g)).cuda()
    try:
        ops.set_cta_pairs(False)
        vals1, idx1 = ops.encode_topk_tc(x, W, b, k)
        ops.set_cta_pairs(True)
        vals2, idx2 = ops.encode_topk_tc(x, W, b, k)
        torch.cuda.synchronize()
    finally:
        ops.set_cta_pairs(None)  # back to the per-shape choice
    ops.check_status(x.device)
    pre = O.preacts(x.cpu().double(), W.cpu().double(), b.cpu().double()).float()
    check_topk_sets(vals1, idx1, pre, k)
    check_topk_sets(vals2, idx2, pre, k)
    # same accumulation order per output element in both forms: the values agree exactly
    assert torch.equal(vals1, vals2) and torch.equal(idx1, idx2)


def test_encoder_tc_few_positive(cuda_lib):
    """Rows with fewer than k positive pre-activations still return k distinct
    valid indices (zeros fill the tail), as torch.topk over post-ReLU values does."""
    from sparsify_b200 import ops
    N, D, M, k = 128, 64, 512, 16
    x = torch.ones(N, D)
    W = -torch.ones(M, D) / D
    W[:5] = 1.0 / D
    b = torch.zeros(M)
    vals, idx = ops.encode_topk_tc(x.cuda().bfloat16(), W.cuda().bfloat16(), b.cuda(), k)
    vals, idx = vals.cpu(), idx.cpu()
    for n in range(N):
        assert len(set(idx[n].tolist())) == k
        assert set(idx[n, vals[n] > 0].tolist()) == {0, 1, 2, 3, 4}
    assert bool(((idx >= 0) & (idx < M)).all())


# ----------------------------------------------------------------------------- losses / optimiser
def test_losses(cuda_lib):
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(5)
    y = torch.randn(1000, 96, generator=g) * torch.rand(96, generator=g) * 5 + 3
    out = torch.randn(1000, 96, generator=g)
    tv = ops.total_variance(y.cuda())
    ref = (y.double() - y.double().mean(0)).pow(2).sum()
    assert abs(float(tv) - float(ref)) < 1e-5 * float(ref)
    sse, diff = ops.sq_err(y.cuda(), out.cuda(), want_diff=True)
    assert abs(float(sse) - float((y.double() - out.double()).pow(2).sum())) < 1e-5 * float(sse)
    assert torch.equal(diff.cpu(), y - out)


def test_normalize_and_adam(cuda_lib):
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(6)
    M, D = 300, 200
    W = torch.randn(M, D, generator=g)
    Wg = W.clone().cuda()
    shadow = torch.empty(M, D, dtype=torch.bfloat16, device="cuda")
    ops.normalize_rows_(Wg, torch.finfo(torch.float32).eps, shadow)
    ref = W.clone()
    O.normalize_decoder_(ref)
    assert rel_l2(Wg, ref) < 1e-6
    assert torch.equal(shadow.cpu(), Wg.cpu().bfloat16())
    for project in (False, True):
        p, gr = ref.clone(), torch.randn(M, D, generator=g)
        m, v = torch.zeros(M, D), torch.zeros(M, D)
        pg, gg, mg, vg = p.clone().cuda(), gr.clone().cuda(), m.clone().cuda(), v.clone().cuda()
        for step in (1, 2, 3):
            if project:
                O.project_out_parallel_(gr, p)
            O.adam_step_(p, gr, m, v, step, 1e-3)
            ops.adam_rows_(pg, gg, mg, vg, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, step=step,
                           project=project)
        assert rel_l2(pg, p) < 1e-6 and rel_l2(mg, m) < 1e-5 and rel_l2(vg, v) < 5e-5


# ----------------------------------------------------------------------------- dense GEMM / Muon
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 520, 264), (1024, 4096, 1024), (4096, 1000, 72)])
def test_gemm_tc(cuda_lib, M, N, K):
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(8)
    A = bf16_round(torch.randn(M, K, generator=g))
    B = bf16_round(torch.randn(N, K, generator=g))
    C = bf16_round(torch.randn(M, N, generator=g))
    bias = torch.randn(N, generator=g)
    ref = 0.5 * (A.double() @ B.double().T) - 1.5 * C.double() + bias.double()
    out = ops.gemm_nt(A.cuda().bfloat16(), B.cuda().bfloat16(), alpha=0.5, beta=-1.5, Cin=C.cuda().bfloat16(),
                      bias=bias.cuda(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert int(ops.gemm_nt.last_status[0]) == 0
    assert rel_l2(out, ref) < 1e-5
    out_bf = ops.gemm_nt(A.cuda().bfloat16(), B.cuda().bfloat16(), relu=True)
    assert rel_l2(out_bf.float(), (A.double() @ B.double().T).clamp_min(0)) < 4e-3  # bf16 output rounding
    t = ops.transpose_bf16(A.cuda().bfloat16())
    assert torch.equal(t.cpu(), A.bfloat16().T.contiguous())


@pytest.mark.parametrize("M,K", [(640, 512), (1000, 264), (128, 64), (2048 + 128, 128)])
def test_gemm_symmetric(cuda_lib, M, K):
    """X X^T and bA + cAA with only the tiles that reach the upper triangle computed:
    same values as the full product, and exactly symmetric."""
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(M + K)
    X = torch.randn(M, K, generator=g).cuda().bfloat16()
    full = ops.gemm_nt(X, X, out_dtype=torch.float32)
    sym = ops.gemm_nt(X, X, out_dtype=torch.float32, symmetric=True)
    torch.cuda.synchronize()
    assert int(ops.gemm_nt.last_status[0]) == 0
    assert torch.equal(sym, sym.T)
    assert torch.equal(sym.triu(), full.triu())
    assert rel_l2(sym, X.double() @ X.double().T) < 1e-5
    if M % 8 == 0:
        A = sym.bfloat16()
        B = ops.gemm_nt(A, A, alpha=0.25, beta=-1.0, Cin=A, symmetric=True)
        want = 0.25 * (A.double() @ A.double().T) - A.double()
        assert torch.equal(B, B.T) and rel_l2(B.float(), want) < 4e-3


@pytest.mark.parametrize("M,N,K", [(300, 520, 128), (1024, 256, 64)])
def test_gemm_transposed_copy(cuda_lib, M, N, K):
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(M)
    A = torch.randn(M, K, generator=g).cuda().bfloat16()
    B = torch.randn(N, K, generator=g).cuda().bfloat16()
    C = torch.randn(M, N, generator=g).cuda().bfloat16()
    for dt in (torch.bfloat16, torch.float32):
        out_t = torch.empty(N, M, dtype=dt, device="cuda")
        out = ops.gemm_nt(A, B, alpha=1.0, beta=0.5, Cin=C, out_dtype=dt, out_t=out_t)
        assert torch.equal(out_t, out.T)
        assert rel_l2(out.float(), A.double() @ B.double().T + 0.5 * C.double()) < (4e-3 if dt == torch.bfloat16 else 1e-5)


def test_newtonschulz_tc_vs_oracle(cuda_lib):
    from sparsify_b200.muon import quintic_newtonschulz
    for name in ("wide", "tall"):
        t, _ = load_golden(f"newtonschulz_{name}")
        X = quintic_newtonschulz(t["G"].cuda(), 5).float().cpu()
        assert X.shape == t["G"].shape
        assert rel_l2(X, t["X"]) < 8e-2  # bf16 iteration: rounding differences grow over 5 steps
    g = torch.Generator().manual_seed(9)
    G = torch.randn(256, 1024, generator=g)
    X = quintic_newtonschulz(G.cuda(), 5).float().cpu()
    ref = O.quintic_newtonschulz(G, 5).float()
    assert rel_l2(X, ref) < 8e-2
    s = torch.linalg.svdvals(X)
    assert float(s.max()) < 1.6 and float(s.min()) > 0.3  # singular values pushed towards 1


@pytest.mark.parametrize("ydtype", [torch.float32, torch.bfloat16])
def test_decode_residual(cuda_lib, ydtype):
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(12)
    N, D, M, k = 300, 768, 4096, 32
    W = bf16_round(torch.randn(M, D, generator=g))
    b = torch.randn(D, generator=g)
    acts = torch.rand(N, k, generator=g)
    idx = torch.stack([torch.randperm(M, generator=g)[:k] for _ in range(N)])
    y = torch.randn(N, D, generator=g)
    if ydtype == torch.bfloat16:
        y = bf16_round(y)
    out, e32, e16, sse = ops.decode_residual(idx.cuda(), acts.cuda(), W.cuda().bfloat16(), b.cuda(),
                                             y.cuda().to(ydtype), want_e32=True, want_e16=True)
    ref_out = O.decode(idx, acts, W, b)
    ref_e = y - ref_out
    assert rel_l2(out, ref_out) < F32_TOL
    assert rel_l2(e32, ref_e) < F32_TOL
    assert torch.equal(e16.cpu(), e32.cpu().bfloat16())
    assert abs(float(sse) - float(ref_e.double().pow(2).sum())) < 1e-5 * float(sse)
    tv = ops.total_variance(y.cuda().to(ydtype))
    ref_tv = (y.double() - y.double().mean(0)).pow(2).sum()
    assert abs(float(tv) - float(ref_tv)) < 1e-5 * float(ref_tv)
    gacts16 = ops.embedding_bag_bwd_acts(idx.cuda(), e16, W.cuda().bfloat16())
    _, gacts_ref = O.decode_backward(idx, acts, W, e16.float().cpu())
    assert rel_l2(gacts16, gacts_ref) < F32_TOL


@pytest.mark.parametrize("N,D,M,k,ydtype,both", [
    (300, 4096, 2048, 32, torch.bfloat16, False),   # the training step's case: bf16 residual only
    (65, 520, 300, 7, torch.float32, True),         # ragged width, fp32 residual kept
    (130, 1024, 512, 32, torch.bfloat16, False),    # every register slot in use
    (33, 260, 100, 20, torch.float32, True),        # ragged width and k, fp32 residual kept
])
def test_decode_residual_dots(cuda_lib, N, D, M, k, ydtype, both):
    """sc_decode_residual_dots: the decode / residual outputs equal sc_decode_residual's bit for bit,
    and the dots equal sc_embedding_bag_bwd_acts on the stored residual (up to summation order) and
    the fp64 dot products; entries with an id outside [0, M) contribute nothing and get dot 0."""
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(N + k)
    W = bf16_round(torch.randn(M, D, generator=g))
    b = torch.randn(D, generator=g)
    acts = torch.rand(N, k, generator=g)
    idx = torch.stack([torch.randperm(M, generator=g)[:k] for _ in range(N)])
    idx[0, 0], idx[N - 1, k - 1] = -1, M          # invalid ids
    y = torch.randn(N, D, generator=g)
    if ydtype == torch.bfloat16:
        y = bf16_round(y)
    Wc, args = W.cuda().bfloat16(), (idx.cuda(), acts.cuda())
    assert ops.decode_dots_supported(Wc, k)
    kw = dict(want_out=both, want_e32=both, want_e16=True)
    out, e32, e16, sse = ops.decode_residual(*args, Wc, b.cuda(), y.cuda().to(ydtype), **kw)
    out2, e32b, e16b, sse2, dots = ops.decode_residual(*args, Wc, b.cuda(), y.cuda().to(ydtype), want_dots=True, **kw)
    assert torch.equal(e16, e16b)
    if both:
        assert torch.equal(out, out2) and torch.equal(e32, e32b)
    assert abs(float(sse) - float(sse2)) <= 1e-6 * float(sse)
    stored = e32 if both else e16
    sep = ops.embedding_bag_bwd_acts(args[0], stored, Wc)
    assert rel_l2(dots, sep) < 1e-5
    valid = (idx >= 0) & (idx < M)
    rows = W.double()[idx.clamp(0, M - 1)]                       # [N, k, D]
    ref = torch.einsum("nd,nkd->nk", stored.double().cpu(), rows) * valid
    assert rel_l2(dots, ref.float()) < F32_TOL
    assert float(dots[0, 0]) == 0.0 and float(dots[N - 1, k - 1]) == 0.0
    assert not ops.decode_dots_supported(Wc, 33)      # wider selections keep the two separate kernels


@pytest.mark.parametrize("n", [4096 * 3, 1001])
def test_signum_schedulefree_kernel(cuda_lib, n):
    """sc_signum_schedulefree against the oracle's restatement, several steps, with the bf16 copy."""
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(n)
    y = torch.randn(n, generator=g); z = y.clone()
    yd, zd = y.cuda(), z.cuda()
    shadow = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    lr, beta, wsum = 3e-3, 0.95, 0.0
    for step in range(4):
        grad = torch.randn(n, generator=g)
        grad[::7] = 0.0  # sign(0) = 0
        wsum += lr ** 2
        c = lr ** 2 / wsum
        O.signum_schedulefree_step_(y, z, grad, lr, beta, c)
        ops.signum_schedulefree_(yd, zd, grad.cuda(), lr, beta, c, shadow)
    assert rel_l2(yd, y) < 1e-6 and rel_l2(zd, z) < 1e-6
    assert torch.equal(shadow, yd.bfloat16())


def test_project_rows_kernel(cuda_lib):
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(3)
    grad, w = torch.randn(37, 100, generator=g), torch.nn.functional.normalize(torch.randn(37, 100, generator=g), dim=1)
    want = grad.clone()
    O.project_out_parallel_(want, w)
    gd = grad.cuda()
    ops.project_rows_(gd, w.cuda())
    assert rel_l2(gd, want) < 1e-6


def test_muon_elementwise_kernels(cuda_lib):
    """Momentum + Nesterov + bf16 cast + sum of squares, the scaled transpose and the
    decay + update pass against the tensor expressions of sparsify/muon.py."""
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(12)
    R, C, beta = 72, 40, 0.95
    grad, buf = torch.randn(R, C, generator=g), torch.randn(R, C, generator=g)
    want_buf = buf.clone().lerp_(grad, 1 - beta)
    want_u = grad.clone().lerp_(want_buf, beta).bfloat16()
    bd = buf.cuda()
    xb, sumsq = ops.muon_momentum_(grad.cuda(), bd, beta, True)
    assert rel_l2(bd, want_buf) < 1e-6
    assert (xb.cpu().float() - want_u.float()).abs().max() <= 2 ** -7 * want_u.float().abs().max()
    assert abs(float(sumsq) - float(xb.float().pow(2).sum())) < 1e-4 * float(sumsq)
    want = xb.cpu() / (xb.cpu().norm() + 1e-7)          # bf16 arithmetic, as the reference normalises
    s_, t_ = ops.scale_transpose_bf16(xb, sumsq)
    assert torch.equal(s_.cpu(), want) and torch.equal(t_.cpu(), want.T.contiguous())
    p = torch.randn(R, C, generator=g)
    pd, shadow = p.cuda(), torch.empty(R, C, dtype=torch.bfloat16, device="cuda")
    ops.muon_apply_(pd, s_, 0.999, 0.03, shadow)
    want_p = p * 0.999 - 0.03 * want.float()
    assert rel_l2(pd, want_p) < 1e-6 and torch.equal(shadow, pd.bfloat16())


@pytest.mark.parametrize("N,D,M,k", [(200, 128, 4096, 8), (130, 64, 2048, 32), (300, 256, 3072, 4),
                                      (128, 64, 192, 3), (1000, 128, 16384, 64)])
def test_encode_groupmax_tc(cuda_lib, N, D, M, k):
    """Groupmax in the tensor-core encoder against the oracle on the same bf16-rounded
    operands (fused_encoder.py:34-43): group sizes below, equal to and above one tile."""
    from sparsify_b200 import ops
    assert ops.tc_groupmax_supported(D, M, k)
    g = torch.Generator().manual_seed(N + M)
    x = bf16_round(torch.randn(N, D, generator=g))
    W = bf16_round(torch.randn(M, D, generator=g) / D ** 0.5)
    b = 0.1 * torch.randn(M, generator=g)
    vals, idx = ops.encode_groupmax_tc(x.cuda().bfloat16(), W.cuda().bfloat16(), b.cuda(), k)
    torch.cuda.synchronize()
    assert int(ops.encode_groupmax_tc.last_status[0]) == 0
    pre = O.preacts(x, W, b)
    rv, ri = O.groupmax(pre, k)
    vals, idx = vals.cpu(), idx.cpu()
    assert rel_l2(vals, rv) < 1e-5
    # the chosen latent lies in its group and holds (up to accumulation order) the group's maximum
    gsz = M // k
    assert torch.equal(idx // gsz, torch.arange(k).expand(N, k))
    assert (pre.gather(1, idx) - rv).abs().max() < 1e-4
    assert (idx == ri).float().mean() > 0.999


def test_topk_mask_rows(cuda_lib):
    """Dense bf16 row with everything but the k largest entries zeroed, against torch.topk."""
    from sparsify_b200 import ops
    g = torch.Generator().manual_seed(21)
    pre = torch.randn(37, 1000, generator=g).clamp_min(0)  # post-ReLU: many ties at zero
    k = 300
    out = ops.topk_mask_rows(pre.cuda(), k).cpu()
    vals, idx = pre.topk(k, dim=1)
    want = torch.zeros_like(pre).scatter_(1, idx, vals).bfloat16()
    assert torch.equal(out, want)
    mask = torch.zeros(1000, dtype=torch.bool); mask[::3] = True
    out = ops.topk_mask_rows(pre.cuda(), 50, col_mask=mask.cuda()).cpu()
    vals, idx = torch.where(mask, pre, torch.full_like(pre, -1.0)).topk(50, dim=1)
    assert torch.equal(out, torch.zeros_like(pre).scatter_(1, idx, vals).bfloat16())
