"""SparseCoder / fused_encoder / decoder_impl on the GPU against the
reference-generated fixtures (fp32 mode) and against the oracle evaluated on
the same bf16-rounded operands (bf16 mode)."""

import pytest
import torch

from oracle import sae_oracle as O
from tests.conftest import load_golden, rel_l2, sort_topk

pytestmark = pytest.mark.gpu


def build_sae(t, cfg_dict, precision):
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    cfg = SparseCoderConfig(**cfg_dict)
    D = t["param.b_dec"].numel()
    sae = SparseCoder(D, cfg, device="cuda", dtype=torch.float32)
    sae.precision = precision
    with torch.no_grad():
        sae.encoder.weight.copy_(t["param.W_enc"])
        sae.encoder.bias.copy_(t["param.b_enc"])
        sae.W_dec.copy_(t["param.W_dec"])
        sae.b_dec.copy_(t["param.b_dec"])
        if "param.W_skip" in t:
            sae.W_skip.copy_(t["param.W_skip"])
    return sae


@pytest.mark.parametrize("name", ["sae_plain", "sae_auxk", "sae_multitopk", "transcoder_skip"])
def test_forward_backward_fp32_golden(cuda_lib, name):
    t, meta = load_golden(f"forward_{name}")
    sae = build_sae(t, meta["cfg"], "fp32")
    x = t["x"].cuda()
    y = t["y"].cuda() if "y" in t else None
    dead = t["dead_mask"].cuda() if "dead_mask" in t else None
    out = sae(x, y, dead_mask=dead)
    loss = out.fvu + meta["auxk_alpha"] * out.auxk_loss + out.multi_topk_fvu / 8
    loss.backward()
    acts, idx = sort_topk(out.latent_acts.detach().cpu(), out.latent_indices.cpu())
    assert torch.equal(idx, t["latent_indices"])
    assert rel_l2(acts, t["latent_acts"]) < 2e-5
    assert rel_l2(out.sae_out.detach(), t["sae_out"]) < 2e-5
    for key in ("fvu", "auxk_loss", "multi_topk_fvu"):
        assert abs(float(getattr(out, key)) - float(t[key])) <= 2e-5 * max(1.0, abs(float(t[key]))), key
    grads = {"W_enc": sae.encoder.weight.grad, "b_enc": sae.encoder.bias.grad,
             "W_dec": sae.W_dec.grad, "b_dec": sae.b_dec.grad}
    if sae.W_skip is not None:
        grads["W_skip"] = sae.W_skip.grad
    for pname, g in grads.items():
        ref = t[f"grad.{pname}"]
        if float(ref.norm()) == 0:
            assert g is None or float(g.norm()) < 1e-7, pname
        else:
            assert rel_l2(g, ref) < 1e-4, (pname, rel_l2(g, ref))


def test_fused_encoder_golden(cuda_lib):
    from sparsify_b200 import fused_encoder
    for tag in ("topk", "groupmax"):
        t, meta = load_golden(f"encoder_{tag}")
        x = t["x"].cuda().requires_grad_(True)
        W = t["W"].cuda().requires_grad_(True)
        b = t["b"].cuda().requires_grad_(True)
        vals, idx, pre = fused_encoder(x, W, b, meta["k"], meta["activation"])
        assert rel_l2(pre, t["pre"]) < 2e-5
        order = torch.argsort(vals, dim=-1, descending=True, stable=True)
        assert torch.equal(idx.gather(-1, order).cpu(), t["idx"])
        (vals.gather(-1, order) * t["coef"].cuda()).sum().backward()
        assert rel_l2(x.grad, t["gx"]) < 2e-5
        assert rel_l2(W.grad, t["gW"]) < 2e-5
        assert rel_l2(b.grad, t["gb"]) < 2e-5
    with pytest.raises(ValueError):
        fused_encoder(x, W, b, 4, "softmax")


@pytest.mark.parametrize("d_in", [48, 64])
def test_decoder_impl_like_reference_test(cuda_lib, d_in):
    """Shapes of the reference's tests/test_decode.py."""
    from sparsify_b200.utils import decoder_impl
    t, _ = load_golden(f"decoder_d{d_in}")
    W = t["W_dec"].cuda().requires_grad_(True)
    acts = t["acts"].cuda().requires_grad_(True)
    out = decoder_impl(t["idx"].cuda(), acts, W.mT)
    torch.testing.assert_close(out.cpu(), t["out"])
    (out * t["gout"].cuda()).sum().backward()
    torch.testing.assert_close(W.grad.cpu(), t["gW"])
    torch.testing.assert_close(acts.grad.cpu(), t["gacts"])


def test_forward_backward_bf16_vs_oracle(cuda_lib):
    """bf16 configuration: tensor-core encoder and bf16 row gathers, compared
    with the oracle fed the same bf16-rounded operands."""
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    torch.manual_seed(0)
    N, D, M, k = 512, 256, 4096, 32
    sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=k), device="cuda", dtype=torch.float32)
    assert sae.precision == "bf16"
    g = torch.Generator().manual_seed(9)
    atoms = torch.nn.functional.normalize(torch.randn(2048, D, generator=g), dim=1)
    ids = torch.randint(0, 2048, (N, 16), generator=g)
    x = (atoms[ids] * torch.rand(N, 16, 1, generator=g)).sum(1) + 0.05 * torch.randn(N, D, generator=g)
    with torch.no_grad():
        sae.b_dec.copy_(x.mean(0))
    out = sae(x.cuda())
    out.fvu.backward()
    rnd = lambda t: t.to(torch.bfloat16).to(torch.float32)
    params = dict(W_enc=sae.encoder.weight.detach().cpu(), b_enc=sae.encoder.bias.detach().cpu(),
                  W_dec=sae.W_dec.detach().cpu(), b_dec=sae.b_dec.detach().cpu())
    ref = O.sae_forward_backward(params, x, cfg=O.OracleCfg(k=k), round_operands=rnd)
    acts, idx = sort_topk(out.latent_acts.detach().cpu(), out.latent_indices.cpu())
    racts, ridx = sort_topk(ref.latent_acts, ref.latent_indices)
    # index sets identical except where the k-th and (k+1)-th pre-activations are within 1e-3 (relative)
    from tests.test_kernels_gpu import check_topk_sets
    pre = O.preacts(rnd(x - params["b_dec"]).double(), rnd(params["W_enc"]).double(), params["b_enc"].double()).float()
    check_topk_sets(out.latent_acts.detach(), out.latent_indices, pre, k)
    assert rel_l2(acts, racts) < 1e-3
    assert rel_l2(out.sae_out.detach(), ref.sae_out) < 1e-3
    assert abs(float(out.fvu) - float(ref.fvu)) < 1e-3 * float(ref.fvu)
    for pname, gt in (("W_enc", sae.encoder.weight.grad), ("b_enc", sae.encoder.bias.grad),
                      ("W_dec", sae.W_dec.grad), ("b_dec", sae.b_dec.grad)):
        assert rel_l2(gt, ref.grads[pname]) < 1e-2, (pname, rel_l2(gt, ref.grads[pname]))


def test_checkpoint_roundtrip(cuda_lib, tmp_path):
    from safetensors import safe_open
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    sae = SparseCoder(32, SparseCoderConfig(num_latents=128, k=4, skip_connection=True), device="cuda")
    sae.save_to_disk(tmp_path / "ckpt")
    with safe_open(str(tmp_path / "ckpt" / "sae.safetensors"), framework="pt") as f:
        assert sorted(f.keys()) == ["W_dec", "W_skip", "b_dec", "encoder.bias", "encoder.weight"]
    back = SparseCoder.load_from_disk(tmp_path / "ckpt", device="cuda")
    for (n1, p1), (n2, p2) in zip(sae.named_parameters(), back.named_parameters()):
        assert n1 == n2 and torch.equal(p1, p2)


def test_cpu_tensors_are_rejected():
    from sparsify_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.embedding_bag_fwd(torch.zeros(2, 2, dtype=torch.long), torch.zeros(2, 2), torch.zeros(4, 4))


@pytest.mark.parametrize("precision,tol,D,M", [("mixed", 1e-5, 256, 4096), ("bf16", 5e-3, 256, 4096),
                                                ("mixed", 1e-5, 5120, 1024)])
def test_sparse_fused_update_matches_dense_path(cuda_lib, precision, tol, D, M):
    """sc_rows_adam (gradients applied in sparse form: projection, Adam, decoder
    normalisation, bf16 copies in one kernel) against the separate kernels."""
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    from sparsify_b200.optim import FusedAdam
    N, k = 1024, 32   # D = 5120: rows wider than 4096 take the kernel's eight-groups-per-thread form
    g = torch.Generator().manual_seed(21)
    xs = [torch.randn(N, D, generator=g).cuda() for _ in range(3)]
    models = []
    for sparse in (False, True):
        torch.manual_seed(0)
        sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=k), device="cuda", dtype=torch.float32)
        sae.precision = precision
        opt = FusedAdam(sae.parameters(), lr=1e-3)
        sae.attach_optimizer(opt)
        if sparse:
            assert opt.enable_sparse_update(sae)
        for x in xs:
            sae.set_decoder_norm_to_unit_norm()
            out = sae(x)
            out.fvu.backward()
            if sparse:
                assert sae.W_dec.grad is None and sae._pending is not None
            opt.step()
            opt.zero_grad(set_to_none=True)
        sae.set_decoder_norm_to_unit_norm()
        models.append((sae, opt))
    (a, oa), (b, ob) = models
    for (n1, p1), (_, p2) in zip(a.named_parameters(), b.named_parameters()):
        # "mixed": both paths use fp32 residual rows (same arithmetic, tight bound);
        # "bf16": the sparse path gathers the residual rows as bf16, the dense one as fp32
        assert rel_l2(p2.detach(), p1.detach()) < tol, n1
    for name in ("encoder.weight",) + (("W_dec",) if precision == "bf16" else ()):
        assert torch.equal(b.shadow(name), dict(b.named_parameters())[name].detach().bfloat16()), name
    sa, sb = oa.state[a.W_dec], ob.state[b.W_dec]
    assert int(sa["step"]) == int(sb["step"]) == 3
    assert rel_l2(sb["exp_avg"], sa["exp_avg"]) < 10 * tol and rel_l2(sb["exp_avg_sq"], sa["exp_avg_sq"]) < 100 * tol
    norms = b.W_dec.detach().norm(dim=1)
    assert torch.allclose(norms, torch.ones_like(norms), atol=1e-5)


def test_transcoder_skip_bf16_vs_oracle(cuda_lib):
    """Transcoder with a dense skip connection in the bf16 configuration: the skip
    product and its gradients run on the tcgen05 GEMM."""
    t, meta = load_golden("forward_transcoder_skip")
    sae = build_sae(t, meta["cfg"], "bf16")
    out = sae(t["x"].cuda(), t["y"].cuda())
    out.fvu.backward()
    assert abs(float(out.fvu) - float(t["fvu"])) < 2e-2 * float(t["fvu"])
    assert rel_l2(out.sae_out.detach(), t["sae_out"]) < 2e-2
    assert rel_l2(sae.W_skip.grad, t["grad.W_skip"]) < 3e-2
    assert rel_l2(sae.W_dec.grad, t["grad.W_dec"]) < 3e-2


@pytest.mark.parametrize("n_dead", [100, 300])
def test_auxk_fused_bf16_vs_oracle(cuda_lib, n_dead):
    """AuxK inside the fused step (dead pre-activations and the auxiliary
    reconstruction as small tensor-core GEMMs) against the oracle on the same
    bf16-rounded operands; n_dead below and above k_aux = D/2."""
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    torch.manual_seed(0)
    N, D, M, k, alpha = 512, 256, 4096, 32, 1 / 32
    sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=k), device="cuda", dtype=torch.float32)
    g = torch.Generator().manual_seed(31)
    x = torch.randn(N, D, generator=g)
    dead = torch.zeros(M, dtype=torch.bool)
    dead[torch.randperm(M, generator=g)[:n_dead]] = True
    with torch.no_grad():
        sae.b_dec.copy_(0.1 * torch.randn(D, generator=g))
        sae.encoder.bias.copy_(0.05 * torch.randn(M, generator=g))
    out = sae(x.cuda(), dead_mask=dead.cuda())
    (out.fvu + alpha * out.auxk_loss).backward()
    rnd = lambda t: t.to(torch.bfloat16).to(torch.float32)
    params = dict(W_enc=sae.encoder.weight.detach().cpu(), b_enc=sae.encoder.bias.detach().cpu(),
                  W_dec=sae.W_dec.detach().cpu(), b_dec=sae.b_dec.detach().cpu())
    ref = O.sae_forward_backward(params, x, dead_mask=dead, cfg=O.OracleCfg(k=k), auxk_alpha=alpha,
                                 round_operands=rnd)
    assert float(ref.auxk_loss) > 0
    assert abs(float(out.auxk_loss) - float(ref.auxk_loss)) < 1e-2 * float(ref.auxk_loss)
    assert abs(float(out.fvu) - float(ref.fvu)) < 1e-3 * float(ref.fvu)
    for pname, gt in (("W_enc", sae.encoder.weight.grad), ("b_enc", sae.encoder.bias.grad),
                      ("W_dec", sae.W_dec.grad), ("b_dec", sae.b_dec.grad)):
        assert rel_l2(gt, ref.grads[pname]) < 1e-2, (pname, rel_l2(gt, ref.grads[pname]))
    # the dead rows carry the auxiliary term
    assert rel_l2(sae.W_dec.grad[dead.cuda()], ref.grads["W_dec"][dead]) < 1e-2


def test_auxk_sparse_update_matches_dense_path(cuda_lib):
    """With dead latents, the sparse fused update (extra dense rows inside
    sc_rows_adam) equals the dense-gradient path."""
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    from sparsify_b200.optim import FusedAdam
    N, D, M, k = 512, 256, 2048, 16
    g = torch.Generator().manual_seed(33)
    x = torch.randn(N, D, generator=g).cuda()
    dead = torch.zeros(M, dtype=torch.bool)
    dead[torch.randperm(M, generator=g)[:64]] = True
    dead = dead.cuda()
    results = []
    for sparse in (False, True):
        torch.manual_seed(0)
        sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=k), device="cuda", dtype=torch.float32)
        sae.precision = "mixed"
        opt = FusedAdam(sae.parameters(), lr=1e-3)
        sae.attach_optimizer(opt)
        if sparse:
            opt.enable_sparse_update(sae)
        for _ in range(2):
            sae.set_decoder_norm_to_unit_norm()
            out = sae(x, dead_mask=dead)
            assert float(out.auxk_loss) > 0
            (out.fvu + out.auxk_loss / 32).backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
        sae.set_decoder_norm_to_unit_norm()
        results.append({n: p.detach().clone() for n, p in sae.named_parameters()})
    for n in results[0]:
        assert rel_l2(results[1][n], results[0][n]) < 1e-5, n


def test_transcoder_skip_fused_vs_oracle(cuda_lib):
    """Transcoder (y != x, no b_dec subtraction) with a dense skip connection on
    the fused path, against the oracle on the same bf16-rounded operands."""
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    torch.manual_seed(0)
    N, D, M, k = 512, 256, 4096, 64
    cfg = SparseCoderConfig(num_latents=M, k=k, transcode=True, skip_connection=True)
    sae = SparseCoder(D, cfg, device="cuda", dtype=torch.float32)
    g = torch.Generator().manual_seed(41)
    x, y = torch.randn(N, D, generator=g), torch.randn(N, D, generator=g)
    with torch.no_grad():
        sae.W_dec.copy_(0.1 * torch.randn(M, D, generator=g))
        sae.W_skip.copy_(0.05 * torch.randn(D, D, generator=g))
        sae.encoder.bias.copy_(0.05 * torch.randn(M, generator=g))
    out = sae(x.cuda(), y.cuda())
    out.fvu.backward()
    rnd = lambda t: t.to(torch.bfloat16).to(torch.float32)
    params = dict(W_enc=sae.encoder.weight.detach().cpu(), b_enc=sae.encoder.bias.detach().cpu(),
                  W_dec=sae.W_dec.detach().cpu(), b_dec=sae.b_dec.detach().cpu(),
                  W_skip=rnd(sae.W_skip.detach().cpu()))
    ref = O.sae_forward_backward(params, rnd(x), y, cfg=O.OracleCfg(k=k, transcode=True, skip_connection=True),
                                 round_operands=rnd)
    assert abs(float(out.fvu) - float(ref.fvu)) < 1e-3 * float(ref.fvu)
    assert rel_l2(out.sae_out.detach(), ref.sae_out) < 1e-3
    for pname, gt in (("W_enc", sae.encoder.weight.grad), ("W_dec", sae.W_dec.grad), ("b_dec", sae.b_dec.grad),
                      ("W_skip", sae.W_skip.grad)):
        assert rel_l2(gt, ref.grads[pname]) < 1e-2, (pname, rel_l2(gt, ref.grads[pname]))


@pytest.mark.parametrize("precision,tol", [("fp32", 1e-4), ("bf16", 1e-2)])
def test_large_k_forward_backward(cuda_lib, precision, tol):
    """k far above the fused kernels' limit (the first steps of a k-decay schedule,
    trainer.py:176-177,229-235): entries are staged in several chunks by the
    gather kernels. k stays below the count of positive pre-activations so the
    selected set is unique."""
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    torch.manual_seed(0)
    N, D, M, k = 96, 256, 8192, 3000
    sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=k), device="cuda", dtype=torch.float32)
    sae.precision = precision
    x = torch.randn(N, D, generator=torch.Generator().manual_seed(4))
    out = sae(x.cuda())
    out.fvu.backward()
    rnd = (lambda t: t.to(torch.bfloat16).to(torch.float32)) if precision == "bf16" else None
    params = dict(W_enc=sae.encoder.weight.detach().cpu(), b_enc=sae.encoder.bias.detach().cpu(),
                  W_dec=sae.W_dec.detach().cpu(), b_dec=sae.b_dec.detach().cpu())
    ref = O.sae_forward_backward(params, x, cfg=O.OracleCfg(k=k), round_operands=rnd)
    assert float(ref.latent_acts.min()) > 0
    # as sets (neighbours in value order swap under a different summation order)
    got = torch.zeros(N, M, dtype=torch.bool).scatter_(1, out.latent_indices.cpu(), True)
    want = torch.zeros(N, M, dtype=torch.bool).scatter_(1, ref.latent_indices, True)
    assert int(got.sum()) == N * k  # no latent twice in a row
    assert (got & want).sum() / (N * k) > (0.999 if rnd else 0.99999)
    assert rel_l2(out.sae_out.detach(), ref.sae_out) < tol
    assert abs(float(out.fvu) - float(ref.fvu)) < tol * float(ref.fvu)
    for pname, gt in (("W_enc", sae.encoder.weight.grad), ("b_enc", sae.encoder.bias.grad),
                      ("W_dec", sae.W_dec.grad), ("b_dec", sae.b_dec.grad)):
        assert rel_l2(gt, ref.grads[pname]) < 10 * tol, (pname, rel_l2(gt, ref.grads[pname]))


def test_multi_topk_bf16_vs_oracle(cuda_lib):
    """Multi-TopK in the bf16 configuration: one tensor-core selection of the top 4k,
    whose leading k is the top-k (no dense pre-activations), against the oracle on
    the same bf16-rounded operands (sparse_coder.py:256-262)."""
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    torch.manual_seed(0)
    N, D, M, k = 384, 256, 4096, 16
    sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=k, multi_topk=True), device="cuda", dtype=torch.float32)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(N, D, generator=g)
    out = sae(x.cuda())
    (out.fvu + out.multi_topk_fvu / 8).backward()
    rnd = lambda t: t.to(torch.bfloat16).to(torch.float32)
    params = dict(W_enc=sae.encoder.weight.detach().cpu(), b_enc=sae.encoder.bias.detach().cpu(),
                  W_dec=sae.W_dec.detach().cpu(), b_dec=sae.b_dec.detach().cpu())
    ref = O.sae_forward_backward(params, x, cfg=O.OracleCfg(k=k, multi_topk=True), round_operands=rnd)
    assert out.latent_indices.shape == (N, 4 * k)  # the returned set is the wide one
    got = torch.zeros(N, M, dtype=torch.bool).scatter_(1, out.latent_indices.cpu(), True)
    want = torch.zeros(N, M, dtype=torch.bool).scatter_(1, ref.latent_indices, True)
    assert (got & want).sum() / (N * 4 * k) > 0.999
    assert rel_l2(out.sae_out.detach(), ref.sae_out) < 2e-3
    assert abs(float(out.fvu) - float(ref.fvu)) < 1e-3 * float(ref.fvu)
    assert abs(float(out.multi_topk_fvu) - float(ref.multi_topk_fvu)) < 1e-3 * float(ref.multi_topk_fvu)
    for pname, gt in (("W_enc", sae.encoder.weight.grad), ("b_enc", sae.encoder.bias.grad),
                      ("W_dec", sae.W_dec.grad), ("b_dec", sae.b_dec.grad)):
        assert rel_l2(gt, ref.grads[pname]) < 1e-2, (pname, rel_l2(gt, ref.grads[pname]))


@pytest.mark.parametrize("precision", ["mixed", "bf16"])
def test_multi_topk_sparse_update_matches_dense_path(cuda_lib, precision):
    """Multi-TopK in the fused step: its two losses' weight gradients handed to sc_rows_adam as one
    sparse problem (a virtual batch of 2N tokens) against the same step with dense gradients."""
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    from sparsify_b200.optim import FusedAdam
    N, D, M, k = 512, 256, 4096, 16
    g = torch.Generator().manual_seed(31)
    xs = [torch.randn(N, D, generator=g).cuda() for _ in range(3)]
    models = []
    for sparse in (False, True):
        torch.manual_seed(0)
        sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=k, multi_topk=True), device="cuda", dtype=torch.float32)
        sae.precision = precision
        opt = FusedAdam(sae.parameters(), lr=1e-3)
        sae.attach_optimizer(opt)
        if sparse:
            assert opt.enable_sparse_update(sae)
        for x in xs:
            sae.set_decoder_norm_to_unit_norm()
            out = sae(x)
            assert out.latent_indices.shape == (N, 4 * k) and float(out.multi_topk_fvu) > 0
            (out.fvu + out.multi_topk_fvu / 8).backward()
            if sparse:
                assert sae.W_dec.grad is None and sae._pending is not None
            opt.step()
            opt.zero_grad(set_to_none=True)
        sae.set_decoder_norm_to_unit_norm()
        models.append(sae)
    a, b = models
    tol = 1e-5 if precision == "mixed" else 2e-4
    for (n1, p1), (_, p2) in zip(a.named_parameters(), b.named_parameters()):
        assert rel_l2(p2.detach(), p1.detach()) < tol, (n1, rel_l2(p2.detach(), p1.detach()))


def test_training_steps_are_reproducible_bit_for_bit(cuda_lib):
    """Three fused training steps run twice from the same state give identical bits: the
    reference's scatter (atomics, xformers.py:132-136, fused_encoder.py:77-82) does not,
    this path sums every latent's contributions in ascending token order."""
    from sparsify_b200 import SparseCoder, SparseCoderConfig
    from sparsify_b200.optim import FusedAdam

    def run():
        torch.manual_seed(3)
        sae = SparseCoder(256, SparseCoderConfig(num_latents=4096, k=16), device="cuda", dtype=torch.float32)
        opt = FusedAdam(sae.parameters(), lr=1e-3)
        sae.attach_optimizer(opt)
        opt.enable_sparse_update(sae)
        g = torch.Generator().manual_seed(5)
        fvus = []
        for _ in range(3):
            x = torch.randn(1024, 256, generator=g).cuda().bfloat16()
            sae.set_decoder_norm_to_unit_norm()
            out = sae(x)
            out.fvu.backward()
            opt.step(); opt.zero_grad(set_to_none=True)
            fvus.append(out.fvu.detach().clone())
        return torch.stack(fvus), {n: p.detach().clone() for n, p in sae.named_parameters()}, out.latent_indices.clone()

    f1, p1, i1 = run()
    f2, p2, i2 = run()
    assert torch.equal(f1, f2) and torch.equal(i1, i2)
    for n in p1:
        assert torch.equal(p1[n], p2[n]), n
