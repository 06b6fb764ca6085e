"""Pins the CPU oracle against fixtures produced by the reference itself
(tests/golden/make_golden.py). fp32, tiny shapes, runs without a GPU."""

import torch

from oracle import sae_oracle as O
from tests.conftest import load_golden, rel_l2, sort_topk

TOL = 2e-5  # fp32 with a different (but fixed) summation order


def test_encoder_topk_forward_backward():
    t, meta = load_golden("encoder_topk")
    vals, idx, pre = O.encoder_forward(t["x"], t["W"], t["b"], meta["k"], "topk")
    vals, idx = sort_topk(vals, idx)
    assert torch.equal(idx, t["idx"])
    assert rel_l2(vals, t["vals"]) < TOL
    assert rel_l2(pre, t["pre"]) < TOL
    gx, gW, gb = O.encoder_backward(t["x"], t["W"], idx, t["coef"])
    assert rel_l2(gx, t["gx"]) < TOL
    assert rel_l2(gW, t["gW"]) < TOL
    assert rel_l2(gb, t["gb"]) < TOL


def test_encoder_groupmax():
    t, meta = load_golden("encoder_groupmax")
    vals, idx, _ = O.encoder_forward(t["x"], t["W"], t["b"], meta["k"], "groupmax")
    vals, idx = sort_topk(vals, idx)
    assert torch.equal(idx, t["idx"])
    assert rel_l2(vals, t["vals"]) < TOL
    gx, gW, gb = O.encoder_backward(t["x"], t["W"], idx, t["coef"])
    assert rel_l2(gx, t["gx"]) < TOL and rel_l2(gW, t["gW"]) < TOL and rel_l2(gb, t["gb"]) < TOL


def test_decoder_forward_backward():
    for d_in in (48, 64):
        t, _ = load_golden(f"decoder_d{d_in}")
        out = O.decode(t["idx"], t["acts"], t["W_dec"])
        assert rel_l2(out, t["out"]) < TOL
        gW, gacts = O.decode_backward(t["idx"], t["acts"], t["W_dec"], t["gout"])
        assert rel_l2(gW, t["gW"]) < TOL
        assert rel_l2(gacts, t["gacts"]) < TOL


def _params(t, prefix="param."):
    return {k[len(prefix):]: v.clone() for k, v in t.items() if k.startswith(prefix)}


def test_forward_and_gradients():
    for name in ("sae_plain", "sae_auxk", "sae_multitopk", "transcoder_skip"):
        t, meta = load_golden(f"forward_{name}")
        c = meta["cfg"]
        cfg = O.OracleCfg(k=c["k"], activation=c["activation"], normalize_decoder=c["normalize_decoder"],
                          multi_topk=c["multi_topk"], skip_connection=c["skip_connection"],
                          transcode=c["transcode"])
        res = O.sae_forward_backward(_params(t), t["x"], t.get("y"), t.get("dead_mask"), cfg,
                                     auxk_alpha=meta["auxk_alpha"])
        acts, idx = sort_topk(res.latent_acts, res.latent_indices)
        assert torch.equal(idx, t["latent_indices"]), name
        assert rel_l2(acts, t["latent_acts"]) < TOL, name
        assert rel_l2(res.sae_out, t["sae_out"]) < TOL, name
        for key in ("fvu", "auxk_loss", "multi_topk_fvu"):
            ref = t[key]
            got = getattr(res, key)
            assert abs(float(got) - float(ref)) <= 1e-5 * max(1.0, abs(float(ref))), (name, key)
        for pname, g in res.grads.items():
            ref = t[f"grad.{pname}"]
            if float(ref.norm()) == 0.0:
                assert float(g.norm()) < 1e-7, (name, pname)
            else:
                assert rel_l2(g, ref) < 5e-5, (name, pname, rel_l2(g, ref))


def test_trainer_trajectory():
    t, meta = load_golden("trainer_adam")
    params = _params(t, "init.")
    cfg = O.OracleCfg(k=meta["k"])
    tr = O.OracleTrainer(params, cfg, lr=meta["lr"], warmup=meta["warmup"], total_steps=meta["steps"],
                         auxk_alpha=meta["auxk_alpha"], dead_threshold=meta["dead_feature_threshold"])
    acts = t["acts"]
    fvus = []
    for s in range(meta["steps"]):
        x = acts[s].reshape(-1, meta["D"])
        fvus.append(float(tr.step(x).fvu))
    ref = t["fvu"].tolist()
    for a, b in zip(fvus, ref):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (fvus, ref)
    for pname in ("W_enc", "b_enc", "W_dec", "b_dec"):
        assert rel_l2(params[pname], t[f"final.{pname}"]) < 2e-3, pname
    assert torch.equal(tr.num_tokens_since_fired, t["num_tokens_since_fired"])


def test_trainer_signum_trajectory():
    """optimizer="signum": the reference Trainer's own SignSGD, learning-rate rule and
    step order around the schedule-free wrapper (whose restatement both sides share)."""
    t, meta = load_golden("trainer_signum")
    params = _params(t, "init.")
    tr = O.OracleTrainer(params, O.OracleCfg(k=meta["k"]), lr=meta["lr"], optimizer="signum")
    fvus = [float(tr.step(t["acts"][s].reshape(-1, meta["D"])).fvu) for s in range(meta["steps"])]
    for a, b in zip(fvus, t["fvu"].tolist()):
        assert abs(a - b) < 5e-4 * max(1.0, abs(b)), (fvus, t["fvu"].tolist())
    for pname in ("W_enc", "b_enc", "W_dec", "b_dec"):
        assert rel_l2(params[pname], t[f"final.{pname}"]) < 5e-3, pname
        x = torch.lerp(params[pname], tr.z[pname], 1 - 1 / 0.95)  # what eval() stores in the checkpoint
        assert rel_l2(x, t[f"saved.{pname}"]) < 5e-3, pname


def test_newtonschulz():
    for name in ("wide", "tall"):
        t, _ = load_golden(f"newtonschulz_{name}")
        X = O.quintic_newtonschulz(t["G"], 5).float()
        assert rel_l2(X, t["X"]) < 1e-2  # bf16 arithmetic
