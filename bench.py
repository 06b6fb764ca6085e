"""Benchmark of the TopK sparse-coder training step (SAE train tokens/s).

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # the reference's own CPU path on the host cores

Workload (default): d_in=4096, 131072 latents, k=32, 16384 tokens per rank per
step, bf16 operands with fp32 accumulation, forward + backward + Adam with the
AuxK branch enabled (inert while no latent is dead), synthetic activations.
One JSON line is printed by rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "sae_train_tokens_per_s"
UNIT = "tokens/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"],
                    help="ours: this library; reference: the reference's own CPU path on the host cores; "
                         "reference-gpu: the reference's own CUDA path (bf16 autocast, its Triton decoder) on one "
                         "GPU of this box, printed as context next to this library's figure")
    ap.add_argument("--tokens", type=int, default=16384, help="tokens per rank per step")
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--latents", type=int, default=131072)
    ap.add_argument("--k", type=int, default=32)
    ap.add_argument("--atoms", type=int, default=262144)
    ap.add_argument("--active", type=int, default=64)
    ap.add_argument("--cpu-tokens", type=int, default=1024,
                    help="tokens per step of the bounded CPU sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--config0-steps", type=int, default=10,
                    help="timed steps of the CPU arm's second figure, the reference's CPU-sized configuration "
                         "(d_in=768, 24576 latents, k=32, 4096 tokens per step); 0 skips it")
    ap.add_argument("--no-gpu-reference", action="store_true",
                    help="skip the same-box figure of the reference's own CUDA path (a child process, N=1 only)")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the secondary workloads (AuxK active, transcoder k=64 with skip, and on several "
                         "ranks the hookpoint-sharded Muon workload) that follow the headline measurement")
    ap.add_argument("--no-parity", action="store_true",
                    help="skip the multi-rank parity check that precedes the timed region on several ranks")
    ap.add_argument("--transcode", action="store_true",
                    help="transcoder workload: target y = W2 gelu(W1 layernorm(x)) with seeded W1 [3.5d, d], "
                         "W2 [d, 3.5d], a learned dense skip connection, decoder initialised at zero")
    ap.add_argument("--overlap", type=int, default=0,
                    help="1: run the step on a high-priority stream and the decoder half of the weight "
                         "update on a normal-priority side stream under the next encoder GEMM "
                         "(measured slower on B200: 25.7 vs 23.0 ms/step; off by default)")
    ap.add_argument("--multi-topk", action="store_true",
                    help="secondary workload: Multi-TopK loss (top 4k selected in the encoder kernel)")
    ap.add_argument("--dead-frac", type=float, default=0.0,
                    help="mark this fraction of the latents dead (fixed seed) so that the AuxK branch is "
                         "active in every step; 0 = the natural state (no latent dead yet)")
    ap.add_argument("--reserve-sms", type=int, default=4,
                    help="SMs the persistent kernels leave free for NCCL's kernels when several ranks run "
                         "(measured at 8 GPUs: 23.6 ms per step with 4, 24.0 ms with 0); ignored on one GPU")
    ap.add_argument("--cta-pairs", type=int, default=-1,
                    help="1: the tensor-core encoder runs as CTA pairs (tcgen05 cta_group::2); 0: one CTA per work "
                         "unit; -1 (default): the library chooses per shape (one CTA at k=32, where it measured "
                         "14.2 against 15.5 ms per launch; pairs for wide top-k lists)")
    ap.add_argument("--modules", type=int, default=0,
                    help="secondary workload: this many hookpoints per rank, each with its own sparse coder "
                         "trained by Muon on activations gathered from every rank (distribute_modules); "
                         "--tokens is then the tokens per hookpoint per step over all ranks")
    ap.add_argument("--kernel", default=None,
                    help="time one kernel alone on random inputs of the given sizes instead of the step: "
                         "encode | decode | bwd_acts | csr | rows | topk_mask | rows_adam | adam | normalize | all | ns | gemm")
    return ap.parse_args()


def workload_name(a) -> str:
    aux = f"AuxK active on {a.dead_frac:.0%} dead latents" if a.dead_frac > 0 else "AuxK enabled"
    if getattr(a, "multi_topk", False):
        aux += ", Multi-TopK loss"
    if a.transcode:
        return (f"transcoder train step d_in={a.d} latents={a.latents} k={a.k} tokens/rank/step={a.tokens} "
                f"dense skip connection, bf16 operands fp32 accumulate, fwd+bwd+Adam, {aux}")
    return (f"SAE train step d_in={a.d} latents={a.latents} k={a.k} tokens/rank/step={a.tokens} "
            f"bf16 operands fp32 accumulate, fwd+bwd+Adam, {aux}")


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        burst = d.get("bf16_tflops")
        return {"tflops_sustained": d.get("bf16_tflops_sustained", burst), "tflops_burst": burst,
                "hbm": d.get("hbm_gbs"), "source": "measured"}
    return {"tflops_sustained": 1400.0, "tflops_burst": 1590.0, "hbm": 6650.0, "source": "fallback"}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and clock-event reasons while the timed region runs: NVML
    queries (read-only) from a thread every 20 ms; `nvidia-smi -lms` as the fallback when
    the NVML binding is missing. Only samples taken after mark() are reported."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.thread = None
        self.stop_flag = threading.Event()
        self.samples: list[tuple[float, float, float, tuple[str, ...]]] = []  # (t, sm, max, reasons)
        self.t_mark = 0.0
        self.error: str | None = None

    def mark(self):
        """Start of the timed region: samples that arrived earlier (warm-up) are dropped."""
        self.t_mark = time.monotonic()

    def physical_index(self) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            try:
                return int(vis.split(",")[self.index])
            except (ValueError, IndexError):
                pass
        return self.index

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.physical_index())
            bits = [(pynvml.nvmlClocksEventReasonHwSlowdown, "hw_slowdown"),
                    (pynvml.nvmlClocksEventReasonHwThermalSlowdown, "hw_thermal_slowdown"),
                    (pynvml.nvmlClocksEventReasonSwThermalSlowdown, "sw_thermal_slowdown"),
                    (pynvml.nvmlClocksEventReasonSwPowerCap, "sw_power_cap")]
            mx = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))

            def poll():
                while not self.stop_flag.is_set():
                    try:
                        sm = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                        mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                        self.samples.append((time.monotonic(), sm, mx, tuple(n for b, n in bits if mask & b)))
                    except pynvml.NVMLError as exc:
                        self.error = str(exc)
                        return
                    self.stop_flag.wait(0.02)

            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            return
        except Exception as exc:  # no NVML binding or no permission: fall back to nvidia-smi
            self.error = f"nvml: {exc}"
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.physical_index()}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm, mx = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            reasons = tuple(n for n, v in zip(self.NAMES, parts[2:6]) if v.lower().startswith("active"))
            self.samples.append((time.monotonic(), sm, mx, reasons))

    def stop(self) -> dict:
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=2)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread is None and self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source: " + str(self.error)]}
        used = [smp for smp in self.samples if smp[0] >= self.t_mark]
        sm = [smp[1] for smp in used]
        reasons = sorted({r for smp in used for r in smp[3]})
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": used[-1][2] if used else None, "reasons": reasons, "samples": len(sm)}


# --------------------------------------------------------------------------- CPU arm
def host_threads() -> int:
    """Uses every core this process may run on. A launcher's OMP_NUM_THREADS=1
    (torch.distributed.run exports it) would otherwise leave the CPU arm on one thread."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def _stored_batches(D: int, atoms: int, active: int, tokens: int, steps: int) -> torch.Tensor:
    """[steps, 1, tokens, D] fp32 synthetic activations on the host."""
    from sparsify_b200.synthetic import SyntheticActivations, batch_seed
    gen = SyntheticActivations(D, min(atoms, 65536), active, device="cpu")
    return torch.stack([gen.batch(tokens, batch_seed(t)).reshape(1, tokens, D) for t in range(steps)])


def reference_sample(D: int, M: int, k: int, tokens: int, atoms: int, active: int, steps: int, warmup: int) -> dict:
    """Times the reference's own code on the host: `sparsify.Trainer.fit()` of the vendored,
    unmodified package (oracle/_ref) - its hook, SparseCoder.forward (eager embedding_bag
    path), backward, decoder normalisation and projection, torch.optim.Adam, schedule and
    dead-latent bookkeeping - in fp32 on every host thread, `tokens` tokens per step."""
    import contextlib

    from oracle import ref_loader
    cores = host_threads()
    acts = _stored_batches(D, atoms, active, tokens, warmup + steps)
    with contextlib.redirect_stdout(sys.stderr):  # the reference prints progress; stdout carries the JSON line
        res = ref_loader.time_reference_trainer(acts, num_latents=M, k=k, warmup_steps=warmup, threads=cores)
    sec = statistics.median(res["seconds"])
    return {"value": tokens / sec, "unit": UNIT, "cores": cores, "kind": "reference",
            "sample": f"sparsify {res['version']} Trainer.fit() on the host, {tokens} tokens/step at d_in={D}, "
                      f"latents={M}, k={k}, fp32, {len(res['seconds'])} timed steps after {warmup} "
                      f"(median {sec:.3f} s/step)",
            "ms_per_step": sec * 1e3, "steps": len(res["seconds"])}


def port_sample(D: int, M: int, k: int, tokens: int, atoms: int, active: int, steps: int, warmup: int) -> dict:
    """Fallback when the vendored reference is absent: the oracle's restatement of the same
    step (CPU, fp32, all host threads)."""
    from oracle import sae_oracle as O
    from sparsify_b200.synthetic import SyntheticActivations

    cores = host_threads()
    g = torch.Generator().manual_seed(0)
    bound = 1.0 / D ** 0.5
    W_enc = (torch.rand(M, D, generator=g) * 2 - 1) * bound
    params = dict(W_enc=W_enc, b_enc=torch.zeros(M), W_dec=W_enc.clone(), b_dec=torch.zeros(D))
    O.normalize_decoder_(params["W_dec"])
    gen = SyntheticActivations(D, min(atoms, 65536), active, device="cpu")
    tr = O.OracleTrainer(params, O.OracleCfg(k=k), warmup=1000, total_steps=10**6, auxk_alpha=1 / 32)
    times = []
    for s in range(warmup + steps):
        x = gen.batch(tokens, seed=s)
        t0 = time.perf_counter()
        tr.step(x)
        if s >= warmup:
            times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return {"value": tokens / sec, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"oracle restatement of the reference step (the vendored reference is absent), {tokens} "
                      f"tokens/step at d_in={D}, latents={M}, k={k}, fp32, {steps} timed steps "
                      f"(median {sec:.3f} s/step)",
            "ms_per_step": sec * 1e3, "steps": steps}


def cpu_arm(a, steps: int, warmup: int, config0_steps: int) -> dict:
    """The CPU figures of a run: the workload's own width with a bounded number of tokens per
    step (the figure comparable with the GPU arm), and the reference's CPU-sized configuration
    (d_in=768, 24576 latents, k=32, 4096 tokens per step) in full."""
    from oracle import ref_loader
    sample = reference_sample if ref_loader.find_reference() is not None else port_sample
    base = sample(a.d, a.latents, a.k, a.cpu_tokens, a.atoms, a.active, steps, warmup)
    if config0_steps > 0:
        c0 = sample(768, 24576, 32, 4096, 65536, 32, config0_steps, 3)
        base["config0"] = {"value": c0["value"], "unit": UNIT, "ms_per_step": c0["ms_per_step"],
                           "kind": c0["kind"], "sample": c0["sample"]}
    return base


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # every step costs seconds on the host (Adam alone walks 1.07e9 parameters): the timed steps are capped
    steps, warmup = max(1, min(a.steps, 10)), max(1, min(a.warmup, 3))
    base = cpu_arm(a, steps, warmup, config0_steps=a.config0_steps)
    keys = ("value", "unit", "cores", "kind", "sample", "config0")
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": a.gpus,
        "steps": base["steps"], "warmup": warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(a),
                   "note": f"the reference's own CPU path on {base['cores']} host threads; each step is a bounded "
                           f"sample of {a.cpu_tokens} tokens of the workload"},
        "cpu_baseline": {k: base[k] for k in keys if k in base},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_reference_gpu(a):
    """The reference's own GPU path on cuda:0 of this box: sparsify's Trainer.fit() with its
    bf16 autocast forward, dense pre-activations + torch.topk, its Triton embedding-bag
    decoder and torch.optim.Adam, on the workload's full shape. Context for the headline,
    not a contract arm; runs in a process of its own (see gpu_reference_sample)."""
    import contextlib

    from oracle import ref_loader
    from sparsify_b200.synthetic import SyntheticActivations, batch_seed
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    steps, warmup = max(1, min(a.steps, 10)), max(1, min(a.warmup, 3))
    gen = SyntheticActivations(a.d, min(a.atoms, 65536), a.active, device=dev)
    acts = torch.stack([gen.batch(a.tokens, batch_seed(t), torch.bfloat16).reshape(1, a.tokens, a.d)
                        for t in range(warmup + steps)])
    del gen
    torch.cuda.empty_cache()
    with contextlib.redirect_stdout(sys.stderr):
        res = ref_loader.time_reference_trainer(acts, num_latents=a.latents, k=a.k, warmup_steps=warmup, triton=True)
    sec = statistics.median(res["seconds"])
    import sparsify.utils as ref_utils
    print(json.dumps({"impl": "reference-gpu", "metric": METRIC, "value": a.tokens / sec, "unit": UNIT, "n_gpus": 1,
                      "steps": len(res["seconds"]), "warmup": warmup, "ms_per_step": sec * 1e3,
                      "decoder": ref_utils.decoder_impl.__name__,
                      "peak_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
                      "sample": f"sparsify {res['version']} Trainer.fit() on one B200: fp32 parameters, bf16 autocast "
                                f"forward, {ref_utils.decoder_impl.__name__}, torch.optim.Adam; {a.tokens} tokens/step at "
                                f"d_in={a.d}, latents={a.latents}, k={a.k}; median of {len(res['seconds'])} steps after "
                                f"{warmup}, wall clock between device synchronisations"}), flush=True)


def gpu_reference_sample(a) -> dict:
    """Runs `bench.py --impl reference-gpu` as a child process (its own CUDA context and memory;
    a failure of the reference's GPU code cannot take the benchmark down) and returns its
    line, or {"unavailable": reason}."""
    from oracle import ref_loader
    if ref_loader.find_reference() is None:
        return {"unavailable": "the vendored reference (oracle/_ref) is not present"}
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference-gpu", "--steps", "5", "--warmup", "3",
           "--tokens", str(a.tokens), "--d", str(a.d), "--latents", str(a.latents), "--k", str(a.k),
           "--atoms", str(a.atoms), "--active", str(a.active)]
    env = {k_: v for k_, v in os.environ.items() if k_ not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "OMP_NUM_THREADS")}
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=420, cwd=ROOT, env=env)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference's GPU path did not finish within 420 s"}
    lines = [l for l in out.stdout.strip().splitlines() if l.startswith("{")]
    if out.returncode != 0 or not lines:
        tail = (out.stderr.strip().splitlines() or ["no output"])[-1]
        return {"unavailable": f"the reference's GPU path failed here (exit {out.returncode}): {tail[:300]}"}
    d = json.loads(lines[-1])
    return {k_: d[k_] for k_ in ("value", "unit", "ms_per_step", "steps", "decoder", "peak_memory_gb", "sample")}


# --------------------------------------------------------------------------- GPU arm
LAUNCHES_PER_CALL = {  # kernels each C-ABI entry point enqueues
    "sc_encode_topk": 3, "sc_csr_build": 6, "sc_total_variance": 4, "sc_sq_err": 2, "sc_weighted_colsum": 2,
    "sc_decode_residual": 2, "sc_muon_momentum": 2,
}


class LaunchCounter:
    """Counts kernel launches of libsparsecoder by wrapping the ABI call helper."""

    def __init__(self):
        from sparsify_b200 import _lib, ops
        self.n = 0
        self._lib, self._ops = _lib, ops
        self._orig = _lib.call

        def counted(name, *args):
            self.n += LAUNCHES_PER_CALL.get(name, 1)
            return self._orig(name, *args)

        _lib.call = counted
        ops.call = counted

    def close(self):
        self._lib.call = self._orig
        self._ops.call = self._orig


class StepWorkload:
    """One sparse coder, its optimiser, and a pool of device- and host-resident batches: the
    training step the benchmark times (forward, backward, exchange, Adam, dead-latent
    bookkeeping), as the Trainer runs it."""

    def __init__(self, a, gen, dev, rank: int, world: int):
        import torch.distributed as dist

        from sparsify_b200 import SparseCoder, SparseCoderConfig
        from sparsify_b200.optim import FusedAdam
        from sparsify_b200.synthetic import batch_seed

        self.a, self.dev, self.rank, self.world, self.dist = a, dev, rank, world, dist
        N, D, M, k = a.tokens, a.d, a.latents, a.k
        torch.manual_seed(0)  # identical replicas on every rank (sparsify/trainer.py:80-87)
        cfg = SparseCoderConfig(num_latents=M, k=k, transcode=a.transcode, skip_connection=a.transcode,
                                multi_topk=a.multi_topk)
        self.sae = sae = SparseCoder(D, cfg, device=dev, dtype=torch.float32)
        self.opt = opt = FusedAdam(sae.parameters(), lr=2e-4 / (M / 2 ** 14) ** 0.5)
        sae.attach_optimizer(opt)
        # gradients go to the optimiser in sparse form; with several ranks the factors are
        # exchanged and each rank updates its slice of the latents
        self.overlap = bool(a.overlap) and world == 1
        opt.enable_sparse_update(sae, overlap_decoder=self.overlap)
        self.alpha = 1 / 32
        self.since_fired = torch.zeros(M, dtype=torch.long, device=dev)
        self.dead_threshold = 10_000_000
        self.tokens_seen = 0
        self.pool = [gen.batch(N, batch_seed(t, rank, world), torch.bfloat16) for t in range(4)]
        self.targets = None
        if a.transcode:
            # the module being transcoded: a seeded MLP applied to the layer-normed input
            gw = torch.Generator(device=dev).manual_seed(2001)
            H = int(3.5 * D)
            W1 = (torch.randn(H, D, device=dev, generator=gw) / D ** 0.5).bfloat16()
            W2 = (torch.randn(D, H, device=dev, generator=gw) / H ** 0.5).bfloat16()
            ln = torch.nn.functional.layer_norm
            self.targets = [(torch.nn.functional.gelu(ln(b.float(), (D,)).bfloat16() @ W1.T) @ W2.T).bfloat16()
                            for b in self.pool]
            del W1, W2
            torch.cuda.empty_cache()
        self.host_pool = [b.cpu().pin_memory() for b in self.pool]
        with torch.no_grad():
            mean = (self.targets[0] if a.transcode else self.pool[0]).float().mean(0)
            if world > 1:
                dist.all_reduce(mean)
                mean /= world
            sae.b_dec.copy_(mean)
            if a.transcode:  # centre the pre-activations (sparsify/trainer.py:398-401)
                sae.encoder.bias.copy_(-self.pool[0].float().mean(0) @ sae.encoder.weight.T)
        self.params = list(sae.parameters())
        self.fixed_dead = None
        if a.dead_frac > 0:
            gd = torch.Generator(device="cpu").manual_seed(7)
            dead = torch.zeros(M, dtype=torch.bool)
            dead[torch.randperm(M, generator=gd)[: int(a.dead_frac * M)]] = True
            self.fixed_dead = sae.prepare_dead_mask(dead.to(dev))  # read back once, as the Trainer does per step

    def target(self, t):
        return self.targets[t % len(self.targets)] if self.targets is not None else None

    def step(self, x, y=None):
        a, sae, dist, world = self.a, self.sae, self.dist, self.world
        N, M = a.tokens, a.latents
        if not a.transcode:
            sae.set_decoder_norm_to_unit_norm()
        # as the Trainer does: the dead mask is only built once a counter can have passed the threshold
        dead = self.since_fired > self.dead_threshold if self.tokens_seen > self.dead_threshold else None
        if self.fixed_dead is not None:
            dead = self.fixed_dead
        self.tokens_seen += N
        out = sae(x, y, dead_mask=dead)
        loss = out.fvu + self.alpha * out.auxk_loss
        if a.multi_topk:
            loss = loss + out.multi_topk_fvu / 8  # sparsify/trainer.py:444-447
        loss.backward()
        if world > 1:
            for p in self.params:
                if p.grad is not None:  # biases; the matrices travel as sparse factors
                    dist.all_reduce(p.grad)
                    p.grad /= world
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        with torch.no_grad():
            fired = torch.zeros(M, dtype=torch.bool, device=self.dev)
            fired.index_fill_(0, out.latent_indices.flatten(), True)  # (indexed assignment would block the host)
            if world > 1:
                f8 = fired.to(torch.uint8)
                dist.all_reduce(f8, op=dist.ReduceOp.MAX)
                fired = f8.bool()
            self.since_fired.add_(N)
            self.since_fired[fired] = 0
        return out.fvu.detach()

    def sync(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()


def _mean_ms(pairs):
    return statistics.mean(s.elapsed_time(e) for s, e in pairs) if pairs else None


def time_workload(wl: StepWorkload, steps: int, warmup: int, sampler: ClockSampler | None, with_e2e: bool) -> dict:
    """Device-timed steps on resident batches, then (with_e2e) the same steps fed from pinned
    host memory with the loss read back, both as max over ranks."""
    from sparsify_b200 import ops
    dev, dist, world = wl.dev, wl.dist, wl.world
    for t in range(max(warmup, 3)):
        wl.step(wl.pool[t % len(wl.pool)], wl.target(t))
    wl.sync()

    counter = LaunchCounter()
    ops.timers = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wl.sync()
    if sampler is not None:
        sampler.mark()
    e0.record()
    for t in range(steps):
        wl.step(wl.pool[t % len(wl.pool)], wl.target(t))
    e1.record()
    wl.sync()
    clocks = sampler.stop() if sampler is not None else None
    ops.check_status(dev)  # a bounded wait that gave up would have produced garbage: fail loudly
    res = {"ms": e0.elapsed_time(e1) / steps, "clocks": clocks, "launches": counter.n}
    timers, ops.timers = ops.timers, None
    counter.close()
    res["enc_ms"] = _mean_ms(timers.get("encode_topk", []))
    upd = timers.get("rows_adam", [])
    # the optimiser kernel runs as two launches per step (one per matrix): sum them per step
    res["upd_ms"] = sum(s_.elapsed_time(e_) for s_, e_ in upd) / steps if upd else None
    res["spans"] = {name: sum(s_.elapsed_time(e_) for s_, e_ in pairs) / steps
                    for name, pairs in timers.items() if name.startswith("x_")}

    if with_e2e:
        # ---- end to end: pinned host input -> device, step, loss back to host ----
        # Every step's input crosses PCIe inside the timed region. The copy of step t+1 is
        # issued on a copy stream while step t computes (two device buffers), as an input
        # pipeline would do; the loss of every step is read back to the host.
        bufs = [torch.empty_like(wl.pool[0]) for _ in range(2)]
        copy_stream = torch.cuda.Stream(device=dev)
        ready = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]
        main = torch.cuda.current_stream(dev)

        def fetch(t):
            b = t % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[b])  # the step that last read this buffer is done
                bufs[b].copy_(wl.host_pool[t % len(wl.host_pool)], non_blocking=True)
                ready[b].record(copy_stream)

        wl.sync()
        for b in range(2):
            consumed[b].record(main)
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # The loss of every step is copied to pinned host memory and read by the host one step
        # later (while the next step is already queued), as a training loop logs it.
        loss_host = [torch.empty((), dtype=torch.float32).pin_memory() for _ in range(2)]
        loss_ready = [torch.cuda.Event() for _ in range(2)]
        losses = []
        f0.record()
        fetch(0)
        for t in range(steps):
            if t + 1 < steps:
                fetch(t + 1)
            main.wait_event(ready[t % 2])
            fvu = wl.step(bufs[t % 2], wl.target(t))
            consumed[t % 2].record(main)
            loss_host[t % 2].copy_(fvu, non_blocking=True)
            loss_ready[t % 2].record(main)
            if t > 0:
                loss_ready[(t - 1) % 2].synchronize()
                losses.append(float(loss_host[(t - 1) % 2]))
        loss_ready[(steps - 1) % 2].synchronize()
        losses.append(float(loss_host[(steps - 1) % 2]))
        f1.record()
        wl.sync()
        assert len(losses) == steps and all(v == v for v in losses), "a step's loss did not reach the host"
        ops.check_status(dev)
        res["ms_e2e"] = f0.elapsed_time(f1) / steps
        res["last_fvu"] = losses[-1]
    if world > 1:
        for key in ("ms", "ms_e2e"):
            if key in res:
                t_ = torch.tensor([res[key]], device=dev)
                dist.all_reduce(t_, op=dist.ReduceOp.MAX)
                res[key] = float(t_)
    return res


def step_roofline(a, peaks: dict, ms: float) -> dict:
    """BASELINE.json's step roofline: the slower of the encoder's FLOPs at the tensor peak and
    the gather / scatter bytes at the HBM peak - against both measured tensor peaks."""
    N, D, M, k = a.tokens, a.d, a.latents, a.k
    flops = 2.0 * N * D * M
    gathers = 2 if a.transcode else 3  # decode, grad-acts (+ grad-x: a transcoder's input needs no gradient)
    gs_bytes = gathers * (N * k * D * 2 + N * D * 4) + N * k * 24 + 2 * M * D * 4 + 2 * N * D * 4
    t_hbm = gs_bytes / (peaks["hbm"] * 1e9) * 1e3
    out = {"def": "max(encoder FLOPs / tensor peak, gather+scatter bytes / HBM peak); sustained = cuBLAS bf16 "
                  "back to back for seconds under the power cap, burst = best of ten",
           "peak_source": peaks["source"]}
    for kind in ("sustained", "burst"):
        t = max(flops / (peaks[f"tflops_{kind}"] * 1e12) * 1e3, t_hbm)
        out[f"ms_{kind}"] = t
        out[f"frac_{kind}"] = t / ms
    out["ms"], out["frac"] = out["ms_sustained"], out["frac_sustained"]
    return out


def dp_parity(dev, rank: int, world: int) -> dict:
    """Correctness of the multi-rank path, checked inside the run that is timed: a small coder
    takes three optimiser steps through the sharded sparse update (exchange of the gradient
    factors, every rank updating its slice of the latents, all-gather of the bf16 copies), once
    plain and once with dead latents (AuxK active), and is compared on every rank with the
    same steps computed locally from all ranks' seeded batches with the per-rank losses
    averaged - what DistributedDataParallel's gradient mean gives the reference
    (sparsify/trainer.py:457-468). Also checks that all replicas are bit-identical."""
    import torch.distributed as dist

    from sparsify_b200 import SparseCoder, SparseCoderConfig
    from sparsify_b200.optim import FusedAdam
    from sparsify_b200.synthetic import SyntheticActivations

    N, D, M, k, steps = 2048, 256, 4096, 16, 3
    gen = SyntheticActivations(D, 4096, 16, seed=77, device=dev)

    def build():
        torch.manual_seed(0)
        sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=k), device=dev, dtype=torch.float32)
        opt = FusedAdam(sae.parameters(), lr=1e-3)
        sae.attach_optimizer(opt)
        return sae, opt

    worst, equal = 0.0, True
    for case in ("plain", "dead_mask"):
        dead = None
        if case == "dead_mask":
            g = torch.Generator().manual_seed(5)
            dead = torch.zeros(M, dtype=torch.bool)
            dead[torch.randperm(M, generator=g)[:192]] = True
            dead = dead.to(dev)
        data = lambda r, s: gen.batch(N, seed=1000 + 10 * s + r)
        sae, opt = build()
        assert opt.enable_sparse_update(sae) and sae._shard == (rank, world)
        for s in range(steps):
            sae.set_decoder_norm_to_unit_norm()
            out = sae(data(rank, s), dead_mask=dead)
            (out.fvu + out.auxk_loss / 32).backward()
            for p in sae.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad)
                    p.grad /= world
            opt.step()
            opt.zero_grad(set_to_none=True)
        opt.sync_masters()
        ref, ropt = build()  # single-process form: dense gradients, no exchange
        for s in range(steps):
            ref.set_decoder_norm_to_unit_norm()
            outs = [ref(data(r, s), dead_mask=dead) for r in range(world)]
            (sum(o.fvu + o.auxk_loss / 32 for o in outs) / world).backward()
            ropt.step()
            ropt.zero_grad(set_to_none=True)
        ref.set_decoder_norm_to_unit_norm()
        for (name, p), (_, q) in zip(sae.named_parameters(), ref.named_parameters()):
            rel = float((p.detach().double() - q.detach().double()).norm() / q.detach().double().norm())
            worst = max(worst, rel)
            # bit pattern of the replica: identical on every rank?
            digest = p.detach().contiguous().view(torch.int32).to(torch.int64).sum().reshape(1)
            all_d = [torch.empty_like(digest) for _ in range(world)]
            dist.all_gather(all_d, digest)
            equal = equal and all(int(d_) == int(all_d[0]) for d_ in all_d)
        for name in ("encoder.weight", "W_dec"):
            digest = sae.shadow(name).view(torch.int16).to(torch.int64).sum().reshape(1)
            all_d = [torch.empty_like(digest) for _ in range(world)]
            dist.all_gather(all_d, digest)
            equal = equal and all(int(d_) == int(all_d[0]) for d_ in all_d)
    flag = torch.tensor([worst], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return {"max_rel_l2": float(flag), "replicas_equal": bool(equal), "tolerance": 2e-3,
            "case": f"{N} tokens/rank x d_in={D} x {M} latents, k={k}, {steps} steps, plain and with 192 dead latents, "
                    f"sharded update on {world} ranks vs all ranks' batches computed locally",
            "ok": bool(equal) and float(flag) < 2e-3}


def run_ours(a):
    import copy

    import torch.distributed as dist

    from sparsify_b200 import ops
    from sparsify_b200.synthetic import SyntheticActivations

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    if a.gpus != world:
        print(f"bench.py: --gpus {a.gpus} but the launcher started {world} process(es); "
              f"launch with python -m torch.distributed.run --nproc-per-node {a.gpus} for {a.gpus} GPUs",
              file=sys.stderr, flush=True)
    N, D, M, k = a.tokens, a.d, a.latents, a.k
    ops.set_reserved_sms(max(a.reserve_sms, 0) if world > 1 else 0)

    parity = None
    if world > 1 and not a.no_parity:
        parity = dp_parity(dev, rank, world)
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "value": None, "unit": UNIT, "n_gpus": world,
                                  "error": "multi-rank parity check failed", "dp_parity": parity}), flush=True)
            dist.destroy_process_group()
            sys.exit(1)

    gen = SyntheticActivations(D, a.atoms, a.active, device=dev)
    wl = StepWorkload(a, gen, dev, rank, world)
    if wl.overlap:
        # the step runs on a high-priority stream; the background half of the update runs at
        # normal priority and yields the SMs to the encoder as soon as that is launched
        torch.cuda.set_stream(torch.cuda.Stream(device=dev, priority=-1))
    # the sampler starts before the warm-up so that it is already reporting when the timed
    # region begins; only samples taken after mark() are used
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler is not None:
        sampler.start()
    res = time_workload(wl, a.steps, a.warmup, sampler, with_e2e=True)
    ms, ms_e2e, clocks = res["ms"], res["ms_e2e"], res["clocks"]
    enc_ms, upd_ms = res["enc_ms"], res["upd_ms"]
    del wl
    torch.cuda.empty_cache()

    # ---- secondary workloads: a few steps each, device-timed ------------------------------
    secondary = {}
    if not a.no_secondary and not (a.transcode or a.multi_topk or a.dead_frac > 0):
        peaks = measured_peaks()
        variants = [("auxk_active", dict(dead_frac=0.05)), ("transcoder_k64_skip", dict(transcode=True, k=64)),
                    ("multi_topk", dict(multi_topk=True))]
        for name, over in variants:
            b = copy.copy(a)
            for key, val in over.items():
                setattr(b, key, val)
            # a secondary workload that fails is reported as such; the headline stands
            w2 = None
            try:
                w2 = StepWorkload(b, gen, dev, rank, world)
                r2 = time_workload(w2, 5, 3, None, with_e2e=False)
                roof = step_roofline(b, peaks, r2["ms"])
                secondary[name] = {"workload": workload_name(b), "ms_per_step": r2["ms"], "steps": 5,
                                   "tokens_per_s": world * b.tokens / (r2["ms"] * 1e-3),
                                   "step_roofline_frac_sustained": roof["frac_sustained"],
                                   "step_roofline_frac_burst": roof["frac_burst"]}
            except Exception as exc:  # noqa: BLE001
                secondary[name] = {"workload": workload_name(b), "error": f"{type(exc).__name__}: {exc}"[:300]}
            del w2
            torch.cuda.empty_cache()
    del gen
    torch.cuda.empty_cache()
    if not a.no_secondary and world > 1 and not (a.transcode or a.multi_topk or a.dead_frac > 0):
        # hookpoints sharded over the ranks, trained by Muon (distribute_modules)
        b = copy.copy(a)
        b.modules, b.latents, b.tokens, b.steps, b.warmup = 4, 65536, 8192, 3, 3
        try:
            secondary["modules_muon"] = run_modules(b, emit=False)
        except Exception as exc:  # noqa: BLE001
            secondary["modules_muon"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    if rank == 0:
        peaks = measured_peaks()
        flops = 2.0 * N * D * M
        roof = None
        if enc_ms:
            achieved = flops / (enc_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "kernel": "encode_topk_tc_kernel (+ tau init, merge)",
                    "achieved": achieved, "peak": peaks["tflops_sustained"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["tflops_sustained"],
                    "peak_kind": "sustained cuBLAS bf16 rate (the kernel is timed inside the step loop)",
                    "frac_burst": achieved / peaks["tflops_burst"], "peak_burst": peaks["tflops_burst"],
                    "peak_source": peaks["source"], "ms_per_launch": enc_ms,
                    # dram__bytes_read + write of one launch: 344.4 MB measured by ncu on the
                    # N=4096, M=32768 case, scaled by the units of this launch
                    "traffic": 344.4e6 * (N / 4096) * (M / 32768) if D == 4096 else None}
        mhz = (clocks or {}).get("sm_mhz")
        line = {
            "metric": METRIC, "value": world * N / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(a), "l2": "inputs and weights per step exceed L2 (x 134 MB, weights > 2 GB)",
                       "parallelism": f"dp{world}"},
            "e2e": {"value": world * N / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": N * D * 2,
                    "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e},
            "gpu_launches": res["launches"],
            "clocks": clocks,
            # time x clock: comparable between runs that the power cap held at different clocks
            "ms_x_ghz": None if not mhz else ms * mhz / 1e3,
            "roofline": roof,
            "update_kernel": None if upd_ms is None else {
                "kernel": "rows_adam_kernel", "ms_per_step": upd_ms, "bound": "hbm",
                # parameters, moments and bf16 copies of both matrices (26 B per element), plus the
                # gathered residual and input rows of this rank's share of the exchanged tokens
                "achieved": (2 * M * D * 26 / world + 2 * world * N * k * D * 2 / world) / (upd_ms * 1e-3) / 1e9,
                "peak": peaks["hbm"], "unit": "GB/s",
                "frac": (2 * M * D * 26 / world + 2 * world * N * k * D * 2 / world) / (upd_ms * 1e-3) / 1e9 / peaks["hbm"]},
            "step_roofline": step_roofline(a, peaks, ms),
            "last_fvu": res.get("last_fvu"),
        }
        if res["spans"]:
            line["exchange_ms_per_step"] = res["spans"]
        if parity is not None:
            line["dp_parity"] = parity
        if secondary:
            line["secondary"] = secondary
        if world == 1 and not a.no_cpu_baseline:
            base = cpu_arm(a, 2, 1, config0_steps=a.config0_steps)
            line["cpu_baseline"] = {k_: base[k_] for k_ in ("value", "unit", "cores", "kind", "sample", "config0")
                                    if k_ in base}
        if world == 1 and not a.no_gpu_reference and not (a.transcode or a.multi_topk or a.dead_frac > 0):
            torch.cuda.empty_cache()  # this process holds nothing large any more
            line["gpu_reference"] = gpu_reference_sample(a)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def modules_parity(dev, rank: int, world: int) -> dict:
    """Correctness of hookpoint sharding, checked before the timed region: every rank owns one
    small coder, receives all ranks' slices of its hookpoint through gather_to_owner and takes
    two Muon steps; the same coder trained on the concatenated slices, regenerated locally
    from their seeds, must end up identical."""
    import torch.distributed as dist

    from sparsify_b200 import SparseCoder, SparseCoderConfig, parallel
    from sparsify_b200.muon import Muon
    from sparsify_b200.optim import FusedAdam
    from sparsify_b200.synthetic import SyntheticActivations

    D, M, k, n_local, steps = 256, 2048, 16, 128, 2
    gen = SyntheticActivations(D, 4096, 16, seed=78, device=dev)
    data = lambda h, r, s: gen.batch(n_local, seed=5000 + 1000 * h + 10 * s + r, dtype=torch.bfloat16)

    def build():
        torch.manual_seed(100 + rank)
        sae = SparseCoder(D, SparseCoderConfig(num_latents=M, k=k), device=dev, dtype=torch.float32)
        muon = Muon([p for p in sae.parameters() if p.ndim >= 2], lr=2e-3, ddp=False)
        adam = FusedAdam([p for p in sae.parameters() if p.ndim < 2], lr=2e-3)
        sae.attach_optimizer(muon, project=False)
        return sae, (muon, adam)

    def train(sae, opts, x):
        sae.set_decoder_norm_to_unit_norm()
        out = sae(x)
        (out.fvu + out.auxk_loss / 32).backward()
        sae.remove_gradient_parallel_to_decoder_directions()
        for o in opts:
            o.step()
            o.zero_grad(set_to_none=True)

    sae, opts = build()
    ref, ropts = build()
    for s in range(steps):
        mine = None
        for h in range(world):  # hookpoint h is owned by rank h
            got = parallel.gather_to_owner(data(h, rank, s), h)
            if rank == h:
                mine = got
        train(sae, opts, mine)
        train(ref, ropts, torch.cat([data(rank, r, s) for r in range(world)]))
    worst = 0.0
    for p, q in zip(sae.parameters(), ref.parameters()):
        worst = max(worst, float((p.detach().double() - q.detach().double()).norm() / q.detach().double().norm()))
    flag = torch.tensor([worst], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return {"max_rel_l2": float(flag), "tolerance": 1e-5, "ok": float(flag) < 1e-5,
            "case": f"{world} hookpoints, one per rank, {n_local} tokens per rank per hookpoint, d_in={D}, {M} latents, "
                    f"k={k}, {steps} Muon steps, gathered activations vs the same slices regenerated locally"}


def run_modules(a, emit: bool = True):
    """Hookpoints sharded over ranks, no gradient exchange, Muon (sparsify/trainer.py:358-380,
    123-145): every rank holds a slice of each hookpoint's tokens, the owner gathers them,
    trains its coder, and orthogonalises its own matrices. emit=False: called from the
    headline run (process group already up); returns the figures instead of printing them."""
    import torch.distributed as dist

    from sparsify_b200 import SparseCoder, SparseCoderConfig, parallel
    from sparsify_b200.muon import Muon
    from sparsify_b200.optim import FusedAdam
    from sparsify_b200.synthetic import SyntheticActivations, batch_seed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    H, D, M, k = a.modules, a.d, a.latents, a.k
    from sparsify_b200 import ops as _ops
    _ops.set_reserved_sms(max(a.reserve_sms, 0) if world > 1 else 0)
    parity = None
    if world > 1 and not a.no_parity:
        parity = modules_parity(dev, rank, world)
        if not parity["ok"] and emit:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "value": None, "unit": UNIT, "n_gpus": world,
                                  "error": "hookpoint-sharding parity check failed", "modules_parity": parity}),
                      flush=True)
            dist.destroy_process_group()
            sys.exit(1)
    n_local = a.tokens // world
    saes = []
    for h in range(H):
        torch.manual_seed(rank * H + h)
        saes.append(SparseCoder(D, SparseCoderConfig(num_latents=M, k=k), device=dev, dtype=torch.float32))
    mats = [p for s_ in saes for p in s_.parameters() if p.ndim >= 2]
    vecs = [p for s_ in saes for p in s_.parameters() if p.ndim < 2]
    muon, adam = Muon(mats, lr=2e-3, ddp=False), FusedAdam(vecs, lr=2e-3)
    for s_ in saes:
        s_.attach_optimizer(muon, project=False)
    gen = SyntheticActivations(D, a.atoms, a.active, device=dev)
    pool = [gen.batch(n_local, batch_seed(t, rank, world, hookpoint=t), torch.bfloat16) for t in range(4)]
    del gen
    torch.cuda.empty_cache()
    with torch.no_grad():
        for s_ in saes:
            s_.b_dec.copy_(pool[0].float().mean(0))

    # as the Trainer does it: activations travel on one side stream, the owner trains on another,
    # and the stream that stands for the model's forward only records "activation ready"
    gather_stream = torch.cuda.Stream(device=dev) if world > 1 else None
    sae_stream = torch.cuda.Stream(device=dev) if world > 1 else None

    def train_one(sae, x):
        sae.set_decoder_norm_to_unit_norm()
        out = sae(x)
        (out.fvu + out.auxk_loss / 32).backward()

    def step(t):
        main = torch.cuda.current_stream(dev)
        mine = []
        for g in range(H * world):            # every hookpoint of the model, in order
            owner = g // H
            x = pool[(t + g) % len(pool)]
            if world == 1:
                train_one(saes[g % H], x)
                continue
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(sae_stream):
                sae_stream.wait_event(ready)
                x = parallel.gather_to_owner(x, owner, stream=gather_stream, after=ready)
            if rank == owner:
                mine.append((saes[g % H], x))
        if world > 1:
            # as the Trainer does: owners train once the model's forward (here: the loop that
            # hands out the slices) is over, so nobody's slices wait behind a training call
            with torch.cuda.stream(sae_stream):
                for sae, x in mine:
                    train_one(sae, x)
        if world > 1:
            main.wait_stream(sae_stream)
        for sae in saes:
            sae.remove_gradient_parallel_to_decoder_directions()
        for opt in (muon, adam):
            opt.step()
            opt.zero_grad(set_to_none=True)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0 and emit:
        sampler.start()
    for t in range(max(a.warmup, 3)):
        step(t)
    sync()
    counter = LaunchCounter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark()
    e0.record()
    for t in range(a.steps):
        step(t)
    e1.record()
    sync()
    clocks = sampler.stop() if rank == 0 and emit else None
    _ops.check_status(dev)
    counter.close()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    peaks = measured_peaks()
    ns_flops = 2 * H * 5 * (2 * D * D * M * 2 + 2 * D * D * D)   # per rank, as a library computes them
    enc_flops = 2.0 * H * a.tokens * D * M
    if not emit:
        del saes, muon, adam, mats, vecs, pool
        torch.cuda.empty_cache()
        return {"workload": f"{H * world} hookpoints of width {D} sharded over {world} ranks ({H} per rank), {M} "
                            f"latents, k={k}, {a.tokens} tokens per hookpoint per step, Muon + Adam on the biases",
                "ms_per_step": ms, "steps": a.steps, "tokens_per_s": H * world * a.tokens / (ms * 1e-3),
                "whole_step_tflops": (ns_flops + enc_flops) / (ms * 1e-3) / 1e12,
                "frac_of_sustained_tensor_peak": (ns_flops + enc_flops) / (ms * 1e-3) / 1e12 / peaks["tflops_sustained"],
                "modules_parity": parity}
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": H * world * a.tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{H * world} hookpoints of width {D} sharded over {world} rank(s) "
                                   f"({H} per rank, distribute_modules), {M} latents, k={k}, {a.tokens} tokens per "
                                   f"hookpoint per step, Muon (5 Newton-Schulz steps on W_enc and W_dec) + Adam on "
                                   f"the biases, bf16 operands", "parallelism": f"modules{world}"},
            "gpu_launches": counter.n, "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel + encode_topk_tc_kernel",
                         "achieved": (ns_flops + enc_flops) / (ms * 1e-3) / 1e12, "peak": peaks["tflops_sustained"],
                         "unit": "TFLOP/s",
                         "frac": (ns_flops + enc_flops) / (ms * 1e-3) / 1e12 / peaks["tflops_sustained"],
                         "peak_source": peaks["source"], "traffic": None,
                         "note": "whole step; FLOPs counted as a library computes Newton-Schulz (no symmetry)"},
            "modules_parity": parity,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_kernel(a):
    """Times single entry points in isolation (CUDA events on the launching
    stream, 2 warm-up + 5 timed launches) and prints one JSON line per kernel."""
    from sparsify_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    N, D, M, k = a.tokens, a.d, a.latents, a.k
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(N, D, device=dev, generator=g).bfloat16()
    W = (torch.randn(M, D, device=dev, generator=g) / D ** 0.5).bfloat16()
    b = 0.1 * torch.randn(M, device=dev, generator=g)
    peaks = measured_peaks()

    def timed(fn, reps=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    which = a.kernel
    results = []
    if which in ("ns", "gemm"):
        # Muon's Newton-Schulz on one [latents, d] matrix, and its three products
        from sparsify_b200.muon import quintic_newtonschulz
        del x
        G = torch.randn(M, D, device=dev, generator=g)
        if which == "ns":
            ms = timed(lambda: quintic_newtonschulz(G, 5), reps=3)
            flops = 5 * (2 * D * D * M * 2 + 2 * D * D * D)  # as a library computes it, no symmetry
            results.append(dict(kernel="newtonschulz5", ms=ms, tflops_equiv=flops / ms / 1e9,
                                frac=flops / ms / 1e9 / peaks["tflops_sustained"]))
        else:
            Wd = W.T.contiguous()                               # wide [D, M]
            A = ops.gemm_nt(Wd, Wd)
            for name, fn, fl in (
                ("gemm_XXt", lambda: ops.gemm_nt(Wd, Wd), 2 * D * D * M),
                ("gemm_XXt_symmetric", lambda: ops.gemm_nt(Wd, Wd, symmetric=True), 2 * D * D * M),
                ("gemm_AA_symmetric", lambda: ops.gemm_nt(A, A, alpha=2.0, beta=-4.0, Cin=A, symmetric=True), 2 * D * D * D),
                ("gemm_TB", lambda: ops.gemm_nt(W, A, beta=3.0, Cin=W), 2 * D * D * M),
                ("gemm_TB_out_t", lambda: ops.gemm_nt(W, A, beta=3.0, Cin=W, out_t=Wd), 2 * D * D * M),
            ):
                ms = timed(fn)
                results.append(dict(kernel=name, ms=ms, tflops_equiv=fl / ms / 1e9, frac=fl / ms / 1e9 / peaks["tflops_sustained"]))
        for r in results:
            r.update(D=D, M=M)
            print(json.dumps(r), flush=True)
        return
    vals, idx = ops.encode_topk_tc(x, W, b, k)
    if which in ("encode", "all"):
        ms = timed(lambda: ops.encode_topk_tc(x, W, b, k))
        tf = 2.0 * N * D * M / (ms * 1e-3) / 1e12
        results.append(dict(kernel="encode_topk", ms=ms, tflops=tf, frac=tf / peaks["tflops_sustained"]))
    gout = torch.randn(N, D, device=dev, generator=g)
    if which in ("decode", "all"):
        ms = timed(lambda: ops.embedding_bag_fwd(idx, vals, W, None))
        nbytes = N * k * D * 2 + N * k * 12 + N * D * 4
        results.append(dict(kernel="embedding_bag_fwd", ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / peaks["hbm"]))
    if which in ("decode", "all"):
        yb = gout.bfloat16()
        ms = timed(lambda: ops.decode_residual(idx, vals, W, None, yb, want_e16=True))
        nbytes = N * k * D * 2 + N * k * 12 + N * D * (2 + 4 + 2)
        results.append(dict(kernel="decode_residual", ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / peaks["hbm"]))
    if which in ("decode", "all") and ops.decode_dots_supported(W, k):
        yb = gout.bfloat16()
        ms = timed(lambda: ops.decode_residual(idx, vals, W, None, yb, want_out=False, want_e16=True, want_dots=True))
        nbytes = N * k * D * 2 + N * k * 16 + N * D * (2 + 2)
        results.append(dict(kernel="decode_residual_dots", ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / peaks["hbm"]))
        ms = timed(lambda: ops.decode_residual(idx, vals, W, None, yb, want_out=False, want_e16=True))
        results.append(dict(kernel="decode_residual (no out)", ms=ms))
        e16 = ops.decode_residual(idx, vals, W, None, yb, want_out=False, want_e16=True)[2]
        ms = timed(lambda: ops.embedding_bag_bwd_acts(idx, e16, W))
        results.append(dict(kernel="embedding_bag_bwd_acts (bf16 gradient)", ms=ms))
    if which in ("bwd_acts", "all"):
        ms = timed(lambda: ops.embedding_bag_bwd_acts(idx, gout, W))
        nbytes = N * k * D * 2 + N * D * 4 + N * k * 12
        results.append(dict(kernel="embedding_bag_bwd_acts", ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / peaks["hbm"]))
    if which in ("csr", "rows", "all"):
        ms = timed(lambda: ops.csr_build(idx, M))
        results.append(dict(kernel="csr_build", ms=ms))
        row_ptr, entries = ops.csr_build(idx, M)
        out = {}
        gacts = torch.randn(N, k, device=dev, generator=g)
        def rows():
            nonlocal out
            out = ops.rows_accumulate(row_ptr, entries, k, M, D, vals, gout, coefB=gacts, vecB=x,
                                      biasB=True, out=out)
        ms = timed(rows)
        nbytes = 2 * M * D * 4 + N * D * 4 + N * D * 2 + N * k * 12
        results.append(dict(kernel="rows_accumulate", ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / peaks["hbm"]))
        del out
    if which in ("topk_mask", "all"):
        # the AuxK selection: the 2048 largest of 6560 post-ReLU pre-activations per token, written back densely
        nd, k_aux = 6560, 2048
        P = torch.relu(torch.randn(N, nd, device=dev, generator=g))
        ms = timed(lambda: ops.topk_mask_rows(P, k_aux))
        nbytes = N * nd * 6
        results.append(dict(kernel="topk_mask_rows", ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / peaks["hbm"]))
        del P
    if which in ("rows_adam", "all"):
        # the fused sparse update of both matrices, as the training step launches it (one launch per matrix)
        row_ptr, entries = ops.csr_build(idx, M)
        gacts = torch.randn(N, k, device=dev, generator=g)
        e16 = gout.bfloat16()
        mats = [[torch.randn(M, D, device=dev, generator=g) / D ** 0.5, torch.zeros(M, D, device=dev),
                 torch.zeros(M, D, device=dev), torch.empty(M, D, device=dev, dtype=torch.bfloat16)] for _ in range(2)]
        hp = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, step=3)
        kw = dict(pA=mats[0][0], mA=mats[0][1], vA=mats[0][2], shadowA=mats[0][3], projectA=True, normalizeA=True,
                  norm_eps=1.2e-7, hpA=hp, pB=mats[1][0], mB=mats[1][1], vB=mats[1][2], shadowB=mats[1][3], hpB=hp)
        for name, parts in (("rows_adam_encoder", 2), ("rows_adam_decoder", 1)):
            ms = timed(lambda: ops.rows_adam_(row_ptr, entries, k, vals, e16, gacts, x, parts=parts, **kw))
            nbytes = M * D * 26 + N * k * D * 2 + N * k * 8
            results.append(dict(kernel=name, ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / peaks["hbm"]))
        del mats, kw
    if which in ("adam", "normalize", "all"):
        p = torch.randn(M, D, device=dev, generator=g)
        gr, m, v = torch.randn_like(p), torch.zeros_like(p), torch.zeros_like(p)
        sh = torch.empty(M, D, device=dev, dtype=torch.bfloat16)
        kw = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, step=3)
        ms = timed(lambda: ops.adam_rows_(p, gr, m, v, project=False, shadow=sh, **kw))
        results.append(dict(kernel="adam_flat", ms=ms, gbs=M * D * 30 / ms / 1e6, frac=M * D * 30 / ms / 1e6 / peaks["hbm"]))
        ms = timed(lambda: ops.adam_rows_(p, gr, m, v, project=True, shadow=sh, **kw))
        results.append(dict(kernel="adam_rows_project", ms=ms, gbs=M * D * 34 / ms / 1e6, frac=M * D * 34 / ms / 1e6 / peaks["hbm"]))
        ms = timed(lambda: ops.normalize_rows_(p, 1e-7, sh))
        results.append(dict(kernel="normalize_rows", ms=ms, gbs=M * D * 10 / ms / 1e6, frac=M * D * 10 / ms / 1e6 / peaks["hbm"]))
    for r in results:
        r.update(N=N, D=D, M=M, k=k)
        print(json.dumps(r), flush=True)


if __name__ == "__main__":
    args = parse_args()
    if args.impl == "ours" and args.cta_pairs >= 0:
        from sparsify_b200 import ops as _ops_cfg
        _ops_cfg.set_cta_pairs(bool(args.cta_pairs))
    if args.kernel:
        run_kernel(args)
    elif args.modules:
        run_modules(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    else:
        run_ours(args)
